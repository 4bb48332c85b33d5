"""Plain, slow MiniMax M2 forward pass: whole sequences, no cache, one function per part.

Written from the formulas of CURRENTF/SparseEngine's own files (each function cites
file:line inside that project). It shares no code with ``sparseengine_b200``: it
reads the raw ``config.json`` dictionary and a ``{tensor name: tensor}`` mapping.

``act`` is the activation dtype. With ``torch.float32`` every rounding point is
an identity; with ``torch.bfloat16`` values are rounded to bfloat16 exactly where
the reference rounds them (projection outputs, the residual stream, the QK-norm
result before its weight multiply, P before P·V, gate/up before SiLU, logits),
while statistics, softmax, rotation, the router and all accumulations stay in
32-bit.  All arithmetic runs on the CPU in float32 tensors.

SparseEngine's whole M2 model cannot be built on a CPU (its norm, router and expert
providers need CUDA + Triton), so this file rests on the formulas; the attention
front end (QKV split, whole-projection QK norm, partial rotary) is compared once with
SparseEngine's own CPU code in ``tests/golden/``.
"""
from __future__ import annotations

import math

import torch


def _round(x: torch.Tensor, act: torch.dtype) -> torch.Tensor:
    """Round a float32 tensor to ``act`` and bring it back to float32."""
    if act == torch.float32:
        return x
    return x.to(act).to(torch.float32)


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """h0 = embed_tokens.weight[input_ids]  (src/sparseengine/layers/embed_head.py:54-61)."""
    return table[ids.long()].to(torch.float32)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, act: torch.dtype) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, all in 32-bit, then cast.

    src/sparseengine/kernels/triton/rmsnorm.py:56-61 (variance, normalized, output);
    src/sparseengine/layers/layernorm.py:120-159.
    """
    x = x.to(torch.float32)
    var = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return _round(x * torch.rsqrt(var + eps) * w.to(torch.float32), act)


def add_rms_norm(x, residual, w, eps, act):
    """Fused residual add + norm: the unrounded 32-bit sum is normalised, the
    rounded sum becomes the new residual (src/sparseengine/kernels/triton/rmsnorm.py:43-54)."""
    s = x.to(torch.float32) + residual.to(torch.float32)
    var = (s * s).sum(-1, keepdim=True) / s.shape[-1]
    y = _round(s * torch.rsqrt(var + eps) * w.to(torch.float32), act)
    return y, _round(s, act)


def linear(x: torch.Tensor, w: torch.Tensor, act: torch.dtype) -> torch.Tensor:
    """y = x · Wᵀ with a 32-bit accumulator, rounded to act, no bias
    (src/sparseengine/layers/linear.py:174-191)."""
    return _round(x.to(torch.float32) @ w.to(torch.float32).t(), act)


def whole_projection_rms_norm(x, w, eps, act):
    """QK norm over the whole flat projection (not per head):
    inv = rsqrt(sum(x^2)/N + eps); y = cast(x32 * inv) * cast(w), the product in act.

    src/sparseengine/layers/layernorm.py:204-210 (_apply_global_rms), :217-255.
    """
    x = x.to(torch.float32)
    n = x.shape[-1]
    inv = torch.rsqrt((x * x).sum(-1) / n + eps)
    normed = _round(x * inv.unsqueeze(-1), act)
    return _round(normed * _round(w.to(torch.float32), act), act)


def rope_inv_freq(rotary_dim: int, theta: float) -> torch.Tensor:
    """inv_freq_j = 1 / theta^(2j/R)  (src/sparseengine/layers/rotary_embedding.py:15-24)."""
    return 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))


def rope_scaling_of(cfg: dict):
    """The configuration's frequency scaling: ``rope_parameters`` if present, else
    ``rope_scaling``; no type or "default" means none (src/sparseengine/models/rope.py:14-35)."""
    params = dict(cfg.get("rope_parameters") or cfg.get("rope_scaling") or {})
    kind = str(params.get("rope_type", params.get("type", "default")) or "default").lower()
    return None if kind == "default" else dict(params, rope_type=kind)


def rope_frequencies(rotary_dim: int, theta: float, scaling: dict | None):
    """(inv_freq, factor on cos and sin) for the scaled rotary encodings
    (src/sparseengine/layers/rotary_embedding.py:26-101): linear :34-35, llama3 :36-59, yarn :60-100
    with the amplitude 0.1·m·ln(factor)+1 of :8-12."""
    inv = rope_inv_freq(rotary_dim, theta)
    if scaling is None:
        return inv, 1.0
    kind, factor = scaling["rope_type"], float(scaling["factor"])
    if kind == "linear":
        return inv / factor, 1.0
    old = float(scaling["original_max_position_embeddings"])
    if kind == "llama3":
        lo, hi = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        out = []
        for f in inv.tolist():
            wavelen = 2 * math.pi / f
            if wavelen > old / lo:
                out.append(f / factor)
            elif wavelen < old / hi:
                out.append(f)
            else:
                smooth = (old / wavelen - lo) / (hi - lo)
                out.append((1 - smooth) * f / factor + smooth * f)
        return torch.tensor(out, dtype=torch.float32), 1.0
    assert kind == "yarn", kind
    beta_fast, beta_slow = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))

    def correction_dim(rotations):
        return rotary_dim * math.log(old / (rotations * 2 * math.pi)) / (2 * math.log(theta))

    low, high = correction_dim(beta_fast), correction_dim(beta_slow)
    if scaling.get("truncate", True):
        low, high = math.floor(low), math.ceil(high)
    low, high = max(low, 0), min(high, rotary_dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(rotary_dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
    inv = inv / factor * ramp + inv * (1 - ramp)

    def mscale(mult=1.0):
        return 1.0 if factor <= 1.0 else 0.1 * mult * math.log(factor) + 1.0

    att = scaling.get("attention_factor")
    if att is None:
        m, m_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
        att = mscale(float(m)) / mscale(float(m_all)) if m and m_all else mscale()
    return inv, float(att)


def partial_rotary(x, positions, rotary_dim, theta, act, scaling=None, interleaved=False):
    """Rotate the first ``rotary_dim`` dims of each head (split-half pairing), pass the
    rest through untouched.  x: [T, heads, D].  cos and sin carry the scaled encodings'
    factor (src/sparseengine/layers/rotary_embedding.py:208-212).  ``interleaved``: pair i is
    the adjacent dims (2i, 2i+1) and the results are written as split halves (:115-127).

    src/sparseengine/layers/rotary_embedding.py:104-112 (apply_rotary_emb),
    :129-167 (apply_partial_rotary_emb); cos/sin cache :190-222.
    """
    inv, factor = rope_frequencies(rotary_dim, theta, scaling)
    ang = positions.to(torch.float32).unsqueeze(-1) * inv.to(positions.device)  # [T, R/2]
    cos = (torch.cos(ang) * factor).unsqueeze(1)
    sin = (torch.sin(ang) * factor).unsqueeze(1)
    x = x.to(torch.float32)
    rot, rest = x[..., :rotary_dim], x[..., rotary_dim:]
    if interleaved:
        x1, x2 = rot[..., 0::2], rot[..., 1::2]
    else:
        x1, x2 = rot[..., : rotary_dim // 2], rot[..., rotary_dim // 2:]
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat((_round(y1, act), _round(y2, act), rest), dim=-1)


def causal_attention(q, k, v, act, window: int | None = None):
    """GQA causal attention over a whole sequence.  q [T,Hq,D], k,v [T,Hkv,D].

    score = q·k · D^-0.5; query p sees keys 0..p; 32-bit softmax; P rounded to act
    before P·V; output rounded.  Query head h reads KV head h // (Hq/Hkv).
    src/sparseengine/models/minimax_m2.py:324-332;
    src/sparseengine/kernels/triton/context_flashattention_nopad.py:92-127.
    ``window`` (keys p-window+1..p) is not used by M2; it serves tests of the part.
    """
    t, hq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    scale = d ** -0.5
    out = torch.empty(t, hq, d, dtype=torch.float32, device=q.device)
    pos = torch.arange(t, device=q.device)
    mask = pos[None, :] <= pos[:, None]
    if window is not None:
        mask &= pos[None, :] > pos[:, None] - window
    for h in range(hq):
        kh = k[:, h // group].to(torch.float32)
        vh = v[:, h // group].to(torch.float32)
        s = (q[:, h].to(torch.float32) @ kh.t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        m = s.max(-1, keepdim=True).values
        e = torch.exp(s - m)
        denom = e.sum(-1, keepdim=True)
        p = _round(e, act)  # flash kernels round the unnormalised P tile
        out[:, h] = (p @ vh) / denom
    return _round(out, act)


def router(x, gate_w, bias, top_k):
    """Sigmoid router with a selection bias, 32-bit throughout.

    logits = float(x)·Wgᵀ; p = sigmoid(logits); score = p + bias (NaN → +inf);
    pick top-k by score; returned order: entries strictly above the k-th value in
    ascending expert index, then ties with it in ascending index; weights are the
    unbiased p renormalised over the selection (epsilon 0).
    src/sparseengine/models/minimax_m2.py:140-172;
    src/sparseengine/kernels/triton/moe_biased_sigmoid.py:71-111,202-238;
    src/sparseengine/kernels/triton/minimax_m2_router.py:50-63.
    """
    logits = x.to(torch.float32) @ gate_w.to(torch.float32).t()
    p = torch.sigmoid(logits)
    score = p + bias.to(torch.float32)
    score = torch.where(torch.isnan(score), torch.full_like(score, float("inf")), score)
    t, e = score.shape
    thr = torch.topk(score, top_k, dim=-1).values.min(-1, keepdim=True).values      # the k-th value
    index = torch.arange(e, device=score.device).expand(t, e)
    # sort key: strictly greater entries by ascending index, then ties by ascending index, then the rest
    key = torch.where(score > thr, index, torch.where(score == thr, index + e, index + 2 * e))
    ids = torch.sort(key, dim=-1).values[:, :top_k] % e
    w = p.gather(1, ids)
    w = w / w.sum(-1, keepdim=True)
    return ids, w, logits


def experts(x, ids, weights, w1, w3, w2, act):
    """SwiGLU experts, combined in router slot order.

    g = cast(x·W1ᵀ), u = cast(x·W3ᵀ); a = cast(silu32(g)) * u (in act);
    d = cast((a·W2ᵀ)_32 · w_e); out = cast(Σ_slots d) accumulated in 32-bit.
    src/sparseengine/layers/packed_moe.py:138-155;
    src/sparseengine/kernels/triton/moe.py:557-563,726-732,1128-1157,1374-1440;
    src/sparseengine/kernels/triton/silu_and_mul.py:41-60.
    w1/w3: [E, I, H], w2: [E, H, I].
    """
    t, k = ids.shape
    out = torch.zeros(t, w2.shape[1], dtype=torch.float32, device=x.device)
    x = x.to(torch.float32)
    for slot in range(k):                       # slot order: token i adds its slot-0 expert first, then slot 1, ...
        col = ids[:, slot]
        for e in torch.unique(col).tolist():    # the tokens that chose expert e in this slot, as one product
            rows = (col == e).nonzero().squeeze(-1)
            xi = x[rows]
            g = _round(xi @ w1[e].to(torch.float32).t(), act)
            u = _round(xi @ w3[e].to(torch.float32).t(), act)
            a = _round(_round(g / (1.0 + torch.exp(-g)), act) * u, act)
            d = a @ w2[e].to(torch.float32).t()
            out[rows] += _round(d * weights[rows, slot].unsqueeze(-1), act)
    return _round(out, act)


def sampling_kept(row: torch.Tensor, top_k: int, top_p: float, temperature: float) -> torch.Tensor:
    """Which tokens of one row of logits survive the sampler's cuts (a bool mask).

    Sorted by logit / temperature, descending; top-k keeps the first k (0 = all); softmax over
    those; top-p then drops an entry if the mass *before* it already exceeds top_p (so the
    first entry always stays) (src/sparseengine/layers/sampler.py:101-118)."""
    scaled = row.to(torch.float32) / temperature
    order = torch.argsort(scaled, descending=True, stable=True)
    keep = len(order) if top_k <= 0 else min(top_k, len(order))
    s = scaled[order].clone()
    s[keep:] = float("-inf")
    p = torch.softmax(s, -1)
    before = torch.cumsum(p, 0) - p
    drop = torch.cumsum(p, 0) > top_p
    drop = torch.cat((torch.tensor([False]), drop[:-1]))
    mask = torch.zeros(len(order), dtype=torch.bool)
    mask[order[:keep][~drop[:keep]]] = True
    return mask


def _layer_tensors(tensors, i, cfg):
    p = f"model.layers.{i}."
    e = int(cfg["num_local_experts"])
    moe = p + "block_sparse_moe."
    return {
        "ln1": tensors[p + "input_layernorm.weight"],
        "ln2": tensors[p + "post_attention_layernorm.weight"],
        "wq": tensors[p + "self_attn.q_proj.weight"],
        "wk": tensors[p + "self_attn.k_proj.weight"],
        "wv": tensors[p + "self_attn.v_proj.weight"],
        "wo": tensors[p + "self_attn.o_proj.weight"],
        "qn": tensors[p + "self_attn.q_norm.weight"],
        "kn": tensors[p + "self_attn.k_norm.weight"],
        "gate": tensors[moe + "gate.weight"],
        "bias": tensors[moe + "e_score_correction_bias"],
        # the experts' matrices stacked [E, ...]; a caller with many large experts may give the stacks
        # themselves under "<moe>experts.stacked.w1" (w3, w2) to save the copies
        **{w: (tensors[f"{moe}experts.stacked.{w}"] if f"{moe}experts.stacked.{w}" in tensors else
               torch.stack([tensors[f"{moe}experts.{j}.{w}.weight"] for j in range(e)])) for w in ("w1", "w3", "w2")},
    }


def attention_block(x, lt, cfg, positions, act):
    """QKV projection → whole-projection QK norm → partial rotary → causal GQA → o_proj
    (src/sparseengine/models/minimax_m2.py:334-359)."""
    hq = int(cfg["num_attention_heads"])
    hkv = int(cfg["num_key_value_heads"])
    d = int(cfg["head_dim"])
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    rot = int(cfg["rotary_dim"])
    theta = float(cfg.get("rope_theta", 10000.0))
    t = x.shape[0]
    q = linear(x, lt["wq"], act)
    k = linear(x, lt["wk"], act)
    v = linear(x, lt["wv"], act)
    q = whole_projection_rms_norm(q, lt["qn"], eps, act).view(t, hq, d)
    k = whole_projection_rms_norm(k, lt["kn"], eps, act).view(t, hkv, d)
    v = v.view(t, hkv, d)
    scaling = rope_scaling_of(cfg)
    q = partial_rotary(q, positions, rot, theta, act, scaling)
    k = partial_rotary(k, positions, rot, theta, act, scaling)
    o = causal_attention(q, k, v, act)
    return linear(o.reshape(t, hq * d), lt["wo"], act), (q, k, v)


def moe_block(x, lt, cfg, act, forced_ids=None, info=None):
    """Router then experts (src/sparseengine/models/minimax_m2.py:244-269).

    ``forced_ids`` [T, k] replaces the router's own choice of experts (the weights are
    still this router's unbiased scores of those experts, renormalised): a test uses it
    to follow an engine through a near-tie, where rounding may pick either expert.
    ``info`` (a dict) receives this router's own ids and, per token, the gap between its
    k-th and (k+1)-th selection scores."""
    k = int(cfg["num_experts_per_tok"])
    ids, w, logits = router(x, lt["gate"], lt["bias"], k)
    if info is not None:
        score = torch.sigmoid(logits) + lt["bias"].to(torch.float32)
        srt = score.sort(-1, descending=True).values
        info.setdefault("ids", []).append(ids)
        info.setdefault("margin", []).append(srt[:, k - 1] - srt[:, k] if srt.shape[1] > k
                                             else torch.full((x.shape[0],), float("inf"), device=x.device))
    if forced_ids is not None:
        ids = forced_ids.long()
        p = torch.sigmoid(logits).gather(1, ids)
        w = p / p.sum(-1, keepdim=True)
    return experts(x, ids, w, lt["w1"], lt["w3"], lt["w2"], act)


def forward(cfg: dict, tensors: dict, token_ids, act: torch.dtype = torch.float32, forced_ids=None,
            info=None, want=None) -> torch.Tensor:
    """Logits [T, V] (float32) at every position of one whole sequence (``want``: only at these
    positions, [len(want), V]; the final norm and the head are per position).  Runs where the
    tensors live.

    ``forced_ids``: optional list (one entry per layer) of expert ids [T, k] to use
    instead of the router's own; ``info``: optional dict that receives the routers' own
    ids and score gaps per layer (see :func:`moe_block`).

    Pre-norm residual convention of src/sparseengine/models/minimax_m2.py:381-397 and
    src/sparseengine/models/qwen3.py:291-328: the residual stream is rounded to act
    after each add, the norm reads the unrounded sum.
    """
    device = tensors["model.embed_tokens.weight"].device
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=device)
    t = ids.shape[0]
    positions = torch.arange(t, device=device)
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    tensors = {n: v.to(torch.float32) if v.dtype == torch.float32 else _round(v.to(torch.float32), act)
               for n, v in tensors.items()}
    hidden = _round(embedding(tensors["model.embed_tokens.weight"], ids), act)
    residual = None
    for i in range(int(cfg["num_hidden_layers"])):
        lt = _layer_tensors(tensors, i, cfg)
        if residual is None:
            residual = hidden
            x = rms_norm(hidden, lt["ln1"], eps, act)
        else:
            x, residual = add_rms_norm(hidden, residual, lt["ln1"], eps, act)
        hidden, _ = attention_block(x, lt, cfg, positions, act)
        x, residual = add_rms_norm(hidden, residual, lt["ln2"], eps, act)
        hidden = moe_block(x, lt, cfg, act, None if forced_ids is None else forced_ids[i], info)
    if want is not None:
        rows = torch.as_tensor(want, dtype=torch.long, device=device)
        hidden, residual = hidden[rows], residual[rows]
    x, _ = add_rms_norm(hidden, residual, tensors["model.norm.weight"], eps, act)
    return linear(x, tensors["lm_head.weight"], act)


def random_tensors(cfg: dict, seed: int, std: float = 0.02, norm_std: float = 0.0,
                   bias_std: float = 0.0) -> dict:
    """Seeded random weights under the checkpoint's tensor names (float32).

    Matrices N(0, std); norm weights 1 + N(0, norm_std); the router's selection bias
    N(0, bias_std).  Names: src/sparseengine/models/minimax_m2.py:54-61,419-423,513-530.
    """
    g = torch.Generator().manual_seed(seed)
    h = int(cfg["hidden_size"]); v = int(cfg["vocab_size"]); d = int(cfg["head_dim"])
    hq = int(cfg["num_attention_heads"]); hkv = int(cfg["num_key_value_heads"])
    e = int(cfg["num_local_experts"]); inter = int(cfg["intermediate_size"])

    def mat(*shape):
        return torch.randn(*shape, generator=g) * std

    def norm(n):
        return 1.0 + torch.randn(n, generator=g) * norm_std

    out = {"model.embed_tokens.weight": mat(v, h)}
    for i in range(int(cfg["num_hidden_layers"])):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = norm(h)
        out[p + "post_attention_layernorm.weight"] = norm(h)
        out[p + "self_attn.q_proj.weight"] = mat(hq * d, h)
        out[p + "self_attn.k_proj.weight"] = mat(hkv * d, h)
        out[p + "self_attn.v_proj.weight"] = mat(hkv * d, h)
        out[p + "self_attn.o_proj.weight"] = mat(h, hq * d)
        out[p + "self_attn.q_norm.weight"] = norm(hq * d)
        out[p + "self_attn.k_norm.weight"] = norm(hkv * d)
        out[p + "block_sparse_moe.gate.weight"] = mat(e, h)
        out[p + "block_sparse_moe.e_score_correction_bias"] = torch.randn(e, generator=g) * bias_std
        for j in range(e):
            q = f"{p}block_sparse_moe.experts.{j}."
            out[q + "w1.weight"] = mat(inter, h)
            out[q + "w2.weight"] = mat(h, inter)
            out[q + "w3.weight"] = mat(inter, h)
    out["model.norm.weight"] = norm(h)
    out["lm_head.weight"] = mat(v, h)
    return out


TINY_A = {
    "architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "rotary_dim": 8, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "num_local_experts": 4, "num_experts_per_tok": 2, "intermediate_size": 32,
    "vocab_size": 256, "max_position_embeddings": 512, "tie_word_embeddings": False,
    "hidden_act": "silu", "qk_norm_type": "per_layer", "use_qk_norm": True,
    "scoring_func": "sigmoid", "use_routing_bias": True, "use_mtp": True,
    "shared_intermediate_size": 0, "torch_dtype": "float32",
}

TINY_B = {
    "architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 32, "rotary_dim": 32, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "num_local_experts": 8, "num_experts_per_tok": 3, "intermediate_size": 48,
    "vocab_size": 384, "max_position_embeddings": 1024, "tie_word_embeddings": False,
    "hidden_act": "silu", "qk_norm_type": "per_layer", "use_qk_norm": True,
    "scoring_func": "sigmoid", "use_routing_bias": True, "use_mtp": True,
    "shared_intermediate_size": 0, "torch_dtype": "float32",
}

# A third shape with sizes that are no powers of two: 5 query heads on 1 KV head,
# head size 48 with 16 rotated dims, width 80, 6 experts top-4, vocabulary 203.
TINY_C = {
    "architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2",
    "num_hidden_layers": 1, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 1,
    "head_dim": 48, "rotary_dim": 16, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "num_local_experts": 6, "num_experts_per_tok": 4, "intermediate_size": 40,
    "vocab_size": 203, "max_position_embeddings": 2048, "tie_word_embeddings": False,
    "hidden_act": "silu", "qk_norm_type": "per_layer", "use_qk_norm": True,
    "scoring_func": "sigmoid", "use_routing_bias": True, "use_mtp": True,
    "shared_intermediate_size": 0, "torch_dtype": "float32",
}

# Head sizes 128 and 64, which the engine's tensor-core attention kernels take (the shapes
# above all go through its plain attention kernel): 6 query heads on 2 KV heads of 128 with
# half of the dims rotated, as MiniMax M2 has them; and 4 on 4 heads of 64, fully rotated.
TINY_D = {
    "architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2",
    "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 128, "rotary_dim": 64, "rope_theta": 5000000.0, "rms_norm_eps": 1e-6,
    "num_local_experts": 8, "num_experts_per_tok": 2, "intermediate_size": 64,
    "vocab_size": 320, "max_position_embeddings": 4096, "tie_word_embeddings": False,
    "hidden_act": "silu", "qk_norm_type": "per_layer", "use_qk_norm": True,
    "scoring_func": "sigmoid", "use_routing_bias": True, "use_mtp": True,
    "shared_intermediate_size": 0, "torch_dtype": "float32",
}

TINY_E = {
    "architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2",
    "num_hidden_layers": 1, "hidden_size": 192, "num_attention_heads": 4, "num_key_value_heads": 4,
    "head_dim": 64, "rotary_dim": 64, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
    "num_local_experts": 5, "num_experts_per_tok": 3, "intermediate_size": 96,
    "vocab_size": 150, "max_position_embeddings": 4096, "tie_word_embeddings": False,
    "hidden_act": "silu", "qk_norm_type": "per_layer", "use_qk_norm": True,
    "scoring_func": "sigmoid", "use_routing_bias": True, "use_mtp": True,
    "shared_intermediate_size": 0, "torch_dtype": "float32",
}
