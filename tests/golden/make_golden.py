"""Golden outputs from CURRENTF/SparseEngine's own CPU code for the parts of MiniMax M2
that can run without CUDA: the whole-projection QK RMSNorm pair
(src/sparseengine/layers/layernorm.py:217-255), the partial rotary encoding
(src/sparseengine/layers/rotary_embedding.py:129-167 with the torch backend) and the
greedy branch of the sampler (src/sparseengine/layers/sampler.py:123-135).

The reference's RMSNorm, router and expert *kernels* need CUDA + Triton and its whole model
cannot be built on a CPU.  For those parts the reference ships pure-torch oracles in its own
test files, which do run on a CPU and are imported from the checkout here:
``_rmsnorm_reference`` (tests/test_minimax_m2_model.py:45-56), ``_reference`` of the M2 router
at its 256 experts / top-8 (tests/test_minimax_m2_router.py:16-25), ``_oracle_local_moe``
(tests/test_triton_moe.py:76-98); ``Sampler._sample`` is torch only
(src/sparseengine/layers/sampler.py:66-122) and gives, over many draws, the set of tokens that
survive its top-k / top-p cuts; ``_compute_rope_parameters``
(src/sparseengine/layers/rotary_embedding.py:15-101) gives the scaled frequency tables and
``apply_interleaved_rotary_emb`` (:115-127) the adjacent-pairs rotation.

Run once, with the reference checkout importable:

    PYTHONPATH=<reference>/src:<reference>/tests SPARSEENGINE_PLATFORM=cpu CUDA_VISIBLE_DEVICES="" \
        python tests/golden/make_golden.py

It writes tests/golden/m2_front_end.safetensors and tests/golden/m2_oracles.safetensors (inputs
and outputs, float32, some tens of KB), which tests/test_plain.py compares with the plain
implementation.
"""
import os
import sys

import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
import plain_m2  # noqa: E402
from golden_cases import ROPE_SCALINGS, SAMPLER_CASES  # noqa: E402

from sparseengine.distributed import ParallelContext, ParallelGroup  # noqa: E402
from sparseengine.layers.layernorm import ColumnParallelRMSNorm  # noqa: E402
from sparseengine.layers.rotary_embedding import apply_partial_rotary_emb, apply_rotary_emb, get_rope  # noqa: E402
from sparseengine.layers.sampler import Sampler  # noqa: E402


def context():
    g = ParallelGroup(None, (0,), 0, 1)
    return ParallelContext(world=g, moe_tp=g, attn_tp=g, moe_ep=g, attn_dp=g)


def main():
    out = {}
    ctx = context()
    for name, cfg in (("A", plain_m2.TINY_A), ("B", plain_m2.TINY_B), ("C", plain_m2.TINY_C)):
        torch.manual_seed(11)
        hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        rot, theta, eps = cfg["rotary_dim"], cfg["rope_theta"], cfg["rms_norm_eps"]
        t = 7
        q = torch.randn(t, hq * d) * 3.0
        k = torch.randn(t, hkv * d) * 0.3
        qw = 1.0 + 0.1 * torch.randn(hq * d)
        kw = 1.0 + 0.1 * torch.randn(hkv * d)
        positions = torch.tensor([0, 1, 2, 5, 17, 100, 411])
        qn = ColumnParallelRMSNorm(hq * d, eps=eps, parallel_context=ctx)
        kn = ColumnParallelRMSNorm(hkv * d, eps=eps, parallel_context=ctx)
        with torch.no_grad():
            qn.weight.copy_(qw)
            kn.weight.copy_(kw)
            q1, k1 = qn.forward_pair(q, k, kn)
            rope = get_rope(rot, rotary_dim=rot, max_position=cfg["max_position_embeddings"], base=theta,
                            rope_scaling=None)
            rope.backend = "torch"
            q3, k3 = q1.view(t, hq, d), k1.view(t, hkv, d)
            if rot == d:
                cos, sin = rope.cos_sin_cache[positions].chunk(2, dim=-1)
                q2 = apply_rotary_emb(q3, cos, sin)      # the cache is [positions, 1, R]
                k2 = apply_rotary_emb(k3, cos, sin)
            else:
                q2, k2 = apply_partial_rotary_emb(rope, positions, q3, k3, rot)
        for key, val in (("q", q), ("k", k), ("qw", qw), ("kw", kw), ("positions", positions.float()),
                         ("q_normed", q1), ("k_normed", k1), ("q_out", q2), ("k_out", k2)):
            out[f"{name}.{key}"] = val.contiguous().float()
    torch.manual_seed(5)
    logits = torch.randn(6, 97)
    logits[2, 40] = logits[2, 41] = 9.0          # a tie: argmax takes the first
    out["sampler.logits"] = logits
    out["sampler.greedy"] = Sampler()(logits, None, all_greedy=True).float()
    save_file(out, os.path.join(HERE, "m2_front_end.safetensors"))
    print("wrote", len(out), "tensors")
    oracles()


def oracles():
    from test_minimax_m2_model import _rmsnorm_reference
    from test_minimax_m2_router import _reference as router_reference
    from test_triton_moe import _oracle_local_moe
    from sparseengine.layers.rotary_embedding import _compute_rope_parameters, apply_interleaved_rotary_emb
    out = {}
    g = torch.Generator().manual_seed(23)

    def rnd(*shape, scale=1.0):
        return torch.randn(*shape, generator=g) * scale

    # RMSNorm, float32 and bfloat16 inputs
    x, w = rnd(6, 100, scale=2.0), 1 + 0.1 * rnd(100)
    out["rmsnorm.x"], out["rmsnorm.w"] = x, w
    out["rmsnorm.f32"] = _rmsnorm_reference(x, w, 1e-5)
    out["rmsnorm.bf16"] = _rmsnorm_reference(x.bfloat16(), w.bfloat16(), 1e-5).float()

    # the M2 router at its own size (256 experts, top-8); no ties in random data
    logits, bias = rnd(48, 256, scale=3.0), rnd(256, scale=0.1)
    weights, ids = router_reference(logits, bias)
    out["router.logits"], out["router.bias"] = logits, bias
    out["router.weights"], out["router.ids"] = weights, ids.float()

    # experts: per-expert F.linear loop
    t, h, inter, e, k = 11, 24, 16, 5, 2
    hidden, w13, w2 = rnd(t, h), rnd(e, 2 * inter, h, scale=0.3), rnd(e, h, inter, scale=0.3)
    topk_ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)])
    topk_w = torch.rand(t, k, generator=g)
    out["moe.x"], out["moe.w13"], out["moe.w2"] = hidden, w13, w2
    out["moe.ids"], out["moe.weights"] = topk_ids.float(), topk_w
    out["moe.out"] = _oracle_local_moe(hidden, w13, w2, topk_ids, topk_w, 0)

    # the sampler's cuts: which tokens many draws can produce
    vocab, draws = 40, 6000
    row = torch.linspace(2.5, -2.5, vocab)[torch.randperm(vocab, generator=g)]
    out["sampler.row"] = row
    sampler = Sampler()
    torch.manual_seed(77)
    for i, (top_k, top_p, temp) in enumerate(SAMPLER_CASES):
        toks = sampler._sample(row.repeat(draws, 1), torch.full((draws,), temp), torch.full((draws,), top_p),
                               torch.full((draws,), top_k, dtype=torch.long))
        out[f"sampler.support.{i}"] = torch.bincount(toks, minlength=vocab).gt(0).float()

    # scaled rotary frequency tables
    for name, scaling in ROPE_SCALINGS.items():
        inv, factor = _compute_rope_parameters(64, 5e6, tuple(sorted(scaling.items())))
        out[f"rope.{name}.inv_freq"] = inv.float()
        out[f"rope.{name}.factor"] = torch.tensor([factor])

    # rotation of adjacent pairs
    xr = rnd(5, 3, 16)
    ang = torch.tensor([0.0, 1.0, 2.0, 7.0, 300.0])[:, None] * (1.0 / (10000.0 ** (torch.arange(0, 16, 2).float() / 16)))
    out["interleaved.x"], out["interleaved.angle"] = xr, ang
    out["interleaved.out"] = apply_interleaved_rotary_emb(xr, ang.cos()[:, None, :], ang.sin()[:, None, :])
    save_file({k: v.contiguous().float() for k, v in out.items()}, os.path.join(HERE, "m2_oracles.safetensors"))
    print("wrote", len(out), "oracle tensors")


if __name__ == "__main__":
    main()
