"""Each kind of part alone, and their assembly as data: a toy architecture defined here
(not a model of anyone's) mixes a windowed attention layer with a dense feed-forward, a
mixer with state of its own, a softmax router, a layer that runs twice, an entry that
reads another entry's cache, a block with four norms, a scaled embedding and capped logits.  Nothing in the framework's files changes for it: the
mixer, its spec and the architecture are registered from this file."""
import json
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import plain_m2
import trace_util as tu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---- a mixer with state of its own: y_t = W · mean(x_0..x_t) ----------------------------

@dataclass(frozen=True)
class CompressedRotarySpec:
    rotary_dim: int
    theta: float
    factor: float
    amplitude: float
    pairing: str = "interleaved"
    kind: str = "compressed_rotary"


@dataclass(frozen=True)
class PositionRoutedSpec:
    hidden_size: int
    intermediate_size: int
    num_experts: int
    top_k: int
    kind: str = "position_routed"


@dataclass(frozen=True)
class RunningMeanSpec:
    kind: str = "running_mean"
    hidden_size: int = 0


def _register_toy():
    from sparseengine_b200.config.registry import register_architecture
    from sparseengine_b200.config.specs import (AttentionSpec, DenseMLPSpec, LayerSpec, ModelSpec, MoESpec, ParamSpec,
                                                RMSNormSpec, RotarySpec, ScheduleEntry, Source)
    from sparseengine_b200.parts.base import Mixer, StateRequest, register_mixer
    from sparseengine_b200.parts.linear import linear

    class RunningMean(Mixer):
        """State of its own, kept on the device and reached through the step's device tensors
        only (no host list is read), so that the part may be captured in a CUDA graph: entry e
        owns state row ``step.state_rows[e]`` and tokens ``cu_q[e] .. cu_q[e+1]``; token i
        belongs to entry ``token_seq[i]``."""
        graph_safe = True

        def parameters(self):
            return {"w": ParamSpec((self.spec.hidden_size, self.spec.hidden_size))}

        def state_request(self):
            return StateRequest((self.spec.hidden_size + 1,), torch.float32)     # running sum and count

        def forward(self, x, step, slot):
            h = self.spec.hidden_size
            t = x.shape[0]
            seq = step.token_seq.long()
            rows = step.state_rows.long()
            idx = torch.arange(t, device=x.device)
            # per-request inclusive sums within the step: token i adds the tokens j <= i of its own request
            same = (seq[:, None] == seq[None, :]) & (idx[None, :] <= idx[:, None])
            csum = same.float() @ x.float() + slot.state[rows][seq, :h]
            cnt = (idx - step.cu_q.long()[seq] + 1).float() + slot.state[rows][seq, h]
            out = (csum / cnt[:, None]).to(x.dtype)
            last = step.cu_q.long()[1:] - 1                      # each entry's last token
            slot.state[rows] = torch.cat((csum[last], cnt[last, None]), 1)
            return linear(out, self.w)

    register_mixer("running_mean", RunningMean)

    # another position encoding: rotary with compressed positions (every frequency divided by
    # `factor`), the rotated dims scaled by `amplitude`, and adjacent dims (2i, 2i+1) as pairs; the
    # attention part only asks its position encoding for (frequencies, number of rotated dims,
    # amplitude, pairing)
    from sparseengine_b200.parts.base import PositionEncoding, register_position

    class CompressedRotary(PositionEncoding):
        graph_safe = True

        _table = None

        def kernel_args(self, device):
            from sparseengine_b200.parts.position import RotaryArgs
            r = self.spec.rotary_dim
            if self._table is None:          # once: a graph-safe part copies nothing from the host in a step
                inv = 1.0 / (self.spec.theta ** (torch.arange(0, r, 2, dtype=torch.float32) / r))
                self._table = (inv / self.spec.factor).to(device)
            return RotaryArgs(self._table, r, float(self.spec.amplitude), self.spec.pairing)

    register_position("compressed_rotary", CompressedRotary)

    # a feed-forward with a routing of its own: the token at position p goes to experts
    # p, p + 1, ... (mod E) with equal weights; the experts themselves are the framework's
    from sparseengine_b200.config.specs import ParamSpec
    from sparseengine_b200.parts.base import register_feed_forward
    from sparseengine_b200.parts.moe import _RoutedSwiGLU

    class PositionRouted(_RoutedSwiGLU):
        def __init__(self, spec, dtype):
            super().__init__(spec, dtype)
            self.num_experts, self.top_k = spec.num_experts, spec.top_k
            self.hidden, self.inter = spec.hidden_size, spec.intermediate_size

        def parameters(self):
            sp = self.spec
            return {"w13": ParamSpec((sp.num_experts, 2 * sp.intermediate_size, sp.hidden_size)),
                    "w2": ParamSpec((sp.num_experts, sp.hidden_size, sp.intermediate_size))}

        def forward(self, x, step):
            k = torch.arange(self.top_k, dtype=torch.int32, device=x.device)
            ids = ((step.positions[:, None] + k[None, :]) % self.num_experts).to(torch.int32).contiguous()
            weights = torch.full(ids.shape, 1.0 / self.top_k, dtype=torch.float32, device=x.device)
            return self.run_experts(x, ids, weights)

    register_feed_forward("position_routed", PositionRouted)

    # another arrangement of a block: a norm before and one after each sublayer (four norms); the
    # two further norms come from LayerSpec.extra, by the names this arrangement gives them
    from sparseengine_b200.parts.base import make_feed_forward, make_mixer, make_norm
    from sparseengine_b200.parts.block import ARRANGEMENTS

    class SandwichBlock:
        def __init__(self, spec, dtype):
            self.mixer = make_mixer(spec.mixer, dtype)
            self.feed_forward = make_feed_forward(spec.feed_forward, dtype)
            self.norms = {k: make_norm(v, dtype) for k, v in
                          (("mixer_norm", spec.mixer_norm), ("feed_forward_norm", spec.feed_forward_norm),
                           ("after_mixer", spec.extra["after_mixer"]), ("after_feed_forward", spec.extra["after_feed_forward"]))}

        def parts(self):
            return {"mixer": self.mixer, "feed_forward": self.feed_forward, **self.norms}

        def forward(self, hidden, residual, step, slot):
            x, residual = self.norms["mixer_norm"].forward(hidden, residual)
            hidden, _ = self.norms["after_mixer"].forward(self.mixer.forward(x, step, slot))
            x, residual = self.norms["feed_forward_norm"].forward(hidden, residual)
            hidden, _ = self.norms["after_feed_forward"].forward(self.feed_forward.forward(x, step))
            return hidden, residual

    ARRANGEMENTS["sandwich"] = SandwichBlock

    @dataclass(frozen=True)
    class ToyConfig:
        raw: tuple

        @classmethod
        def from_dict(cls, raw):
            return cls(tuple(sorted((k, json.dumps(v)) for k, v in raw.items())))

        def get(self, k):
            return json.loads(dict(self.raw)[k])

    def build(cfg):
        h, v = cfg.get("hidden_size"), cfg.get("vocab_size")
        hq, hkv, d = cfg.get("heads"), cfg.get("kv_heads"), cfg.get("head_dim")
        norm = RMSNormSpec(size=h, eps=cfg.get("eps"))
        att = AttentionSpec(hidden_size=h, num_heads=hq, num_kv_heads=hkv, head_dim=d, scale=d ** -0.5,
                            qk_norm=None, window=cfg.get("window"),
                            position=CompressedRotarySpec(rotary_dim=d, theta=cfg.get("theta"), factor=cfg.get("factor"),
                                                          amplitude=cfg.get("amplitude")))
        att_full = AttentionSpec(hidden_size=h, num_heads=hq, num_kv_heads=hkv, head_dim=d, scale=d ** -0.5,
                                 qk_norm=None, window=None, position=None)
        dense = DenseMLPSpec(hidden_size=h, intermediate_size=cfg.get("inter"))
        moe = MoESpec(hidden_size=h, num_experts=cfg.get("experts"), top_k=cfg.get("top_k"),
                      intermediate_size=cfg.get("inter"), score_fn="softmax", selection_bias=False,
                      renormalize=False, routed_scale=cfg.get("routed_scale"))

        def att_sources(p):
            return {"mixer.qkv": (Source(p + "qkv"),), "mixer.o": (Source(p + "o"),)}

        def norms(p):
            return {"mixer_norm.weight": (Source(p + "n1"),), "feed_forward_norm.weight": (Source(p + "n2"),)}

        l0 = LayerSpec(att, dense, norm, norm, sources={**att_sources("l0."), **norms("l0."),
                                                         "feed_forward.w13": (Source("l0.w13"),),
                                                         "feed_forward.w2": (Source("l0.w2"),)})
        l1 = LayerSpec(RunningMeanSpec(hidden_size=h), moe, norm, norm,
                       sources={"mixer.w": (Source("l1.w"),), **norms("l1."), "feed_forward.gate": (Source("l1.gate"),),
                                "feed_forward.w13": (Source("l1.w13"),), "feed_forward.w2": (Source("l1.w2"),)})
        routed = PositionRoutedSpec(hidden_size=h, intermediate_size=cfg.get("inter"), num_experts=3, top_k=2)
        l2 = LayerSpec(att_full, routed, norm, norm, arrangement="sandwich",
                       extra={"after_mixer": norm, "after_feed_forward": norm},
                       sources={**att_sources("l2."), **norms("l2."), "feed_forward.w13": (Source("l2.w13"),),
                                "feed_forward.w2": (Source("l2.w2"),), "after_mixer.weight": (Source("l2.n3"),),
                                "after_feed_forward.weight": (Source("l2.n4"),)})
        # layer 0 runs twice (each visit with a cache of its own), layer 1 runs twice (each
        # visit with a state of its own), and the last entry reads the cache entry 3 wrote.
        order = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2), ScheduleEntry(1),
                 ScheduleEntry(2, cache=3)]
        return ModelSpec(architecture="ToyForCausalLM", hidden_size=h, vocab_size=v, max_position=cfg.get("max_pos"),
                         layers=[l0, l1, l2], order=order, final_norm=norm, final_norm_source="norm",
                         embed_source="embed", head_source=None, embed_scale=cfg.get("embed_scale"),
                         logit_softcap=cfg.get("logit_softcap"))

    register_architecture("ToyForCausalLM", ToyConfig, build)


TOY = {"architectures": ["ToyForCausalLM"], "hidden_size": 40, "vocab_size": 131, "heads": 6, "kv_heads": 2,
       "head_dim": 16, "eps": 2e-6, "window": 5, "theta": 777.0, "inter": 24, "experts": 5, "top_k": 2,
       "routed_scale": 1.7, "max_pos": 256, "factor": 4.0, "amplitude": 0.5, "embed_scale": 1.5, "logit_softcap": 12.0}


def toy_tensors(seed=3):
    g = torch.Generator().manual_seed(seed)
    c = TOY
    h, q, kv = c["hidden_size"], c["heads"] * c["head_dim"], c["kv_heads"] * c["head_dim"]

    def m(*s, std=0.15):
        return torch.randn(*s, generator=g) * std

    def n():
        return 1 + 0.1 * torch.randn(h, generator=g)

    t = {"embed": m(c["vocab_size"], h, std=0.5), "norm": n()}
    for l, e in (("l0.", 1), ("l2.", 3)):
        t.update({l + "qkv": m(q + 2 * kv, h), l + "o": m(h, q), l + "n1": n(), l + "n2": n(),
                  l + "w13": m(e, 2 * c["inter"], h), l + "w2": m(e, h, c["inter"])})
    # the norms after the sublayers scale their outputs down to the size the sublayers' own outputs
    # have elsewhere in this model (a norm with weights near 1 would triple that layer's share of the
    # residual stream, and with it the share of its bfloat16 rounding in the logits)
    t.update({"l2.n3": 0.3 * n(), "l2.n4": 0.3 * n()})
    t.update({"l1.w": m(h, h), "l1.n1": n(), "l1.n2": n(), "l1.gate": m(c["experts"], h, std=0.5),
              "l1.w13": m(c["experts"], 2 * c["inter"], h), "l1.w2": m(c["experts"], h, c["inter"])})
    return t


def toy_plain(t, tokens, act=torch.float32, forced=None, probs=None, exact_probs=None):
    """The toy model written out with the plain implementation's functions.  ``forced``:
    expert ids [T, k] for each of the two visits of the routed layer (the engine's own
    choice, followed through near-ties).  ``probs``: a list that receives the router's
    probabilities of each visit; ``exact_probs``: those of a 32-bit run, by which a bfloat16 run
    measures how far rounding moves its routers' probabilities."""
    c = TOY
    n = len(tokens)
    t = {k: (v if k == "l1.gate" else plain_m2._round(v, act)) for k, v in t.items()}   # the router stays 32-bit
    hq, hkv, d, inter = c["heads"], c["kv_heads"], c["head_dim"], c["inter"]
    pos = torch.arange(n)

    def compressed_rotary(x):
        inv = plain_m2.rope_inv_freq(d, c["theta"]) / c["factor"]
        ang = pos.to(torch.float32).unsqueeze(-1) * inv
        cos, sin = (torch.cos(ang) * c["amplitude"]).unsqueeze(1), (torch.sin(ang) * c["amplitude"]).unsqueeze(1)
        x = x.to(torch.float32)
        x1, x2 = x[..., 0::2], x[..., 1::2]                 # adjacent pairs, written back in place
        out = torch.empty_like(x)
        out[..., 0::2] = plain_m2._round(x1 * cos - x2 * sin, act)
        out[..., 1::2] = plain_m2._round(x2 * cos + x1 * sin, act)
        return out

    def attention(x, l, window, rotate, kv=None):
        qkv = plain_m2.linear(x, t[l + "qkv"], act)
        q = qkv[:, :hq * d].view(n, hq, d)
        rot = compressed_rotary if rotate else (lambda y: y)
        if kv is None:
            k = qkv[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
            v = qkv[:, (hq + hkv) * d:].view(n, hkv, d)
            k = rot(k)
        else:
            k, v = kv
        q = rot(q)
        o = plain_m2.causal_attention(q, k, v, act, window)
        return plain_m2.linear(o.reshape(n, hq * d), t[l + "o"], act), (k, v)

    def dense(x, l):
        if l == "l2.":          # the position-routed feed-forward: experts p and p + 1 (mod 3), half each
            ids = (pos[:, None] + torch.arange(2)[None, :]) % 3
            w = torch.full((n, 2), 0.5)
        else:
            ids, w = torch.zeros(n, 1, dtype=torch.long), torch.ones(n, 1)
        return plain_m2.experts(x, ids, w, t[l + "w13"][:, :inter], t[l + "w13"][:, inter:], t[l + "w2"], act)

    def running_mean(x):
        mean = torch.cumsum(x.float(), 0) / torch.arange(1, n + 1)[:, None]
        return plain_m2.linear(plain_m2._round(mean, act), t["l1.w"], act)

    visits = []

    def moe(x):
        p = torch.softmax(x.float() @ t["l1.gate"].t(), -1)
        thr_ids, _, _ = plain_m2.router(x, t["l1.gate"], torch.zeros(c["experts"]), c["top_k"])   # sigmoid is monotone
        if forced is not None:
            own, thr_ids = thr_ids, forced[len(visits)].long()
            srt = p.sort(-1, descending=True).values
            gap = srt[:, c["top_k"] - 1] - srt[:, c["top_k"]]
            # Where the plain router's gap is clear the engine must have chosen the same experts.
            # "Clear" in bfloat16: the router's input carries the rounding of several bfloat16
            # layers (about 1 % of its size), which moves a logit (40 terms, gate weights of
            # 0.5) by about 0.03 and a probability near 0.3 by about 0.01; where this request's
            # own bfloat16 and 32-bit probabilities differ by more (measured, when the 32-bit ones
            # are given), twice that difference.
            clear = 2e-3 if act == torch.float32 else 1e-2
            if exact_probs is not None:
                clear = max(clear, 2 * float((p - exact_probs[len(visits)]).abs().max()))
            for i in range(n):
                if gap[i] > clear:
                    assert sorted(own[i].tolist()) == sorted(thr_ids[i].tolist()), (len(visits), i, float(gap[i]))
        visits.append(1)
        if probs is not None:
            probs.append(p)
        w = p.gather(1, thr_ids) * c["routed_scale"]
        return plain_m2.experts(x, thr_ids, w, t["l1.w13"][:, :inter], t["l1.w13"][:, inter:], t["l1.w2"], act)

    hidden = plain_m2._round(plain_m2.embedding(t["embed"], torch.tensor(tokens)) * c["embed_scale"], act)
    residual = None
    shared = None
    for step, (layer, share) in enumerate([("l0.", False), ("l1.", False), ("l0.", False), ("l2.", False),
                                           ("l1.", False), ("l2.", True)]):
        eps = c["eps"]
        if residual is None:
            residual, x = hidden, plain_m2.rms_norm(hidden, t[layer + "n1"], eps, act)
        else:
            x, residual = plain_m2.add_rms_norm(hidden, residual, t[layer + "n1"], eps, act)
        if layer == "l1.":
            hidden = running_mean(x)
        elif layer == "l0.":
            hidden, _ = attention(x, layer, c["window"], True)
        else:
            hidden, kv = attention(x, layer, None, False, kv=shared if share else None)
            if not share:
                shared = kv
            hidden = plain_m2.rms_norm(hidden, t["l2.n3"], eps, act)           # the sandwich block's norm after the mixer
        x, residual = plain_m2.add_rms_norm(hidden, residual, t[layer + "n2"], eps, act)
        hidden = moe(x) if layer == "l1." else dense(x, layer)
        if layer == "l2.":
            hidden = plain_m2.rms_norm(hidden, t["l2.n4"], eps, act)           # and after the feed-forward
    x, _ = plain_m2.add_rms_norm(hidden, residual, t["norm"], c["eps"], act)
    logits = plain_m2.linear(x, t["embed"], act)        # tied head
    return plain_m2._round(torch.tanh(logits / c["logit_softcap"]) * c["logit_softcap"], act)


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    _register_toy()
    d = str(tmp_path_factory.mktemp("toy"))
    t = toy_tensors()
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(TOY, f)
    save_file(t, os.path.join(d, "model.safetensors"))
    return d, t


def test_toy_architecture_layout(toy_folder):
    from sparseengine_b200.config.registry import load_model_spec
    from sparseengine_b200.engine.model import Model
    _, spec = load_model_spec(toy_folder[0])
    lay = Model(spec, torch.float32).layout
    assert len(lay.groups) == 2                                   # windowed pages and all-keys pages
    assert {g[0].window: g[1] for g in lay.groups} == {5: 2, None: 1}
    assert len(lay.states) == 2                                   # one state per visit of the stateful layer
    assert lay.entries[5].cache_layer == lay.entries[3].cache_layer and not lay.entries[5].write
    assert lay.entries[0].cache_layer != lay.entries[2].cache_layer


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_steps_like_its_plain_form(toy_folder, dtype):
    from sparseengine_b200.engine.factory import build_runner
    folder, t = toy_folder
    act = torch.float32 if dtype == "float32" else torch.bfloat16
    seqs = {f"s{i}": tu.random_prompt(TOY["vocab_size"], n, i) for i, n in enumerate([3, 11, 26, 40, 17])}
    for cut in (tu.trace_whole, tu.trace_chunks, tu.trace_mixed):
        steps = cut(seqs)
        page = 4
        runner = build_runner(folder, dtype=dtype, page_size=page, num_pages=tu.max_live_tokens(steps) // page,
                              max_rows=4)
        got, routed = tu.run_trace_runner(runner, steps, capture=True)
        for sid, toks in seqs.items():
            mine = {k: v for k, v in got.items() if k[0] == sid}
            if dtype == "float32":
                tu.compare(mine, {sid: toy_plain(t, toks, act).numpy()}, 2e-5, 2e-5, what=f"toy {dtype} {cut.__name__}")
                continue
            # bfloat16.  The toy's logits are about ten times larger than the tiny M2 models' (tied head
            # on an embedding of std 0.5) and it runs six visits without a QK norm, so rounding moves
            # them a lot: its plain form in bfloat16 differs from its plain form in 32-bit by 0.1 to 0.3
            # at the worst logit of a request.  That difference, measured here for each request, is how
            # far bfloat16 rounding moves this model's logits, and the bound between two bfloat16
            # implementations: the engine may differ from the plain form by as much as the plain form
            # differs from the exact one (plus one unit in the last place of the logit).
            exact_probs = []
            exact = toy_plain(t, toks, probs=exact_probs).numpy()
            ref = toy_plain(t, toks, act, routed[sid], exact_probs=exact_probs).numpy()
            noise = float(np.abs(ref - exact).max())
            assert noise < 0.12 * float(np.sqrt(np.mean(exact ** 2)))         # and that is a small share of their size
            tu.compare(mine, {sid: ref}, noise, tu.BF16_ULP, what=f"toy {dtype} {cut.__name__}")
        for g in runner.cache.groups:
            assert g.pool.free == g.pool.num_pages
        win = [g for g in runner.cache.groups if g.window][0]
        assert win.pool.reused_total > 0                          # windowed pages come back while a request lives
        runner.cache.check()


def test_toy_stateful_mixer_decodes_in_cuda_graphs(toy_folder):
    """A mixer with state of its own that reads the step's device tensors only declares itself
    graph-safe, and the whole toy model's decode steps replay CUDA graphs: same logits as launch
    by launch, and as the plain form."""
    from sparseengine_b200.engine.factory import build_runner
    folder, t = toy_folder
    seqs = {f"s{i}": tu.random_prompt(TOY["vocab_size"], n, 40 + i) for i, n in enumerate([45, 38, 50])}
    steps = tu.trace_mixed(seqs, live=3, chunk=9, decode_tail=30, seed=2)
    out = {}
    for graphs in (True, False):
        runner = build_runner(folder, dtype="float32", page_size=4, num_pages=tu.max_live_tokens(steps) // 4, max_rows=4,
                              decode_graphs=graphs)
        assert runner.decode_graphs == graphs
        out[graphs] = tu.run_trace_runner(runner, steps)
        assert (runner.graph_replays > 10) == graphs
    ref = {sid: toy_plain(t, toks).numpy() for sid, toks in seqs.items()}
    tu.compare(out[True], ref, 2e-5, 2e-5, what="toy with graphs")
    for k in out[True]:
        assert np.abs(out[True][k] - out[False][k]).max() <= 1e-6, k


# ---- the built-in parts alone -----------------------------------------------------------

def _step_context(q_lens, starts, rows, dtype):
    from sparseengine_b200.parts.base import StepContext
    i32 = dict(dtype=torch.int32, device=DEV)
    t = sum(q_lens)
    return StepContext(
        num_tokens=t, num_seqs=len(q_lens), token_ids=torch.zeros(t, **i32),
        positions=torch.cat([torch.arange(s, s + n) for s, n in zip(starts, q_lens)]).to(**i32),
        token_seq=torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(**i32),
        seq_rows=torch.tensor(rows, **i32), cu_q=torch.tensor(np.concatenate(([0], np.cumsum(q_lens))), **i32),
        kv_len=torch.tensor([s + n for s, n in zip(starts, q_lens)], **i32), q_lens=list(q_lens),
        q_starts=list(starts), kv_lens=[s + n for s, n in zip(starts, q_lens)], rows=list(rows), dtype=dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_attention_part_whole_then_continued(dtype, name):
    """The attention mixer alone: a whole sequence in one call equals the plain block; the
    same sequence in two calls (second reads the first's keys from the pages) too."""
    from sparseengine_b200.config.registry import load_model_spec
    from sparseengine_b200.parts.base import LayerSlot, make_mixer
    cfg = tu.TINY[name][0]
    _, spec = load_model_spec(cfg)
    aspec = spec.layers[0].mixer
    hq, hkv, d = aspec.num_heads, aspec.num_kv_heads, aspec.head_dim
    g = torch.Generator().manual_seed(1)
    w = {"qkv": torch.randn((hq + 2 * hkv) * d, aspec.hidden_size, generator=g) * 0.2,
         "o": torch.randn(aspec.hidden_size, hq * d, generator=g) * 0.2,
         "q_norm": 1 + 0.1 * torch.randn(hq * d, generator=g), "k_norm": 1 + 0.1 * torch.randn(hkv * d, generator=g)}
    part = make_mixer(aspec, dtype)
    part.bind({k: v.to(dtype).to(DEV) for k, v in w.items()})
    n, page = 29, 4
    x = (torch.randn(n, aspec.hidden_size, generator=g)).to(dtype)
    lt = {"wq": w["qkv"][:hq * d], "wk": w["qkv"][hq * d:(hq + hkv) * d], "wv": w["qkv"][(hq + hkv) * d:],
          "wo": w["o"], "qn": w["q_norm"], "kn": w["k_norm"]}
    lt = {k: plain_m2._round(v, dtype) for k, v in lt.items()}
    ref, _ = plain_m2.attention_block(x.float(), lt, cfg, torch.arange(n), dtype)
    table = torch.arange(8, dtype=torch.int32, device=DEV).flip(0).view(1, 8).contiguous()
    for cuts in ([n], [17, 12], [1] * n):
        slot = LayerSlot(kv=torch.zeros(8, 2, hkv, page, d, dtype=dtype, device=DEV), table=table, page_size=page)
        outs, a = [], 0
        for c in cuts:
            outs.append(part.forward(x[a:a + c].to(DEV), _step_context([c], [a], [0], dtype), slot))
            a += c
        torch.testing.assert_close(torch.cat(outs).float().cpu(), ref,
                                   **(dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_moe_part_alone(dtype, name):
    from sparseengine_b200.config.registry import load_model_spec
    from sparseengine_b200.parts.base import make_feed_forward
    cfg, seed, std, _, bias_std, _ = tu.TINY[name]
    _, spec = load_model_spec(cfg)
    part = make_feed_forward(spec.layers[0].feed_forward, dtype)
    tensors = plain_m2.random_tensors(cfg, seed, 0.1, 0.0, 0.2)
    lt = plain_m2._layer_tensors(tensors, 0, cfg)
    part.bind({"gate": lt["gate"].to(DEV), "selection_bias": lt["bias"].to(DEV),
               "w13": torch.cat([lt["w1"], lt["w3"]], 1).to(dtype).to(DEV), "w2": lt["w2"].to(dtype).to(DEV)})
    x = torch.randn(37, cfg["hidden_size"], generator=torch.Generator().manual_seed(2)).to(dtype)
    out = part.forward(x.to(DEV), None)
    ltr = {k: (v if k in ("gate", "bias") else plain_m2._round(v, dtype)) for k, v in lt.items()}
    ref = plain_m2.moe_block(x.float(), ltr, cfg, dtype)
    torch.testing.assert_close(out.float().cpu(), ref,
                               **(dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)))


def test_norm_and_position_parts_alone():
    from sparseengine_b200.config.specs import RMSNormSpec, RotarySpec
    from sparseengine_b200.parts.base import make_norm, make_position
    norm = make_norm(RMSNormSpec(size=100, eps=1e-5), torch.float32)
    w = 1 + 0.1 * torch.randn(100)
    norm.bind({"weight": w.to(DEV)})
    x, r = torch.randn(6, 100), torch.randn(6, 100)
    y, res = norm.forward(x.to(DEV))
    assert res.data_ptr() == res.data_ptr() and torch.allclose(y.cpu(), plain_m2.rms_norm(x, w, 1e-5, torch.float32), atol=1e-6)
    y, res = norm.forward(x.to(DEV), r.to(DEV))
    ry, rr = plain_m2.add_rms_norm(x, r, w, 1e-5, torch.float32)
    assert torch.allclose(y.cpu(), ry, atol=1e-6) and torch.equal(res.cpu(), rr)
    pos = make_position(RotarySpec(rotary_dim=24, theta=5e6), torch.float32)
    args = pos.kernel_args(DEV)
    assert args.rotary_dim == 24 and args.scale == 1.0 and args.pairing == "split_half"
    assert torch.equal(args.inv_freq.cpu(), plain_m2.rope_inv_freq(24, 5e6))
    assert make_position(RotarySpec(rotary_dim=24, pairing="interleaved"), torch.float32).kernel_args(DEV).pairing == "interleaved"
    with pytest.raises(ValueError):
        make_position(RotarySpec(rotary_dim=24, pairing="triples"), torch.float32)
    with pytest.raises(ValueError, match="no norm registered"):
        make_norm(type("S", (), {"kind": "layer_norm"})(), torch.float32)
