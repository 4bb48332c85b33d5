"""The engine at MiniMax M2's own layer sizes against the plain implementation: two layers,
random weights N(0, 0.02), prompts of 1 / 300 / 1,024 / 2,047 uniform random tokens, each run
whole, with its last 32 tokens one by one, in 128-token portions, and mixed (four live requests,
portions of some beside single tokens of others, with so few pages that they are used again).
In 32-bit the logits are compared tightly; in bfloat16 the plain implementation follows the
engine's choice of experts through near-ties of a router, and must have chosen the same experts
wherever its own gap is clear.

At these sizes the engine takes kernels that the tiny configurations never reach together (the
tiled router over 256 experts, selection by a warp from 128 tokens, the three-launch routing
build, expert tiles of 128 and 256 rows, row tiles of 48 query heads on 8 KV heads).  Both sides
use the same tensors: the plain implementation reads views of the engine's parameters by
checkpoint name, and runs on the GPU in 32-bit arithmetic (no reduced-precision matrix mode),
with one matrix product per (slot, expert) group.  The 200,064-wide head is asked for at a few
dozen positions of each prompt (edges of pages, of portions and of the prompt)."""
import numpy as np
import pytest
import torch

import plain_m2
import trace_util as tu

pytestmark = pytest.mark.gpu

M2_LAYER_SIZES = {
    "architectures": ["MiniMaxM2ForCausalLM"], "model_type": "minimax_m2", "num_hidden_layers": 2,
    "hidden_size": 3072, "num_attention_heads": 48, "num_key_value_heads": 8, "head_dim": 128,
    "rotary_dim": 64, "rope_theta": 5000000.0, "rms_norm_eps": 1e-6,
    "num_local_experts": 256, "num_experts_per_tok": 8, "intermediate_size": 1536,
    "vocab_size": 200064, "max_position_embeddings": 4096, "tie_word_embeddings": False,
    "hidden_act": "silu", "qk_norm_type": "per_layer", "use_qk_norm": True, "scoring_func": "sigmoid",
    "use_routing_bias": True, "use_mtp": True, "shared_intermediate_size": 0,
}
LENGTHS = (1, 300, 1024, 2047)
PAGE = 16
ACT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# gap of router scores above which the engine must have chosen the plain router's experts
CLEAR_GAP = {"float32": 1e-5, "bfloat16": 1e-2}


def wanted_positions(n: int) -> list:
    marks = {0, 1, 15, 16, 17, 31, 32, 127, 128, 129, 255, 256, 299, 511, 512, 1023, 1024, 2046} | set(range(n - 33, n))
    return sorted(p for p in marks if 0 <= p < n)


def restrict_wants(steps: list, wanted: dict) -> list:
    """The same steps asking only for the positions in ``wanted[id]``."""
    pos: dict = {}
    out = []
    for s in steps:
        entries = []
        for e in s["entries"]:
            a = pos.get(e["id"], 0)
            entries.append({"id": e["id"], "tokens": e["tokens"],
                            "want": [w for w in range(len(e["tokens"])) if a + w in wanted[e["id"]]]})
            pos[e["id"]] = a + len(e["tokens"])
        out.append({"step": s["step"], "entries": entries, "end": s["end"]})
    return out


def portions_of_128(seqs: dict) -> list:
    steps, n = [], 0
    for sid, toks in seqs.items():
        for a in range(0, len(toks), 128):
            b = min(len(toks), a + 128)
            steps.append({"step": n, "entries": [{"id": sid, "tokens": toks[a:b], "want": list(range(b - a))}],
                          "end": [sid] if b == len(toks) else []})
            n += 1
    return steps


CUTS = {
    "whole": tu.trace_whole,
    "tail32": tu.trace_tail_decode,
    "portions128": portions_of_128,
    "mixed": lambda seqs: tu.trace_mixed(seqs, live=4, chunk=128, decode_tail=32, seed=4),
}


def checkpoint_views(model) -> dict:
    """{checkpoint tensor name: view of the engine's parameter}, plus the experts' stacks."""
    from sparseengine_b200.weights.loader import _dest
    out = {}
    for p in model.params():
        t = getattr(p.owner, p.name)
        for src in p.sources:
            out[src.name] = _dest(t, src.index)
    inter = M2_LAYER_SIZES["intermediate_size"]
    for i, block in enumerate(model.blocks):
        ff = block.feed_forward
        base = f"model.layers.{i}.block_sparse_moe.experts.stacked."
        out[base + "w1"], out[base + "w3"], out[base + "w2"] = ff.w13[:, :inter], ff.w13[:, inter:], ff.w2
    return out


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request):
    from sparseengine_b200.engine.factory import build_runner
    dtype = request.param
    torch.backends.cuda.matmul.allow_tf32 = False
    seqs = {f"p{n}": tu.random_prompt(M2_LAYER_SIZES["vocab_size"], n, 400 + n) for n in LENGTHS}
    traces = {cut: restrict_wants(fn(seqs), {sid: set(wanted_positions(len(t))) for sid, t in seqs.items()})
              for cut, fn in CUTS.items()}
    most = max(tu.max_live_tokens(steps) for steps in traces.values())
    runner = build_runner(dict(M2_LAYER_SIZES, torch_dtype=dtype), dtype=dtype, page_size=PAGE, num_pages=most // PAGE,
                          max_rows=4, max_seq_len=4096, random_weights=True, seed=4, random_std=0.02, norm_std=0.05,
                          bias_std=0.05)
    yield dtype, runner, seqs, traces, checkpoint_views(runner.model)
    del runner
    torch.cuda.empty_cache()


_plain_cache: dict = {}


def plain_logits(dtype, tensors, seqs, routed):
    """{id: {position: logits row}} from the plain implementation, on the GPU."""
    out = {}
    for sid, toks in seqs.items():
        want = wanted_positions(len(toks))
        forced = None if routed is None else [f.to("cuda") for f in routed[sid]]
        key = (dtype, sid, None if forced is None else tuple(hash(f.cpu().numpy().tobytes()) for f in forced))
        if key not in _plain_cache:
            info = {}
            logits = plain_m2.forward(M2_LAYER_SIZES, tensors, toks, ACT[dtype], forced_ids=forced, info=info, want=want)
            if forced is not None:
                for layer, (own, gap, eng) in enumerate(zip(info["ids"], info["margin"], forced)):
                    clear = gap > CLEAR_GAP[dtype]
                    same = (own.sort(-1).values == eng.long().sort(-1).values).all(-1)
                    bad = (clear & ~same).nonzero()
                    assert len(bad) == 0, (f"{dtype} request {sid} layer {layer} position {int(bad[0])}: engine routed to "
                                           f"{eng[int(bad[0])].tolist()}, plain to {own[int(bad[0])].tolist()} with a "
                                           f"clear gap {float(gap[int(bad[0])]):.2e}")
            _plain_cache[key] = dict(zip(want, logits.cpu().numpy()))
        out[sid] = _plain_cache[key]
    return out


@pytest.mark.parametrize("cut", list(CUTS))
def test_m2_layer_sizes_give_the_plain_logits_under_every_cut(setup, cut):
    from sparseengine_b200.csrc import ops
    dtype, runner, seqs, traces, tensors = setup
    steps = traces[cut]
    if cut == "mixed":
        assert max(len(s["entries"]) for s in steps) == 4
        assert any(len({len(e["tokens"]) > 1 for e in s["entries"]}) == 2 for s in steps)   # a portion beside a decode
    pool = runner.cache.groups[0].pool
    reused = pool.reused_total
    before = dict(ops.calls)
    routed = None
    if dtype == "bfloat16":
        got, routed = tu.run_trace_runner(runner, steps, capture=True)
    else:
        got = tu.run_trace_runner(runner, steps)
    ops.error_check("cuda:0")
    took = {k for k, v in ops.calls.items() if v > before.get(k, 0)}
    if dtype == "bfloat16":
        assert "se_moe_grouped_gemm_tc" in took and "se_paged_attention_plain" not in took
        assert "se_attn_prefill_tc" in took
    assert len(got) == sum(len(wanted_positions(len(t))) for t in seqs.values())
    ref = plain_logits(dtype, tensors, seqs, routed)
    rms = float(np.sqrt(np.mean(np.concatenate([np.stack(list(r.values())).ravel() for r in ref.values()]) ** 2)))
    # 32-bit: only the order of sums differs (products of 3,072 and 1,536 terms): 1e-4 of the logits'
    # size.  bfloat16: activations carry 8 bits through two layers; 4% of the logits' size and one
    # unit in the last place of the logit itself.
    atol, rtol = (1e-4 * rms, 1e-4) if dtype == "float32" else (4e-2 * rms, 2.0 ** -7)
    worst = tu.compare(got, ref, atol, rtol, what=f"M2 layer sizes {dtype} {cut}")
    print(f"[m2 sizes vs plain] {dtype} {cut}: logits rms {rms:.3f}, worst |diff| {worst:.3e}")
    assert pool.free == pool.num_pages and pool.reused_total > reused      # everything came back; pages were used again
    runner.cache.check()
