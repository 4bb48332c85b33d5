"""Replay on the GPU, in 32-bit and in bfloat16, against the plain implementation: each
request alone and whole; most of it in one step and the last 32 tokens one by one; in
portions of changing size down to two tokens; mixed, up to four live requests with so
few pages that they are used again; long decoding; the first tokens of a sequence; and
the same through the ``bin/trace_run`` program."""
import numpy as np
import pytest
import torch

import plain_m2
import trace_util as tu

pytestmark = pytest.mark.gpu

ACT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# Bounds: trace_util.compare_in_dtype (32-bit: the order of sums; bfloat16: a share of the
# logits' root mean square).
LENGTHS = [5, 9, 13, 47, 70, 33]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in tu.TINY:
        for dtype in ACT:
            d = str(tmp_path_factory.mktemp(f"m2_{name}_{dtype}"))
            out[name, dtype] = (d, tu.make_model_folder(d, name, dtype))
    return out


_REF = {}
NEAR_TIE = {"float32": 1e-5, "bfloat16": 4e-3}    # gap of router scores below which either expert may win


def reference(name, dtype, tensors, seqs, routed=None):
    """Plain logits per request.  In bfloat16 the plain implementation is made to follow
    the engine's choice of experts (``routed``, captured from the engine): where two
    experts' scores are closer than the rounding noise either may win, and the logits
    jump.  Wherever the plain router's own gap is clear the engine must have chosen the
    same experts."""
    cfg = tu.TINY[name][0]
    out = {}
    for sid, toks in seqs.items():
        forced = routed[sid] if routed is not None else None
        key = (name, dtype, tuple(toks), None if forced is None else tuple(tuple(map(tuple, f.tolist())) for f in forced))
        if key not in _REF:
            info = {}
            logits = plain_m2.forward(cfg, tensors, toks, ACT[dtype], forced_ids=forced, info=info).numpy()
            if forced is not None:
                for layer, (own, gap, eng) in enumerate(zip(info["ids"], info["margin"], forced)):
                    for t in range(len(toks)):
                        if gap[t] > NEAR_TIE[dtype]:
                            assert sorted(own[t].tolist()) == sorted(eng[t].tolist()), (
                                f"{name} {dtype} request {sid} layer {layer} position {t}: engine routed to "
                                f"{eng[t].tolist()}, plain to {own[t].tolist()} with a clear gap {float(gap[t]):.2e}")
            _REF[key] = logits
        out[sid] = _REF[key]
    return out


def first_near_tie(name, dtype, tensors, toks):
    """First position at which some router of the plain implementation has a near-tie."""
    info = {}
    plain_m2.forward(tu.TINY[name][0], tensors, toks, ACT[dtype], info=info)
    gap = torch.stack(info["margin"]).min(0).values
    bad = (gap <= NEAR_TIE[dtype]).nonzero()
    return int(bad[0]) if len(bad) else len(toks)


def sequences(name, lengths=LENGTHS):
    vocab = tu.TINY[name][0]["vocab_size"]
    return {f"r{i}": tu.random_prompt(vocab, n, 10 * i + len(name)) for i, n in enumerate(lengths)}


def runner_for(folder, name, dtype, steps, max_rows=4):
    from sparseengine_b200.engine.factory import build_runner
    page = tu.TINY[name][5]
    mt = tu.max_live_tokens(steps)
    return build_runner(folder, dtype=dtype, page_size=page, num_pages=mt // page, max_rows=max_rows)


CUTS = {
    "whole": tu.trace_whole,
    "tail32": tu.trace_tail_decode,
    "portions": tu.trace_chunks,
    "mixed": tu.trace_mixed,
}


@pytest.mark.parametrize("dtype", list(ACT))
@pytest.mark.parametrize("name", list(tu.TINY))
@pytest.mark.parametrize("cut", list(CUTS))
def test_every_way_of_cutting_gives_the_plain_logits(folders, name, dtype, cut):
    folder, tensors = folders[name, dtype]
    seqs = sequences(name)
    steps = CUTS[cut](seqs)
    if cut == "portions":
        assert min(len(e["tokens"]) for s in steps for e in s["entries"]) == 2
    if cut == "mixed":
        assert max(len(s["entries"]) for s in steps) == 4
        assert any(len({len(e["tokens"]) > 1 for e in s["entries"]}) == 2 for s in steps)   # portion beside a decode
    runner = runner_for(folder, name, dtype, steps)
    routed = None
    if dtype == "bfloat16":
        got, routed = tu.run_trace_runner(runner, steps, capture=True)
    else:
        got = tu.run_trace_runner(runner, steps)
        if cut in ("tail32", "mixed"):
            assert runner.graph_replays > 0        # single-token steps replay CUDA graphs
    assert len(got) == sum(len(t) for t in seqs.values())
    ref = reference(name, dtype, tensors, seqs, routed)
    tu.compare_in_dtype(got, ref, dtype, what=f"{name} {dtype} {cut}")
    pool = runner.cache.groups[0].pool
    assert pool.free == pool.num_pages and pool.reused_total > 0      # everything came back; pages were reused
    runner.cache.check()


def random_configuration(rng) -> dict:
    """Sizes drawn at random from what the architecture allows: head sizes in steps of 16, any
    number of heads and groups, widths and vocabularies that are no power of two."""
    d = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128]))
    hkv, group = int(rng.randint(1, 5)), int(rng.randint(1, 7))
    rot = min(int(rng.choice([2, 4, 8, 16, d // 2, d])), d)
    experts = int(rng.randint(2, 10))
    cfg = dict(plain_m2.TINY_A)
    cfg.update(num_hidden_layers=int(rng.randint(1, 4)), hidden_size=int(rng.choice([24, 40, 50, 64, 72, 75, 96, 100, 136, 200])),
               num_attention_heads=hkv * group, num_key_value_heads=hkv, head_dim=d, rotary_dim=rot - rot % 2,
               rope_theta=float(rng.choice([1e4, 5e4, 1e6, 5e6])), rms_norm_eps=float(rng.choice([1e-6, 1e-5, 3e-6])),
               num_local_experts=experts, num_experts_per_tok=int(rng.randint(1, experts + 1)),
               intermediate_size=int(rng.choice([16, 24, 40, 52, 64, 72])), vocab_size=int(rng.randint(40, 500)),
               max_position_embeddings=4096)
    return cfg


@pytest.mark.parametrize("seed", list(range(8)))
def test_random_configurations_in_32_bit(seed, tmp_path):
    """Eight configurations drawn at random, each with a random schedule, in 32-bit (where the
    comparison is tight enough to show a kernel that mishandles a size)."""
    rng = np.random.RandomState(5000 + seed)
    cfg = random_configuration(rng)
    name = f"random{seed}"
    tu.TINY[name] = (cfg, 100 + seed, float(rng.choice([0.02, 0.05, 0.1])), 0.05, 0.05, int(rng.choice([4, 8, 16, 32])))
    try:
        tensors = tu.make_model_folder(str(tmp_path), name, "float32")
        lens = [int(x) for x in rng.randint(2, 120, size=5)]
        seqs = {f"s{i}": tu.random_prompt(cfg["vocab_size"], m, 7 * seed + i) for i, m in enumerate(lens)}
        steps = tu.trace_random(seqs, seed)
        runner = runner_for(str(tmp_path), name, "float32", steps)
        got = tu.run_trace_runner(runner, steps)
        ref = reference(name, "float32", tensors, seqs)
        tu.compare_in_dtype(got, ref, "float32", what=f"{cfg}")
        runner.cache.check()
    finally:
        del tu.TINY[name]


@pytest.mark.parametrize("dtype", list(ACT))
@pytest.mark.parametrize("name", ["A", "D"])
@pytest.mark.parametrize("seed", [3, 11, 12])
def test_random_schedules_give_the_plain_logits(folders, name, dtype, seed):
    """Random request lengths, random cuts, random subsets of the live requests in a step and
    random places asked for, with a pool exactly as large as the schedule needs."""
    folder, tensors = folders[name, dtype]
    rng = np.random.RandomState(seed)
    vocab = tu.TINY[name][0]["vocab_size"]
    lens = [int(x) for x in rng.randint(2, 160, size=rng.randint(4, 9))]
    seqs = {f"s{i}": tu.random_prompt(vocab, n, 31 * seed + i) for i, n in enumerate(lens)}
    steps = tu.trace_random(seqs, seed)
    runner = runner_for(folder, name, dtype, steps)
    routed = None
    if dtype == "bfloat16":
        got, routed = tu.run_trace_runner(runner, steps, capture=True)
    else:
        got = tu.run_trace_runner(runner, steps)
    assert len(got) == sum(len(e["want"]) for s in steps for e in s["entries"])
    ref = reference(name, dtype, tensors, seqs, routed)
    tu.compare_in_dtype(got, ref, dtype, what=f"{name} {dtype} random schedule {seed}")
    pool = runner.cache.groups[0].pool
    assert pool.free == pool.num_pages
    runner.cache.check()


@pytest.mark.parametrize("dtype", list(ACT))
@pytest.mark.parametrize("name", ["D", "E"])
def test_long_portions_through_the_tensor_core_attention(folders, name, dtype):
    """Portions of more than 512 tokens take the prompt-portion attention kernels (tcgen05 for
    head size 128, m16n8k16 tiles for 64; in 32-bit the plain kernel), shorter ones and single
    tokens the split-key kernel: a 1,500-token request in portions of 700, 600 and 200, a
    second request whose 650-token portion shares a step with a decoded token of the first,
    then both decode side by side."""
    folder, tensors = folders[name, dtype]
    vocab = tu.TINY[name][0]["vocab_size"]
    a, b = tu.random_prompt(vocab, 1510, 71), tu.random_prompt(vocab, 659, 72)
    seqs = {"a": a, "b": b}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:700], "want": [0, 1, 350, 699]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[700:1300], "want": [0, 599]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[1300:1500], "want": [0, 100, 199]}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": a[1500:1501], "want": [0]},
                                {"id": "b", "tokens": b[:650], "want": [0, 649]}], "end": []},
    ]
    for i in range(9):
        steps.append({"step": 4 + i, "entries": [{"id": "a", "tokens": [a[1501 + i]], "want": [0]},
                                                  {"id": "b", "tokens": [b[650 + i]], "want": [0]}], "end": []})
    steps[-1]["end"] = ["a", "b"]
    from sparseengine_b200.csrc import ops
    runner = runner_for(folder, name, dtype, steps)
    before = dict(ops.calls)
    routed = None
    if dtype == "bfloat16":
        got, routed = tu.run_trace_runner(runner, steps, capture=True)
    else:
        got = tu.run_trace_runner(runner, steps)
    took = {k for k, v in ops.calls.items() if v > before.get(k, 0)}
    if dtype == "bfloat16":
        assert ("se_attn_prefill_tc" if name == "D" else "se_attn_prefill") in took and "se_attn_decode" in took
        assert "se_moe_grouped_gemm_tc" in took and "se_paged_attention_plain" not in took
    else:
        assert "se_paged_attention_plain" in took and "se_moe_grouped_gemm_plain" in took
    ref = reference(name, dtype, tensors, seqs, routed)
    tu.compare_in_dtype(got, ref, dtype, what=f"{name} {dtype} long portions")
    assert len(got) == 4 + 2 + 3 + 1 + 2 + 18
    ops.error_check("cuda:0")


@pytest.mark.parametrize("dtype", list(ACT))
def test_cuts_agree_with_each_other_more_tightly_than_with_the_plain(folders, dtype):
    """The same request through different cuts and page sets: the logits differ by
    rounding only (in 32-bit: a few ulp of the order of sums)."""
    folder, tensors = folders["B", dtype]
    seqs = sequences("B", [41])
    upto = 41
    if dtype == "bfloat16":     # compare up to the first near-tie of a router; take a prompt where that is late
        cands = [tu.random_prompt(384, 41, s) for s in range(200, 230)]
        ties = [first_near_tie("B", dtype, tensors, c) for c in cands]
        upto = max(ties)
        seqs = {"r0": cands[ties.index(upto)]}
    assert upto >= 8
    base = None
    for cut in CUTS:
        steps = CUTS[cut](seqs)
        got = tu.run_trace_runner(runner_for(folder, "B", dtype, steps), steps)
        arr = np.stack([got["r0", p] for p in range(upto)])
        if base is None:
            base = arr
        else:
            tol = 5e-6 if dtype == "float32" else 2e-2
            assert np.abs(arr - base).max() <= tol, cut


@pytest.mark.parametrize("dtype", list(ACT))
def test_long_decoding_and_first_tokens(folders, dtype):
    """One prompt token, then 200 tokens one by one (crossing many page edges); the
    first positions of a sequence are compared on their own."""
    folder, tensors = folders["A", dtype]
    toks = tu.random_prompt(256, 201, 99)
    steps = [{"step": i, "entries": [{"id": "d", "tokens": [t], "want": [0]}], "end": ["d"] if i == 200 else []}
             for i, t in enumerate(toks)]
    routed = None
    if dtype == "bfloat16":
        got, routed = tu.run_trace_runner(runner_for(folder, "A", dtype, steps), steps, capture=True)
    else:
        got = tu.run_trace_runner(runner_for(folder, "A", dtype, steps), steps)
    ref = reference("A", dtype, tensors, {"d": toks}, routed)
    tu.compare_in_dtype({k: v for k, v in got.items() if k[1] < 3}, ref, dtype, what="first tokens")
    tu.compare_in_dtype(got, ref, dtype, what="long decoding")


def test_out_of_pages_changes_nothing(folders):
    from sparseengine_b200.cache.pages import OutOfPages
    from sparseengine_b200.engine.factory import build_runner
    from sparseengine_b200.engine.runner import StepEntry
    folder, tensors = folders["A", "float32"]
    r = build_runner(folder, dtype="float32", page_size=4, num_pages=3, max_rows=2)
    r.admit("a"), r.admit("b")
    r.step([StepEntry("a", [1, 2, 3, 4, 5], [])])
    with pytest.raises(OutOfPages):
        r.step([StepEntry("a", [6], [0]), StepEntry("b", [1] * 9, [])])     # b needs 3 pages, 1 is free
    assert r.cache.free_pages() == 1 and r.cache.length("a") == 5 and r.cache.length("b") == 0
    out = r.step([StepEntry("a", [6], [0])])
    ref = plain_m2.forward(plain_m2.TINY_A, tensors, [1, 2, 3, 4, 5, 6]).numpy()
    assert np.abs(out.float().cpu().numpy()[0] - ref[5]).max() < 1e-5
    with pytest.raises(ValueError):
        r.step([StepEntry("a", [256], [0])])          # token id outside the vocabulary
    with pytest.raises(ValueError):
        r.step([StepEntry("zz", [1], [0])])           # not admitted


@pytest.mark.parametrize("dtype", list(ACT))
def test_trace_run_program(folders, dtype, tmp_path):
    """The command-line program: the line protocol, the files it writes, a request left
    out of steps, steps in which nothing is wanted."""
    folder, tensors = folders["B", dtype]
    seqs = sequences("B", [23, 31, 7, 16, 1, 40])
    steps = tu.trace_mixed(seqs, seed=3)
    for s in steps[::3]:                                # some steps want nothing from their first entry
        s["entries"][0]["want"] = []
    got = tu.run_trace_cli(folder, dtype, steps, str(tmp_path / "out"), tu.max_live_tokens(steps))
    assert got
    if dtype == "bfloat16":
        # the program cannot tell which experts it chose: compare up to each request's first near-tie
        upto = {sid: first_near_tie("B", dtype, tensors, toks) for sid, toks in seqs.items()}
        kept = {k: v for k, v in got.items() if k[1] < upto[k[0]]}
        assert len(kept) >= 5
        got = kept
    tu.compare_in_dtype(got, reference("B", dtype, tensors, seqs), dtype, what=f"trace_run {dtype}")


@pytest.mark.parametrize("dtype", list(ACT))
def test_decode_graphs_give_what_single_launches_give(folders, dtype):
    """Decode steps replayed as CUDA graphs against the same steps launch by launch: batch
    sizes 1..4, requests joining and leaving, block-table updates inside the graph."""
    from sparseengine_b200.engine.factory import build_runner
    folder, _ = folders["C", dtype]
    seqs = sequences("C", [40, 55, 33, 47])
    steps = tu.trace_mixed(seqs, chunk=7, decode_tail=30, seed=5)
    results = []
    for graphs in (True, False):
        r = build_runner(folder, dtype=dtype, page_size=16, num_pages=tu.max_live_tokens(steps) // 16, max_rows=4)
        r.decode_graphs = graphs
        results.append(tu.run_trace_runner(r, steps))
        assert (r.graph_replays > 20) == graphs
    a, b = results
    assert a.keys() == b.keys()
    for k in a:
        assert np.array_equal(a[k], b[k]), k        # same kernels, same plans at these lengths: bit-equal


def test_decode_graphs_are_kept_up_to_a_limit(folders):
    """Graphs are captured per (batch size, context bucket); the least recently used are dropped."""
    from sparseengine_b200.engine.runner import StepEntry
    folder, _ = folders["A", "float32"]
    from sparseengine_b200.engine.factory import build_runner
    runner = build_runner(folder, dtype="float32", page_size=4, num_pages=64, max_rows=4)
    runner.MAX_GRAPHS, runner.KV_BUCKET = 3, 4
    runner.admit("a")
    outs = []
    for i in range(30):
        outs.append(runner.step([StepEntry("a", [i % 7], [0])]).float().cpu())
        assert len(runner._graphs) <= 3
    assert runner.graph_replays > 10
    plain = build_runner(folder, dtype="float32", page_size=4, num_pages=64, max_rows=4, decode_graphs=False)
    plain.admit("a")
    for i in range(30):
        ref = plain.step([StepEntry("a", [i % 7], [0])]).float().cpu()
        assert (outs[i] - ref).abs().max() < 1e-5
