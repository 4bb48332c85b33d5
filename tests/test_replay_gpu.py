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
# 32-bit: only the order of sums differs.  bfloat16: logits are bfloat16 values (8 bits of
# mantissa) behind several layers of bfloat16 activations.
TOL = {"float32": (1e-5, 1e-5), "bfloat16": (2e-2, 2e-2)}
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


def reference(name, dtype, tensors, seqs):
    cfg = tu.TINY[name][0]
    out = {}
    for sid, toks in seqs.items():
        key = (name, dtype, tuple(toks))
        if key not in _REF:
            _REF[key] = plain_m2.forward(cfg, tensors, toks, ACT[dtype]).numpy()
        out[sid] = _REF[key]
    return out


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
    got = tu.run_trace_runner(runner, steps)
    assert len(got) == sum(len(t) for t in seqs.values())
    tu.compare(got, reference(name, dtype, tensors, seqs), *TOL[dtype], what=f"{name} {dtype} {cut}")
    pool = runner.cache.groups[0].pool
    assert pool.free == pool.num_pages and pool.reused_total > 0      # everything came back; pages were reused
    runner.cache.check()


@pytest.mark.parametrize("dtype", list(ACT))
def test_cuts_agree_with_each_other_more_tightly_than_with_the_plain(folders, dtype):
    """The same request through different cuts and page sets: the logits differ by
    rounding only (in 32-bit: a few ulp of the order of sums)."""
    folder, _ = folders["B", dtype]
    seqs = sequences("B", [41])
    base = None
    for cut in CUTS:
        steps = CUTS[cut](seqs)
        got = tu.run_trace_runner(runner_for(folder, "B", dtype, steps), steps)
        arr = np.stack([got["r0", p] for p in range(41)])
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
    got = tu.run_trace_runner(runner_for(folder, "A", dtype, steps), steps)
    ref = reference("A", dtype, tensors, {"d": toks})
    tu.compare({k: v for k, v in got.items() if k[1] < 3}, ref, *TOL[dtype], what="first tokens")
    tu.compare(got, ref, *TOL[dtype], what="long decoding")


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
    tu.compare(got, reference("B", dtype, tensors, seqs), *TOL[dtype], what=f"trace_run {dtype}")
