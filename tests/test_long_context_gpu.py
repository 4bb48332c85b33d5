"""Long contexts: block tables of more than 8,192 pages (131,072 tokens in pages of 16), the
split of decode attention over the keys, and prompt portions behind a long cached prefix.

Random keys at such a length make attention nearly uniform, which would hide a skipped page
or a split that reads the wrong range, so the kernel tests put one dominating key at chosen
places (first and last page, both sides of a split's edge, the middle).  The engine test feeds
one 131,112-token prompt through the step function in two different ways of cutting it and
compares the last positions, and both with a 32-bit run.

The reference's mechanisms for this case: prompts cut into chunks
(src/sparseengine/engine/scheduler.py:269-297) and decode attention split over the keys
(src/sparseengine/kernels/triton/gqa_flash_decoding_stage1.py:330-393)."""
import numpy as np
import pytest
import torch

import plain_m2
import trace_util as tu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 16
CONTEXT = 131072


def _scattered_table(n_tokens: int, seed: int = 3):
    pages = -(-n_tokens // PAGE)
    perm = torch.randperm(pages + 5, generator=torch.Generator().manual_seed(seed))[:pages]
    table = torch.full((2, pages + 2), -1, dtype=torch.int32)
    table[1, :pages] = perm.int()
    return table.to(DEV), pages + 5


@pytest.mark.parametrize("kernel", ["decode", "prefill_tcgen05", "prefill_mma_sync"])
def test_a_far_key_is_found_behind_8192_pages(kernel):
    from sparseengine_b200.csrc import ops
    hq, hkv, d = 8, 2, 128
    n = CONTEXT + 72
    dtype = torch.bfloat16
    table, num_pages = _scattered_table(n)
    assert table.shape[1] > 8192
    rows = torch.ones(1, dtype=torch.int32, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(5)
    k = (torch.randn(n, hkv, d, generator=g, device=DEV) * 0.1).to(dtype)
    v = torch.randn(n, hkv, d, generator=g, device=DEV).to(dtype)
    q_len = 1 if kernel == "decode" else 200
    q = (torch.randn(q_len, hq, d, generator=g, device=DEV) * 0.1).to(dtype)
    cache = torch.zeros(num_pages, 2, hkv, PAGE, d, dtype=dtype, device=DEV)
    pos = torch.arange(n, device=DEV)
    pg = table[1, (pos // PAGE).long()].long()
    cache[pg, 1, :, (pos % PAGE).long()] = v
    group = hq // hkv
    last = n - 1
    splits, per = ops.attn_decode_plan(1, hq, hkv, n)
    assert splits > 8                                       # the keys of one token are spread over many CTAs
    places = [0, 15, 16, per - 1, per, 3 * per - 1, 3 * per, 65536, CONTEXT - 1, CONTEXT, last - 64, last - 1, last]
    for far in places:
        kk = k.clone()
        kk[far] = (q[-1, ::group].float() * 400.0).to(dtype)    # dominates the last query's scores
        cache[pg, 0, :, (pos % PAGE).long()] = kk
        out = torch.zeros_like(q)
        kw = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=PAGE, scale=d ** -0.5)
        if kernel == "decode":
            ops.attn_decode(q.view(1, -1), cache, table, rows, torch.zeros(1, dtype=torch.int32, device=DEV),
                            torch.tensor([last], dtype=torch.int32, device=DEV), out.view(1, -1), max_keys=n, **kw)
        else:
            fn = ops.attn_prefill_tc if kernel == "prefill_tcgen05" else ops.attn_prefill
            fn(q.view(q_len, -1), cache, table, rows, torch.tensor([0, q_len], dtype=torch.int32, device=DEV),
               torch.tensor([n], dtype=torch.int32, device=DEV), out.view(q_len, -1), entries=1, max_q_len=q_len, **kw)
        ops.error_check(DEV)
        got = out[-1].float()
        for h in range(hkv):
            assert torch.allclose(got[h * group], v[far, h].float(), atol=3e-2), (kernel, far, h)
    # and without a dominating key, with scores spread enough (standard deviation 3) that a few
    # hundred keys anywhere in the context carry the output: the last query against a 32-bit
    # softmax over all keys
    k2, q2 = (k.float() * 10).to(dtype), (q.float() * 30).to(dtype)
    cache[pg, 0, :, (pos % PAGE).long()] = k2
    out = torch.zeros_like(q)
    if kernel == "decode":
        ops.attn_decode(q2.view(1, -1), cache, table, rows, torch.zeros(1, dtype=torch.int32, device=DEV),
                        torch.tensor([last], dtype=torch.int32, device=DEV), out.view(1, -1), max_keys=n, **kw)
    else:
        fn(q2.view(q_len, -1), cache, table, rows, torch.tensor([0, q_len], dtype=torch.int32, device=DEV),
           torch.tensor([n], dtype=torch.int32, device=DEV), out.view(q_len, -1), entries=1, max_q_len=q_len, **kw)
    ops.error_check(DEV)
    ref = torch.stack([torch.softmax((k2[:, h // group].float() @ q2[-1, h].float()) * d ** -0.5, 0)
                       @ v[:, h // group].float() for h in range(hq)])
    rms = float(ref.pow(2).mean().sqrt())
    assert rms > 0.02
    assert (out[-1].float() - ref).abs().max() <= 0.03 * rms + 2.0 ** -7 * float(ref.abs().max()), kernel


LONG = dict(plain_m2.TINY_D, max_position_embeddings=CONTEXT + 1024)


@pytest.fixture(scope="module")
def long_folder(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("long"))
    tu.TINY["LONG"] = (LONG, 3, 0.04, 0.05, 0.05, PAGE)
    try:
        tu.make_model_folder(d, "LONG", "bfloat16")
    finally:
        del tu.TINY["LONG"]
    return d


def _run(folder, dtype, portion, prompt, tail):
    """The prompt in portions of ``portion`` tokens, then ``tail`` tokens one per step; logits of
    the prompt's last position and of every single-token step."""
    from sparseengine_b200.csrc import ops
    from sparseengine_b200.engine.factory import build_runner
    from sparseengine_b200.engine.runner import StepEntry
    total = len(prompt)
    runner = build_runner(folder, dtype=dtype, page_size=PAGE, num_pages=-(-total // PAGE) + 2, max_rows=2)
    runner.admit("r")
    head = total - tail
    rows = []
    for a in range(0, head, portion):
        b = min(head, a + portion)
        out = runner.step([StepEntry("r", prompt[a:b], [b - a - 1] if b == head else [])])
    rows.append(out.float().cpu())
    before = dict(ops.calls)
    for i in range(head, total):
        rows.append(runner.step([StepEntry("r", [prompt[i]], [0])]).float().cpu())
    ops.error_check(DEV)
    took = {k for k, v in ops.calls.items() if v > before.get(k, 0)}
    table_pages = int((runner.cache.groups[0].table_host[runner.cache.row("r")] >= 0).sum())
    runner.release("r")
    runner.cache.check()
    return torch.cat(rows).numpy(), took, table_pages


def test_131072_tokens_in_portions_then_decoding(long_folder):
    vocab = LONG["vocab_size"]
    prompt = tu.random_prompt(vocab, CONTEXT + 40, 77)
    tail = 24
    a, took, pages = _run(long_folder, "bfloat16", 8192, prompt, tail)
    assert pages > 8192 and "se_attn_decode" in took            # a block table of more than 8,192 pages, split over the keys
    b, _, _ = _run(long_folder, "bfloat16", 5000, prompt, tail)
    c, took32, _ = _run(long_folder, "float32", 8192, prompt, tail)
    assert "se_paged_attention_plain" in took32
    assert a.shape == (tail + 1, vocab) and np.isfinite(a).all()
    rms = float(np.sqrt(np.mean(c.astype(np.float64) ** 2)))
    # two ways of cutting, same precision: rounding only (a share of the logits' root mean square,
    # as for every bfloat16 comparison); against the 32-bit run: the same bound
    for name, x, y in (("8192 vs 5000", a, b), ("bfloat16 vs float32", a, c)):
        worst = float(np.abs(x - y).max())
        print(f"[long context] {name}: logits rms {rms:.4f}, worst |diff| {worst:.3e} = {worst / rms:.4f} rms")
        assert (np.abs(x - y) <= tu.BF16_SHARE_OF_RMS * rms + tu.BF16_ULP * np.abs(y)).all(), name


@pytest.mark.parametrize("starts", [[CONTEXT - 7], [CONTEXT - 7, 40_000, 77]])
def test_replayed_decode_steps_equal_launched_ones_at_far_positions(long_folder, starts):
    """Decode steps replayed from a CUDA graph run their kernels back to back, and several of them
    start as dependents of the kernel before them (their set-up overlaps its end); launched one
    by one from Python they never overlap.  Both must give the same bits.  Far positions make the
    rotation angles slow to compute, which widens the window in which a kernel that did not
    wait for its input would read the previous step's."""
    from sparseengine_b200.engine.factory import build_runner
    from sparseengine_b200.engine.runner import StepEntry
    vocab = LONG["vocab_size"]
    outs = {}
    for graphs in (False, True):
        runner = build_runner(long_folder, dtype="bfloat16", page_size=PAGE,
                              num_pages=sum(-(-(s + 40) // PAGE) for s in starts) + 4, max_rows=4, decode_graphs=graphs)
        for i, s in enumerate(starts):          # requests that hold that many tokens without having run them
            runner.admit(i)
            runner.cache.reserve(i, s)
            runner.cache.commit(i, s)
        g = torch.Generator(device=DEV).manual_seed(11)
        for slot in runner.slots:               # random keys and values, the same in both runs
            slot.kv.copy_(torch.randn(slot.kv.shape, generator=g, device=DEV) * 0.5)
        rows = []
        for step in range(24):
            entries = [StepEntry(i, [(31 * step + 7 * i) % vocab], [0]) for i in range(len(starts))]
            rows.append(runner.step(entries).float().cpu())
        outs[graphs] = torch.stack(rows)
        assert (runner.graph_replays > 0) == graphs
    assert torch.isfinite(outs[True]).all()
    assert torch.equal(outs[False], outs[True])
