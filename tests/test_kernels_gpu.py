"""Each kernel alone against a plain PyTorch float32 reference of the same op, at sizes
other than the tiny models': widths and vocabularies that are no power of two, head
sizes in steps of 16, odd head and group counts."""
import math

import numpy as np
import pytest
import torch

import plain_m2

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, f32=1e-5, bf16=2e-2):
    return dict(atol=f32, rtol=f32) if dtype == torch.float32 else dict(atol=bf16, rtol=bf16)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 3072, 5000])
def test_embed_and_gather(dtype, hidden):
    from sparseengine_b200.csrc import ops
    table = rnd(301, hidden, dtype=dtype)
    ids = torch.tensor([0, 300, 7, 7, 150], dtype=torch.int32, device=DEV)
    out = torch.empty(5, hidden, dtype=dtype, device=DEV)
    ops.embed_gather(table, ids, out)
    assert torch.equal(out, table[ids.long()])
    g = torch.empty(3, hidden, dtype=dtype, device=DEV)
    ops.gather_rows(out, torch.tensor([4, 0, 2], dtype=torch.int32, device=DEV), g)
    assert torch.equal(g, out[[4, 0, 2]])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,eps", [(1, 64, 1e-6), (7, 3072, 1e-5), (33, 1000, 1e-6), (3, 20000, 1e-6),
                                             (2, 12288, 1e-6)])      # the last: a row of exactly 48 KB
def test_rmsnorm_with_and_without_residual(dtype, rows, hidden, eps):
    from sparseengine_b200.csrc import ops
    x, r = rnd(rows, hidden, dtype=dtype, seed=1), rnd(rows, hidden, dtype=dtype, scale=3.0, seed=2)
    w = (1 + 0.1 * rnd(hidden, seed=3)).to(dtype)
    y = torch.empty_like(x)
    ops.rmsnorm(x, w, eps, y)
    ref = plain_m2.rms_norm(x.float().cpu(), w.float().cpu(), eps, dtype)
    torch.testing.assert_close(y.float().cpu(), ref, **tol(dtype, 2e-6, 1e-2))
    y2, r2 = torch.empty_like(x), torch.empty_like(x)
    ops.rmsnorm(x, w, eps, y2, residual=r, residual_out=r2)
    ref_y, ref_r = plain_m2.add_rms_norm(x.float().cpu(), r.float().cpu(), w.float().cpu(), eps, dtype)
    assert torch.equal(r2.float().cpu(), ref_r)                  # the residual is the rounded 32-bit sum, exactly
    torch.testing.assert_close(y2.float().cpu(), ref_y, **tol(dtype, 2e-6, 1e-2))


def _cache_setup(tokens_per_seq, hkv, d, page, dtype, firsts=None):
    """Block tables with scattered pages for positions firsts[i] .. firsts[i]+tokens-1 of
    each request; returns metadata tensors for a step that brings all of those tokens."""
    n = len(tokens_per_seq)
    firsts = firsts or [0] * n
    need = [range(f // page, (f + t - 1) // page + 1) for f, t in zip(firsts, tokens_per_seq)]
    total = sum(len(r) for r in need) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(5)).tolist()
    width = max(r.stop for r in need) + 1
    table = torch.full((n + 2, width), -1, dtype=torch.int32)
    rows = [i + 1 for i in range(n)]
    k = 0
    for i, r in enumerate(need):
        for j in r:
            table[rows[i], j] = perm[k]
            k += 1
    positions = torch.cat([torch.arange(f, f + t) for f, t in zip(firsts, tokens_per_seq)]).int()
    token_seq = torch.cat([torch.full((t,), i) for i, t in enumerate(tokens_per_seq)]).int()
    cache = torch.zeros(total, 2, hkv, page, d, dtype=dtype, device=DEV)
    return (table.to(DEV), torch.tensor(rows, dtype=torch.int32, device=DEV), positions.to(DEV), token_seq.to(DEV),
            cache)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,rot,page,theta,norm", [
    (4, 2, 16, 8, 4, 1e4, True), (6, 3, 32, 32, 8, 1e6, True), (5, 1, 48, 16, 16, 5e4, True),
    (7, 7, 80, 0, 3, 1e4, False), (3, 1, 32, 16, 8, 1e4, False), (48, 8, 128, 64, 16, 5e6, True)])
@pytest.mark.parametrize("lens", [[5, 1, 19], [70, 1, 40]], ids=["few_tokens", "many_tokens"])
def test_qk_prep_norm_rotary_and_cache_write(dtype, hq, hkv, d, rot, page, theta, norm, lens):
    """Few tokens take the kernel with a block per head, many tokens the two-pass kernels
    (16-byte groups where the sizes allow it, element by element otherwise)."""
    from sparseengine_b200.csrc import ops
    t = sum(lens)
    # one request sits at large positions (large rotation angles, a far table index)
    table, rows, positions, token_seq, cache = _cache_setup(lens, hkv, d, page, dtype, firsts=[0, 3, 1000])
    qkv = rnd(t, (hq + 2 * hkv) * d, dtype=dtype, scale=2.0, seed=4)
    qw = (1 + 0.1 * rnd(hq * d, seed=5)).to(dtype) if norm else None
    kw = (1 + 0.1 * rnd(hkv * d, seed=6)).to(dtype) if norm else None
    inv = plain_m2.rope_inv_freq(rot, theta).to(DEV) if rot else None
    q_out = torch.empty(t, hq * d, dtype=dtype, device=DEV)
    ops.qk_prep(qkv, qw, kw, inv, positions, token_seq, rows, table, cache, q_out, num_heads=hq, num_kv_heads=hkv,
                head_dim=d, rotary_dim=rot, eps=1e-5, rope_scale=1.0, page_size=page)
    c = qkv.float().cpu()
    q, k, v = c[:, :hq * d], c[:, hq * d:(hq + hkv) * d], c[:, (hq + hkv) * d:]
    if norm:
        q = plain_m2.whole_projection_rms_norm(q, qw.float().cpu(), 1e-5, dtype)
        k = plain_m2.whole_projection_rms_norm(k, kw.float().cpu(), 1e-5, dtype)
    q, k = q.view(t, hq, d), k.view(t, hkv, d)
    if rot:
        q = plain_m2.partial_rotary(q, positions.cpu(), rot, theta, dtype)
        k = plain_m2.partial_rotary(k, positions.cpu(), rot, theta, dtype)
    # large angles: the device's sincosf and the host's cos/sin agree to an ulp of the angle
    torch.testing.assert_close(q_out.float().cpu().view(t, hq, d), q, **tol(dtype, 3e-5, 2e-2))
    if rot < d and not norm:
        assert torch.equal(q_out.float().cpu().view(t, hq, d)[..., rot:], q[..., rot:])     # pass-through is exact
    cc = cache.float().cpu()
    for i in range(t):
        p = int(positions[i])
        page_id = int(table[int(rows[int(token_seq[i])]), p // page])
        torch.testing.assert_close(cc[page_id, 0, :, p % page], k[i], **tol(dtype, 3e-5, 2e-2))
        assert torch.equal(cc[page_id, 1, :, p % page], v[i].view(hkv, d))


def _attention_reference(q, k, v, lens, starts, dtype, window):
    outs = []
    a = 0
    for n, s in zip(lens, starts):
        qs = torch.zeros(s + n, q.shape[1], q.shape[2])
        qs[s:] = q[a:a + n]
        outs.append(plain_m2.causal_attention(qs, k[len(outs)], v[len(outs)], dtype, window)[s:])
        a += n
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page,window", [
    (4, 2, 16, 4, None), (6, 3, 32, 8, None), (5, 1, 48, 16, None), (9, 3, 80, 5, 7), (12, 2, 128, 16, None),
    (2, 2, 256, 32, 20)])
def test_paged_attention_plain(dtype, hq, hkv, d, page, window):
    """Queries are the last q_len positions of each request; earlier keys come from pages
    written before (scattered page order)."""
    from sparseengine_b200.csrc import ops
    kv_lens, q_lens = [37, 1, 64, 130], [5, 1, 1, 33]
    starts = [kv - ql for kv, ql in zip(kv_lens, q_lens)]
    table, rows, _, _, cache = _cache_setup(kv_lens, hkv, d, page, dtype)
    ks = [rnd(n, hkv, d, dtype=dtype, seed=20 + i).cpu() for i, n in enumerate(kv_lens)]
    vs = [rnd(n, hkv, d, dtype=dtype, seed=30 + i).cpu() for i, n in enumerate(kv_lens)]
    for i, n in enumerate(kv_lens):
        for p in range(n):
            pg = int(table[int(rows[i]), p // page])
            cache[pg, 0, :, p % page] = ks[i][p].to(DEV)
            cache[pg, 1, :, p % page] = vs[i][p].to(DEV)
    t = sum(q_lens)
    q = rnd(t, hq, d, dtype=dtype, seed=7)
    positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, q_lens)]).int().to(DEV)
    token_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).int().to(DEV)
    out = torch.empty_like(q)
    ops.paged_attention_plain(q.view(t, hq * d), cache, table, rows, token_seq, positions, out.view(t, hq * d),
                              num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5,
                              window=window)
    ref = _attention_reference(q.float().cpu(), [k.float() for k in ks], [v.float() for v in vs], q_lens, starts,
                               dtype, window)
    torch.testing.assert_close(out.float().cpu(), ref, **tol(dtype, 2e-5, 2e-2))


def test_attention_finds_a_far_key_among_hundreds():
    """One key far back is made to dominate: the output must be its value, whatever page
    it lies on (first slot of a page, last slot, first page)."""
    from sparseengine_b200.csrc import ops
    hq, hkv, d, page, n = 4, 2, 32, 8, 700
    for far in (0, 7, 8, 15, 343, 696):
        table, rows, _, _, cache = _cache_setup([n], hkv, d, page, torch.float32)
        k = rnd(n, hkv, d, scale=0.1, seed=1).cpu()
        v = rnd(n, hkv, d, seed=2).cpu()
        q = rnd(1, hq, d, scale=0.1, seed=3)
        k[far] = q.cpu()[0, ::2] * 400.0               # kv head g gets query head 2g's direction, scaled up
        for p in range(n):
            pg = int(table[1, p // page])
            cache[pg, 0, :, p % page] = k[p].to(DEV)
            cache[pg, 1, :, p % page] = v[p].to(DEV)
        out = torch.empty_like(q)
        ops.paged_attention_plain(q.view(1, -1), cache, table, rows, torch.zeros(1, dtype=torch.int32, device=DEV),
                                  torch.tensor([n - 1], dtype=torch.int32, device=DEV), out.view(1, -1),
                                  num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5)
        got = out.cpu()[0]
        assert torch.allclose(got[0], v[far, 0], atol=1e-3) and torch.allclose(got[2], v[far, 1], atol=1e-3), far
        ref = plain_m2.causal_attention(torch.cat([torch.zeros(n - 1, hq, d), q.cpu()]), k, v, torch.float32)[-1]
        torch.testing.assert_close(got, ref, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,hidden,experts,top_k,bias", [
    (5, 64, 4, 2, False), (9, 96, 8, 3, True), (700, 80, 6, 4, True), (3, 3072, 256, 8, True), (1, 200, 37, 5, True),
    (4, 3072, 256, 8, True)])      # the last: its staged tokens are exactly 48 KB of shared memory
def test_router(dtype, tokens, hidden, experts, top_k, bias):
    from sparseengine_b200.csrc import ops
    x = rnd(tokens, hidden, dtype=dtype, seed=1)
    gate = rnd(experts, hidden, scale=0.2, seed=2)
    b = rnd(experts, scale=0.3, seed=3) if bias else None
    ids = torch.empty(tokens, top_k, dtype=torch.int32, device=DEV)
    w = torch.empty(tokens, top_k, dtype=torch.float32, device=DEV)
    logits = torch.empty(tokens, experts, dtype=torch.float32, device=DEV)
    ops.router(x, gate, b, ids, w, top_k=top_k, logits_out=logits)
    ref_ids, ref_w, ref_logits = plain_m2.router(x.float().cpu(), gate.cpu(),
                                                 b.cpu() if bias else torch.zeros(experts), top_k)
    torch.testing.assert_close(logits.cpu(), ref_logits, atol=2e-5, rtol=2e-5)
    # rows whose k-th and (k+1)-th scores are further apart than the logits' rounding must agree exactly
    score = torch.sigmoid(ref_logits) + (b.cpu() if bias else 0)
    srt = score.sort(-1, descending=True).values
    clear = (srt[:, :-1] - srt[:, 1:]).min(-1).values > 1e-5 if experts > 1 else torch.ones(tokens, dtype=torch.bool)
    assert clear.float().mean() > 0.5
    assert torch.equal(ids.cpu()[clear].long(), ref_ids[clear])
    torch.testing.assert_close(w.cpu()[clear], ref_w[clear], atol=1e-5, rtol=1e-5)


def test_router_logits_do_not_depend_on_the_batch():
    """A token's router logits are bit-equal whether it is routed alone, with seven others
    or with hundreds (the decode and the many-token kernels sum in the same order)."""
    from sparseengine_b200.csrc import ops
    for hidden, experts in ((3072, 256), (200, 37), (77, 5)):
        x = rnd(300, hidden, dtype=torch.bfloat16, seed=1)
        gate = rnd(experts, hidden, scale=0.2, seed=2)
        outs = []
        for sl in (slice(0, 300), slice(0, 8), slice(0, 1), slice(5, 13), slice(7, 8)):
            xs = x[sl].contiguous()
            n = xs.shape[0]
            logits = torch.empty(n, experts, dtype=torch.float32, device=DEV)
            ops.router(xs, gate, None, torch.empty(n, 2, dtype=torch.int32, device=DEV),
                       torch.empty(n, 2, dtype=torch.float32, device=DEV), top_k=2, logits_out=logits)
            outs.append((sl, logits))
        full = outs[0][1]
        for sl, lg in outs[1:]:
            assert torch.equal(lg, full[sl]), (hidden, experts, sl)


@pytest.mark.parametrize("tokens,experts,top_k,kind", [
    (1, 256, 8, "random"), (70, 256, 8, "random"), (9, 37, 5, "random"), (13, 5, 5, "random"), (300, 200, 1, "random"),
    (6, 64, 6, "ties"), (5, 256, 8, "coarse"), (4, 40, 7, "nan")])
def test_router_selection_by_a_warp_equals_selection_by_a_block(tokens, experts, top_k, kind):
    """The two selection kernels give the same experts in the same slots with the same
    weights, bit for bit: on random logits, on logits with many exact ties (where only the tie
    order decides), on coarse logits with ties at the threshold, and with NaN scores."""
    from sparseengine_b200.csrc import ops
    g = torch.Generator().manual_seed(tokens * 1000 + experts)
    logits = torch.randn(tokens, experts, generator=g)
    bias = torch.randn(experts, generator=g) * 0.3
    if kind == "ties":
        logits.zero_()
        bias = torch.tensor([0.0, 0.25, 0.5, 0.25] * (experts // 4))
    elif kind == "coarse":
        logits = (logits * 2).round() / 2
        bias = (bias * 4).round() / 4
    elif kind == "nan":
        bias[3] = float("nan")
        logits[1, 7] = float("nan")
    logits, bias = logits.to(DEV), bias.to(DEV)
    out = {}
    for impl in ("block", "warp", "auto"):
        ids = torch.full((tokens, top_k), -1, dtype=torch.int32, device=DEV)
        w = torch.full((tokens, top_k), -1.0, dtype=torch.float32, device=DEV)
        ops.router_select(logits, bias, ids, w, top_k=top_k, routed_scale=1.25, impl=impl)
        out[impl] = (ids.cpu(), w.cpu())
    assert torch.equal(out["warp"][0], out["block"][0]) and torch.equal(out["auto"][0], out["block"][0])
    same = (out["warp"][1] == out["block"][1]) | (out["warp"][1].isnan() & out["block"][1].isnan())
    assert bool(same.all())
    assert int(out["block"][0].min()) >= 0 and all(len(set(r)) == top_k for r in out["block"][0].tolist())
    # logits that arrive in parts [chunks, tokens, terms, experts] are added inside the kernels, chunk by
    # chunk and term by term: the same choice and weights as from the sums taken in that order beforehand
    parts = torch.randn(3, tokens, 2, experts, generator=g).to(DEV)
    summed = torch.zeros(tokens, experts, device=DEV)
    for c in range(3):
        for k in range(2):
            summed = summed + parts[c, :, k]
    for impl in ("block", "warp"):
        got, want = [], []
        for src, dst in ((parts, got), (summed, want)):
            ids = torch.full((tokens, top_k), -1, dtype=torch.int32, device=DEV)
            w = torch.full((tokens, top_k), -1.0, dtype=torch.float32, device=DEV)
            ops.router_select(src, bias if kind != "nan" else None, ids, w, top_k=top_k, impl=impl)
            dst.extend([ids.cpu(), w.cpu()])
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]), impl
    with pytest.raises(ValueError, match="does not support"):
        ops.router_select(torch.zeros(2, 300, device=DEV), None, torch.empty(2, 2, dtype=torch.int32, device=DEV),
                          torch.empty(2, 2, device=DEV), top_k=2, impl="warp")       # more than 256 experts


def test_router_tie_order_nan_and_softmax():
    from sparseengine_b200.csrc import ops
    x = torch.zeros(2, 8, device=DEV)
    gate = torch.zeros(6, 8, device=DEV)
    b = torch.tensor([0.0, 0.3, 0.0, 0.5, 0.0, 0.3], device=DEV)
    ids = torch.empty(2, 4, dtype=torch.int32, device=DEV)
    w = torch.empty(2, 4, dtype=torch.float32, device=DEV)
    ops.router(x, gate, b, ids, w, top_k=4)
    assert ids.cpu().tolist() == [[1, 3, 5, 0]] * 2 and torch.allclose(w.cpu(), torch.full((2, 4), 0.25))
    b2 = b.clone()
    b2[4] = float("nan")                         # a NaN score counts as +inf
    ids2 = torch.empty(2, 2, dtype=torch.int32, device=DEV)
    ops.router(x, gate, b2, ids2, torch.empty(2, 2, device=DEV), top_k=2)
    assert sorted(ids2.cpu()[0].tolist()) == [3, 4]
    x = rnd(3, 8, seed=4)
    gate = rnd(6, 8, seed=5)
    ids = torch.empty(3, 4, dtype=torch.int32, device=DEV)
    w = torch.empty(3, 4, dtype=torch.float32, device=DEV)
    ops.router(x, gate, None, ids, w, top_k=4, score_fn="softmax", renormalize=False, routed_scale=2.5)
    p = torch.softmax(x.cpu() @ gate.cpu().t(), -1)
    top = p.topk(4).indices
    assert [sorted(r) for r in ids.cpu().tolist()] == [sorted(r) for r in top.tolist()]
    torch.testing.assert_close(w.cpu(), 2.5 * p.gather(1, ids.cpu().long()), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,top_k,experts,tile_rows,width", [
    (1, 8, 256, 16, 3072), (8, 8, 256, 16, 3072), (37, 3, 6, 16, 40), (32, 8, 256, 32, 72),    # one launch
    (33, 8, 256, 32, 72), (700, 2, 1030, 64, 8), (5, 4, 1025, 16, 24)])                        # three launches
def test_routing_build_and_row_gather(dtype, tokens, top_k, experts, tile_rows, width):
    """Assignments sorted by expert (stably), the tile list, and the activation rows gathered
    into that order; few assignments take the single-launch kernel, the rest the three kernels."""
    from sparseengine_b200.csrc import ops
    g = torch.Generator().manual_seed(tokens + experts)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(tokens)]).int()
    if tokens >= 8:
        ids[: tokens // 2, 0] = 3          # one expert with many rows: several tiles
    a = tokens * top_k
    flat = ids.view(-1)
    i32 = dict(dtype=torch.int32, device=DEV)
    max_tiles = ops.moe_max_tiles(a, experts, tile_rows)
    ws = {"counts": torch.full((experts,), -7, **i32), "rank": torch.full((a,), -7, **i32),
          "offsets": torch.full((experts + 1,), -7, **i32), "sorted": torch.full((a,), -7, **i32),
          "inv_pos": torch.full((a,), -7, **i32), "tile_expert": torch.full((max_tiles,), -7, **i32),
          "tile_row0": torch.full((max_tiles,), -7, **i32), "num_tiles": torch.full((1,), -7, **i32)}
    x = rnd(tokens, width, dtype=dtype, seed=5)
    xs = torch.zeros(a, width, dtype=dtype, device=DEV)
    small = bool(ops.library().se_moe_route_is_small(a, experts))
    assert small == (a <= 256 and experts <= 1024)
    before = ops.launch_count
    ops.moe_route_build(flat.contiguous().to(DEV), experts, tile_rows, ws, gather=(x, xs, top_k))
    assert ops.launch_count - before == (1 if small else 3)
    order = torch.sort(flat.long(), stable=True).indices
    counts = torch.bincount(flat.long(), minlength=experts)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)])
    assert torch.equal(ws["sorted"].cpu().long(), order)
    assert torch.equal(ws["offsets"].cpu().long(), offsets)
    assert torch.equal(ws["counts"].cpu().long(), counts)
    inv = torch.empty(a, dtype=torch.long)
    inv[order] = torch.arange(a)
    assert torch.equal(ws["inv_pos"].cpu().long(), inv)
    tiles = [(e, int(offsets[e]) + r) for e in range(experts) for r in range(0, int(counts[e]), tile_rows)]
    n = int(ws["num_tiles"][0])
    assert n == len(tiles) <= max_tiles
    assert ws["tile_expert"][:n].tolist() == [t[0] for t in tiles]
    assert ws["tile_row0"][:n].tolist() == [t[1] for t in tiles]
    assert torch.equal(xs.cpu(), x.cpu()[order // top_k])
    # without the gather: the same tables
    ws2 = {k: torch.full_like(v, -7) for k, v in ws.items()}
    ops.moe_route_build(flat.contiguous().to(DEV), experts, tile_rows, ws2)
    for k in ("offsets", "sorted", "inv_pos", "num_tiles"):
        assert torch.equal(ws2[k], ws[k]), k


@pytest.mark.parametrize("path", ["cuda_cores", "tensor_cores"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,hidden,inter,experts,top_k", [
    (5, 64, 32, 4, 2), (70, 96, 48, 8, 3), (33, 80, 40, 6, 4), (130, 200, 72, 16, 5), (1, 64, 32, 4, 2),
    (300, 264, 136, 3, 2), (150, 264, 136, 4, 2)])      # the last two: tiles of 256 and of 128 rows
def test_routed_experts(dtype, tokens, hidden, inter, experts, top_k, path):
    """Grouped gate/up + SwiGLU, grouped down x routing weight and the combine, on CUDA cores
    (any dtype) and on tensor cores (bfloat16: TMA + tcgen05), against the plain loop."""
    if path == "tensor_cores" and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernels are bfloat16 kernels")
    from sparseengine_b200.config.specs import MoESpec
    from sparseengine_b200.csrc import ops
    from sparseengine_b200.parts.moe import SparseMoE
    x = rnd(tokens, hidden, dtype=dtype, seed=1)
    w13 = rnd(experts, 2 * inter, hidden, dtype=dtype, scale=0.1, seed=2)
    w2 = rnd(experts, hidden, inter, dtype=dtype, scale=0.1, seed=3)
    g = torch.Generator().manual_seed(4)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(tokens)]).int().to(DEV)
    if tokens > 40:
        ids[:, 0] = 1                           # a crowded expert (several row tiles) ...
        ids[ids == experts - 1] = 0             # ... and an empty one
        ids[:, 1] = 2
    wt = torch.rand(tokens, top_k, generator=g).to(DEV)
    part = SparseMoE(MoESpec(hidden_size=hidden, num_experts=experts, top_k=top_k, intermediate_size=inter), dtype)
    part.bind({"w13": w13, "w2": w2})
    part.use_tensor_cores = None if path == "tensor_cores" else False
    assert part.tensor_cores_usable(x) == (path == "tensor_cores")
    out = part.run_experts(x, ids, wt)
    ops.error_check(DEV)
    ref = plain_m2.experts(x.float().cpu(), ids.cpu().long(), wt.cpu(), w13[:, :inter].float().cpu(),
                           w13[:, inter:].float().cpu(), w2.float().cpu(), dtype)
    torch.testing.assert_close(out.float().cpu(), ref, **tol(dtype, 1e-5, 2e-2))


@pytest.mark.parametrize("dtype", DTYPES)
def test_sampling_greedy_and_filters(dtype):
    from sparseengine_b200.csrc import ops_sampling as sops
    vocab = 5003
    logits = rnd(6, vocab, dtype=dtype, scale=2.0, seed=9)
    logits[1, 77] = logits[1, 4000] = 50.0        # a tie: the first wins
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    sops.sample(logits, None, None, None, None, out)
    assert out.cpu().tolist() == logits.float().argmax(-1).cpu().tolist() and int(out[1]) == 77
    big = rnd(3, 200064, dtype=dtype, scale=2.0, seed=10)          # the two-stage path of large vocabularies
    big[2, 199999] = big[2, 5] = 60.0
    out3 = torch.empty(3, dtype=torch.int32, device=DEV)
    sops.sample(big, None, None, None, None, out3)
    assert out3.cpu().tolist() == big.float().argmax(-1).cpu().tolist() and int(out3[2]) == 5
    # top-k = 1 and a tiny top-p are greedy whatever the noise
    temp = torch.full((6,), 0.9, device=DEV)
    seeds = torch.arange(6, dtype=torch.int64, device=DEV) + 12345
    k1 = torch.ones(6, dtype=torch.int32, device=DEV)
    sops.sample(logits, temp, k1, torch.ones(6, device=DEV), seeds, out)
    assert out.cpu().tolist()[0] == int(logits[0].float().argmax()) and int(out[1]) in (77, 4000)
    sops.sample(logits, temp, torch.zeros(6, dtype=torch.int32, device=DEV), torch.full((6,), 1e-4, device=DEV), seeds, out)
    assert out.cpu().tolist()[2:] == logits.float().argmax(-1).cpu().tolist()[2:]


def test_sampling_distribution_topk_topp():
    """Many draws with different seeds follow softmax(logits / T) cut by top-k and top-p
    (the reference's rule: sorted, keep while the mass before an entry is <= top-p)."""
    from sparseengine_b200.csrc import ops_sampling as sops
    vocab, n = 50, 40000
    base = torch.linspace(2.0, -2.0, vocab)
    logits = base.repeat(n, 1).to(DEV)
    temp = torch.full((n,), 0.7, device=DEV)
    seeds = torch.arange(n, dtype=torch.int64, device=DEV) * 7919 + 17
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    for top_k, top_p in ((0, 1.0), (10, 1.0), (0, 0.6), (12, 0.8)):
        sops.sample(logits, temp, torch.full((n,), top_k, dtype=torch.int32, device=DEV),
                    torch.full((n,), top_p, device=DEV), seeds, out)
        p = torch.softmax(base / 0.7, -1)
        if top_k:
            p[top_k:] = 0
            p = p / p.sum()
        if top_p < 1:
            before = torch.cumsum(p, 0) - p
            p[before > top_p] = 0
            p = p / p.sum()
        hist = torch.bincount(out.cpu().long(), minlength=vocab).float() / n
        assert hist[p == 0].sum() == 0, (top_k, top_p)
        assert (hist - p).abs().max() < 0.01, (top_k, top_p)
    # the same seed gives the same token; the row's place in the batch does not matter
    sops.sample(logits[:4], temp[:4], None, None, seeds[10:14].contiguous(), out[:4])
    a = out[:4].cpu().tolist()
    sops.sample(logits[:2], temp[:2], None, None, seeds[12:14].contiguous(), out[:2])
    assert out[:2].cpu().tolist() == a[2:]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,scale", [(200064, 2.0), (200064, 6.0), (5003, 3.0), (300, 1.0)])
def test_sampling_fast_path_picks_what_the_definition_picks(dtype, vocab, scale):
    """The fast path (byte-wise top-k threshold, cut and draw over a short list in shared memory)
    against the same kernel with every cut and the draw over the whole row: same tokens and
    log-probabilities, for top-k, top-p, both, ties at the k-th value, and rows whose candidates
    do not fit the list (flat distributions), which fall back to the whole row."""
    from sparseengine_b200.csrc import ops_sampling as sops
    rows = 24
    logits = rnd(rows, vocab, dtype=dtype, scale=scale, seed=21)
    logits[3, 5:40] = logits[3].max() + 1.0                       # 35 entries tie at the top
    logits[4] = 0.0                                               # a flat row
    temp = torch.tensor([0.7, 1.0, 1.3] * 8, device=DEV)
    top_k = torch.tensor([0, 50, 1, 20, 7, 1000, 0, 3] * 3, dtype=torch.int32, device=DEV)
    top_p = torch.tensor([0.9, 1.0, 0.5, 0.95, 0.3, 0.99, 1e-4, 0.8, 1.0, 0.6, 0.9, 0.2] * 2, device=DEV)
    agree = 0
    for trial in range(4):
        seeds = torch.arange(rows, dtype=torch.int64, device=DEV) * 104729 + 31 * trial
        fast, slow = (torch.empty(rows, dtype=torch.int32, device=DEV) for _ in range(2))
        lp_fast, lp_slow = (torch.empty(rows, dtype=torch.float32, device=DEV) for _ in range(2))
        sops.sample(logits, temp, top_k, top_p, seeds, fast, lp_fast, impl=0)
        sops.sample(logits, temp, top_k, top_p, seeds, slow, lp_slow, impl=1)
        assert torch.equal(fast, slow), (trial, fast.tolist(), slow.tolist())
        torch.testing.assert_close(lp_fast, lp_slow, atol=1e-6, rtol=1e-6)
        agree += rows
        # top-k alone, and top-p alone
        zero_k, one_p = torch.zeros_like(top_k), torch.ones_like(top_p)
        for kk, pp in ((top_k, one_p), (zero_k, top_p)):
            sops.sample(logits, temp, kk, pp, seeds, fast, None, impl=0)
            sops.sample(logits, temp, kk, pp, seeds, slow, None, impl=1)
            assert torch.equal(fast, slow), (trial, fast.tolist(), slow.tolist())
    assert agree == 4 * rows


@pytest.mark.parametrize("dtype", DTYPES)
def test_sampling_without_cuts_many_blocks_per_row(dtype):
    """Temperature rows (and greedy rows among them) over a large vocabulary take kernels with
    many blocks per row: the same tokens as the one-block kernel, log-probabilities to rounding."""
    from sparseengine_b200.csrc import ops_sampling as sops
    rows, vocab = 9, 200064
    logits = rnd(rows, vocab, dtype=dtype, scale=3.0, seed=33)
    logits[2, 7] = logits[2, 150000] = logits[2].max() + 2.0          # a tie at the top of a greedy row
    temp = torch.tensor([0.7, 1.0, 0.0, 1.3, 0.0, 0.5, 2.0, 1.0, 0.9], device=DEV)
    for trial in range(3):
        seeds = torch.arange(rows, dtype=torch.int64, device=DEV) * 7919 + trial
        many, one = (torch.empty(rows, dtype=torch.int32, device=DEV) for _ in range(2))
        lp_many, lp_one = (torch.empty(rows, dtype=torch.float32, device=DEV) for _ in range(2))
        before = dict(sops.calls) if hasattr(sops, "calls") else None
        sops.sample(logits, temp, None, None, seeds, many, lp_many)
        sops.sample(logits, temp, None, None, seeds, one, lp_one, impl=1)
        assert torch.equal(many, one), (many.tolist(), one.tolist())
        assert int(many[2]) == 7
        torch.testing.assert_close(lp_many, lp_one, atol=2e-5, rtol=1e-5)


def test_penalties():
    from sparseengine_b200.csrc import ops_sampling as sops
    logits = torch.tensor([[1.0, -2.0, 3.0, 0.5], [1.0, -2.0, 3.0, 0.5]], device=DEV)
    pairs = torch.tensor([[0, 0, 1], [0, 1, 3], [0, 2, 3], [1, 3, 2]], dtype=torch.int32, device=DEV).view(-1)
    sops.apply_penalties(logits, pairs, 4, torch.tensor([2.0, 1.0], device=DEV), torch.tensor([0.5, 0.25], device=DEV))
    assert logits.cpu().tolist() == [[0.5, -4.5, 1.0, 0.5], [1.0, -2.0, 3.0, 0.25]]


@pytest.mark.parametrize("tokens", [1, 8, 64, 700, 2500, 4100])      # tiles of 16, 16, 16, 32, 128 and 256 rows
def test_tensor_core_experts_at_m2_layer_sizes(tokens):
    """256 experts, top-8, width 3072, expert width 1536: the tensor-core path against the plain
    implementation's experts run on the GPU in 32-bit (one matrix product per slot and expert,
    rounding to bfloat16 where the pipeline rounds), and the CUDA-core path against the same."""
    from sparseengine_b200.config.specs import MoESpec
    from sparseengine_b200.csrc import ops
    from sparseengine_b200.parts.moe import SparseMoE
    hidden, inter, experts, top_k = 3072, 1536, 256, 8
    g = torch.Generator(device=DEV).manual_seed(1)
    w13 = (torch.randn(experts, 2 * inter, hidden, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(experts, hidden, inter, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    x = torch.randn(tokens, hidden, generator=g, device=DEV).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(experts, generator=g, device=DEV)[:top_k] for _ in range(tokens)]).int()
    wt = torch.rand(tokens, top_k, generator=g, device=DEV)
    part = SparseMoE(MoESpec(hidden_size=hidden, num_experts=experts, top_k=top_k, intermediate_size=inter),
                     torch.bfloat16)
    part.bind({"w13": w13, "w2": w2})
    fast = part.run_experts(x, ids, wt)
    ops.error_check(DEV)
    ref = plain_m2.experts(x.float(), ids.long(), wt, w13[:, :inter], w13[:, inter:], w2, torch.bfloat16)
    rms = float(ref.pow(2).mean().sqrt())
    # Outputs are bfloat16 values; a different order of the 32-bit sums flips the last bit of an
    # element now and then (2^-8 of its size per rounding point, three points in a row).  Bound:
    # 2% of the outputs' root mean square plus one unit in the last place; on average far less.
    torch.testing.assert_close(fast.float(), ref, atol=2e-2 * rms, rtol=2.0 ** -7)
    assert (fast.float() - ref).abs().mean() < 2e-3 * rms
    if tokens <= 700:
        part.use_tensor_cores = False
        slow = part.run_experts(x, ids, wt)
        torch.testing.assert_close(slow.float(), ref, atol=2e-2 * rms, rtol=2.0 ** -7)
        assert (slow.float() - ref).abs().mean() < 2e-3 * rms


@pytest.mark.parametrize("rows,n_out,k_dim,nt", [(1, 128, 64, 16), (16, 8192, 3072, 16), (100, 384, 200, 32),
                                                 (333, 3072, 6144, 128), (64, 1000, 3072, 64)])
def test_tensor_core_dense_gemm(rows, n_out, k_dim, nt):
    from sparseengine_b200.csrc import ops
    x = rnd(rows, k_dim, dtype=torch.bfloat16, scale=0.5, seed=1)
    w = rnd(n_out, k_dim, dtype=torch.bfloat16, scale=0.1, seed=2)
    out = torch.empty(rows, n_out, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc_dense(x, w, out, nt)
    ops.error_check(DEV)
    ref = plain_m2.linear(x.float().cpu(), w.float().cpu(), torch.bfloat16)
    torch.testing.assert_close(out.float().cpu(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("hq,hkv,d,page,window", [(12, 2, 128, 16, None), (48, 8, 128, 16, None), (6, 6, 64, 8, None),
                                                  (40, 2, 64, 5, None), (8, 2, 128, 32, 100), (5, 1, 128, 1, None)])
def test_decode_attention_tensor_cores(hq, hkv, d, page, window):
    """The split-key tensor-core kernel against the plain attention of the plain
    implementation: single tokens and short portions, contexts from 1 key to thousands
    (several key splits), scattered pages, groups of 1..20 query heads per KV head."""
    from sparseengine_b200.csrc import ops
    kv_lens, q_lens = [1, 70, 1300, 4100, 257], [1, 3, 1, 1, 2]
    starts = [kv - ql for kv, ql in zip(kv_lens, q_lens)]
    dtype = torch.bfloat16
    table, rows, _, _, cache = _cache_setup(kv_lens, hkv, d, page, dtype)
    ks = [rnd(n, hkv, d, dtype=dtype, seed=20 + i) for i, n in enumerate(kv_lens)]
    vs = [rnd(n, hkv, d, dtype=dtype, seed=30 + i) for i, n in enumerate(kv_lens)]
    for i, n in enumerate(kv_lens):
        p = torch.arange(n, device=DEV)
        pg = table[int(rows[i]), (p // page).long()].long()
        cache[pg, 0, :, (p % page).long()] = ks[i]
        cache[pg, 1, :, (p % page).long()] = vs[i]
    t = sum(q_lens)
    q = rnd(t, hq, d, dtype=dtype, seed=7)
    positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, q_lens)]).int().to(DEV)
    token_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).int().to(DEV)
    out = torch.empty_like(q)
    ops.attn_decode(q.view(t, hq * d), cache, table, rows, token_seq, positions, out.view(t, hq * d), num_heads=hq,
                    num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5, window=window, max_keys=max(kv_lens))
    assert ops.attn_decode_plan(t, hq, hkv, max(kv_lens))[0] > 1          # several key splits are merged
    ref = _attention_reference(q.float().cpu(), [k.float().cpu() for k in ks], [v.float().cpu() for v in vs], q_lens,
                               starts, dtype, window)
    torch.testing.assert_close(out.float().cpu(), ref, atol=2e-2, rtol=2e-2)
    one = torch.empty_like(q)                                             # and without splitting
    plain = torch.empty_like(q)
    ops.paged_attention_plain(q.view(t, hq * d), cache, table, rows, token_seq, positions, plain.view(t, hq * d),
                              num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5, window=window)
    torch.testing.assert_close(out.float(), plain.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("impl", ["mma_sync", "tcgen05"])
@pytest.mark.parametrize("hq,hkv,d,page,window", [(12, 2, 128, 16, None), (48, 8, 128, 16, None), (6, 6, 64, 8, None),
                                                  (20, 4, 64, 5, None), (8, 2, 128, 32, 100), (5, 1, 128, 1, 33)])
def test_prefill_attention_tensor_cores(hq, hkv, d, page, window, impl):
    """The prompt-portion kernels (m16n8k16 tiles, and tcgen05 with tensor memory): whole
    prompts, portions that continue a cached prefix, single tokens beside them, row tiles
    that straddle tokens and requests' ends."""
    from sparseengine_b200.csrc import ops
    if impl == "tcgen05" and not ops.attn_prefill_tc_supported(d, hq, hkv):
        pytest.skip("the tcgen05 kernel takes head size 128")
    fn = ops.attn_prefill_tc if impl == "tcgen05" else ops.attn_prefill
    kv_lens, q_lens = [300, 70, 1, 700, 129, 64], [300, 3, 1, 257, 129, 1]
    starts = [kv - ql for kv, ql in zip(kv_lens, q_lens)]
    dtype = torch.bfloat16
    table, rows, _, _, cache = _cache_setup(kv_lens, hkv, d, page, dtype)
    ks = [rnd(n, hkv, d, dtype=dtype, seed=20 + i) for i, n in enumerate(kv_lens)]
    vs = [rnd(n, hkv, d, dtype=dtype, seed=30 + i) for i, n in enumerate(kv_lens)]
    for i, n in enumerate(kv_lens):
        p = torch.arange(n, device=DEV)
        pg = table[int(rows[i]), (p // page).long()].long()
        cache[pg, 0, :, (p % page).long()] = ks[i]
        cache[pg, 1, :, (p % page).long()] = vs[i]
    t = sum(q_lens)
    q = rnd(t, hq, d, dtype=dtype, seed=7)
    cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(kv_lens, dtype=torch.int32, device=DEV)
    out = torch.zeros_like(q)
    fn(q.view(t, hq * d), cache, table, rows, cu_q, kv_len, out.view(t, hq * d), entries=len(q_lens),
       max_q_len=max(q_lens), num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5, window=window)
    ops.error_check(DEV)
    ref = _attention_reference(q.float().cpu(), [k.float().cpu() for k in ks], [v.float().cpu() for v in vs], q_lens,
                               starts, dtype, window)
    torch.testing.assert_close(out.float().cpu(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("impl", ["mma_sync", "tcgen05"])
@pytest.mark.parametrize("hq,hkv", [(6, 2), (12, 2)])
def test_prefill_attention_when_row_maxima_keep_moving(hq, hkv, impl):
    """Scores with a spread of about 10 (in units of e) make a row's maximum jump by more than
    the kernels' rescaling threshold again and again, in some rows of a tile and not in others:
    the warps of a tile then run at different paces (the ones that rescale wait for the
    accumulator to be at rest), which is where a barrier shared between them, or a wait that may
    be a phase behind, shows.  The last rows of a tile, which see the last keys alone, are the
    ones that rescale there.  Against the plain attention, tightly, and bit for bit against a
    second run."""
    from sparseengine_b200.csrc import ops
    d, page, n = 128, 16, 700
    fn = ops.attn_prefill_tc if impl == "tcgen05" else ops.attn_prefill
    dtype = torch.bfloat16
    table, rows, _, _, cache = _cache_setup([n], hkv, d, page, dtype)
    g = torch.Generator(device=DEV).manual_seed(3)
    q = (torch.randn(n, hq, d, generator=g, device=DEV) * 3).to(dtype)
    k = torch.randn(n, hkv, d, generator=g, device=DEV).to(dtype)
    v = torch.randn(n, hkv, d, generator=g, device=DEV).to(dtype)
    p = torch.arange(n, device=DEV)
    pg = table[int(rows[0]), (p // page).long()].long()
    cache[pg, 0, :, (p % page).long()] = k
    cache[pg, 1, :, (p % page).long()] = v
    outs = []
    for _ in range(3):
        out = torch.zeros_like(q)
        fn(q.view(n, hq * d), cache, table, rows, torch.tensor([0, n], dtype=torch.int32, device=DEV),
           torch.tensor([n], dtype=torch.int32, device=DEV), out.view(n, hq * d), entries=1, max_q_len=n, num_heads=hq,
           num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5)
        outs.append(out)
    ops.error_check(DEV)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ref = _attention_reference(q.float().cpu(), [k.float().cpu()], [v.float().cpu()], [n], [0], dtype, None)
    err = (outs[0].float().cpu() - ref).abs()
    assert float(err.max()) < 3e-2 and float(err.mean()) < 2e-3, (float(err.max()), float(err.mean()))


@pytest.mark.parametrize("kernel", ["decode", "prefill_mma_sync", "prefill_tcgen05"])
@pytest.mark.parametrize("window", [None, 1000])
def test_tensor_core_attention_far_key_and_window_edge(kernel, window):
    """Random keys would hide a key that is skipped or seen wrongly, so one key is made to
    dominate the last query's scores: wherever it lies (first or last slot of a page, the
    first page, a split's or a tile's edge) the output must be its value.  With a window,
    the key just outside it must not be seen at all and the key just inside it must be."""
    from sparseengine_b200.csrc import ops
    hq, hkv, d, page, n = 8, 2, 128, 16, 3000
    dtype = torch.bfloat16
    q_len = 1 if kernel == "decode" else 130          # the last query is the one that is checked
    last = n - 1
    first_seen = 0 if window is None else last - window + 1
    places = [first_seen, first_seen + 1, last, last - 1, 2047, 2048, first_seen + 15, first_seen + 16]
    if window is None:
        places += [15, 16, 1023]
    else:
        places += [first_seen - 1, 0]                 # outside the window: must be invisible
    table, rows, _, _, cache = _cache_setup([n], hkv, d, page, dtype)
    k = rnd(n, hkv, d, dtype=dtype, scale=0.1, seed=1)
    v = rnd(n, hkv, d, dtype=dtype, seed=2)
    q = rnd(q_len, hq, d, dtype=dtype, scale=0.1, seed=3)
    pos = torch.arange(n, device=DEV)
    pg = table[int(rows[0]), (pos // page).long()].long()
    group = hq // hkv
    for far in places:
        kk = k.clone()
        kk[far] = (q[-1, ::group].float() * 300.0).to(dtype)       # KV head g gets the direction of its first query head
        cache[pg, 0, :, (pos % page).long()] = kk
        cache[pg, 1, :, (pos % page).long()] = v
        out = torch.zeros_like(q)
        if kernel == "decode":
            ops.attn_decode(q.view(q_len, hq * d), cache, table, rows, torch.zeros(q_len, dtype=torch.int32, device=DEV),
                            torch.tensor([last], dtype=torch.int32, device=DEV), out.view(q_len, hq * d), num_heads=hq,
                            num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5, window=window, max_keys=n)
        else:
            fn = ops.attn_prefill_tc if kernel == "prefill_tcgen05" else ops.attn_prefill
            fn(q.view(q_len, hq * d), cache, table, rows, torch.tensor([0, q_len], dtype=torch.int32, device=DEV),
               torch.tensor([n], dtype=torch.int32, device=DEV), out.view(q_len, hq * d), entries=1, max_q_len=q_len,
               num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5, window=window)
            ops.error_check(DEV)
        got = out[-1].float().cpu()
        visible = far >= first_seen
        for g in range(hkv):
            hit = torch.allclose(got[g * group], v[far, g].float().cpu(), atol=2e-2)
            assert hit == visible, (kernel, window, far, g)
        qs = torch.zeros(n, hq, d)
        qs[n - q_len:] = q.float().cpu()
        ref = plain_m2.causal_attention(qs, kk.float().cpu(), v.float().cpu(), dtype, window)[n - q_len:]
        torch.testing.assert_close(out.float().cpu(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("rows,n_out,k_dim", [(1, 16, 32), (8, 8192, 3072), (3, 3072, 6144), (16, 1000, 96), (11, 37, 160),
                                             (5, 200064, 3072)])
def test_gemv_for_a_handful_of_rows(rows, n_out, k_dim):
    from sparseengine_b200.csrc import ops
    x = rnd(rows, k_dim, dtype=torch.bfloat16, scale=0.5, seed=1)
    w = rnd(n_out, k_dim, dtype=torch.bfloat16, scale=0.1, seed=2)
    out = torch.full((rows, n_out), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.gemv(x, w, out)
    ref = (x.float() @ w.float().t())
    torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), atol=2e-2, rtol=2e-2)
    assert not ops.gemv_supported(17, n_out, k_dim) and not ops.gemv_supported(4, n_out, 40)


@pytest.mark.parametrize("dtype", DTYPES)
def test_top_logprobs(dtype):
    """The n most likely tokens of chosen rows with 32-bit log-softmax values, most likely first,
    equal logits by ascending id."""
    from sparseengine_b200.csrc import ops_sampling as sops
    vocab, n = 1003, 5
    logits = rnd(6, vocab, dtype=dtype, scale=3.0, seed=11)
    logits[2, 10] = logits[2, 700] = logits[2, 3] = 50.0         # a three-way tie at the top
    rows = torch.tensor([4, 2, 0], dtype=torch.int32, device=DEV)
    ids = torch.empty(3, n, dtype=torch.int32, device=DEV)
    vals = torch.empty(3, n, dtype=torch.float32, device=DEV)
    sops.top_logprobs(logits, rows, ids, vals)
    lp = torch.log_softmax(logits.float().cpu(), -1)
    for k, r in enumerate(rows.tolist()):
        order = sorted(range(vocab), key=lambda i: (-float(lp[r, i]), i))[:n]
        assert ids[k].tolist() == order
        torch.testing.assert_close(vals[k].cpu(), lp[r, order], atol=2e-5, rtol=1e-5)
    assert ids[1].tolist()[:3] == [3, 10, 700]


# ---- indices the kernels are given: an entry outside the pool is not followed ---------------

def _poisoned_setup(d, page, dtype, n=40, hkv=2):
    """One request of ``n`` keys in a cache of 8 pages of which the kernels are told 4 belong to
    the pool; block-table entry 1 names page 6: inside the allocation (nothing can fault, even
    if a check were wrong), outside the declared pool.  Page 6 holds infinities, so a kernel
    that followed the entry would show them in its output."""
    assert n <= 3 * page + page
    table = torch.tensor([[0, 6, 2, 3]], dtype=torch.int32, device=DEV)
    cache = rnd(8, 2, hkv, page, d, dtype=dtype, seed=40)
    cache[6] = float("inf")
    rows = torch.zeros(1, dtype=torch.int32, device=DEV)
    return table, rows, cache


@pytest.mark.parametrize("kernel", ["qk_prep", "qk_prep_many", "plain", "decode", "prefill_mma_sync", "prefill_tcgen05",
                                    "table_update"])
def test_a_block_table_entry_outside_the_pool_is_not_followed(kernel):
    """The entry is skipped and the kernel's code appears in the error word, which the next
    check raises from.  With the true pool size the same call is clean."""
    from sparseengine_b200.csrc import ops
    ops.error_check(DEV)
    hq, hkv, d, page = 4, 2, 128, 16
    dtype = torch.float32 if kernel == "plain" else torch.bfloat16
    table, rows, cache = _poisoned_setup(d, page, dtype)
    n = 40                                                   # positions 16..31 live on the bad entry
    for declared, code in ((4, {"qk_prep": 21, "qk_prep_many": 21, "plain": 22, "decode": 23, "prefill_mma_sync": 24,
                                "prefill_tcgen05": 25, "table_update": 26}[kernel]), (8, 0)):
        word = ops.error_word(DEV)
        if kernel.startswith("qk_prep"):
            t = 70 if kernel == "qk_prep_many" else 3
            first = 31 - t + 1 if t <= 16 else 0             # few tokens: all on the bad entry's page
            qkv = rnd(t, (hq + 2 * hkv) * d, dtype=dtype, seed=1)
            q_out = torch.zeros(t, hq * d, dtype=dtype, device=DEV)
            tbl = torch.tensor([[0, 6, 2, 3, 1]], dtype=torch.int32, device=DEV)
            before = cache.clone()
            ops.qk_prep(qkv, None, None, None, torch.arange(first, first + t, dtype=torch.int32, device=DEV),
                        torch.zeros(t, dtype=torch.int32, device=DEV), rows, tbl, cache, q_out, num_heads=hq,
                        num_kv_heads=hkv, head_dim=d, rotary_dim=0, eps=1e-6, rope_scale=1.0, page_size=page,
                        num_pages=declared)
            assert torch.equal(q_out, qkv[:, :hq * d])                   # the queries are written all the same
            if declared == 4:
                assert torch.equal(cache[6], before[6])                  # nothing was written through the bad entry
            else:
                assert not torch.equal(cache[6], before[6])
        elif kernel == "table_update":
            tbl = torch.full((2, 4), -1, dtype=torch.int32, device=DEV)
            upd = torch.tensor([0, 1, 3, 1, 2, 6, 5, 0, 1, 1, 9, 2], dtype=torch.int32, device=DEV)   # page 6; row 5; index 9
            ops.table_update(tbl, upd, 4, declared)
            want = [[-1, 3, -1, -1], [-1, -1, 6 if declared == 8 else -1, -1]]
            assert tbl.tolist() == want
            code = 26                                                    # row 5 and index 9 are refused either way
        else:
            q = rnd(1 if kernel in ("plain", "decode") else 24, hq, d, dtype=dtype, seed=2)
            t = q.shape[0]
            out = torch.zeros_like(q)
            kw = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5, num_pages=declared)
            if kernel in ("plain", "decode"):
                pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
                seq = torch.zeros(1, dtype=torch.int32, device=DEV)
                if kernel == "plain":
                    ops.paged_attention_plain(q.view(t, -1), cache, table, rows, seq, pos, out.view(t, -1), **kw)
                else:
                    ops.attn_decode(q.view(t, -1), cache, table, rows, seq, pos, out.view(t, -1), max_keys=n, **kw)
            else:
                fn = ops.attn_prefill_tc if kernel == "prefill_tcgen05" else ops.attn_prefill
                fn(q.view(t, -1), cache, table, rows, torch.tensor([0, t], dtype=torch.int32, device=DEV),
                   torch.tensor([n], dtype=torch.int32, device=DEV), out.view(t, -1), entries=1, max_q_len=t, **kw)
            finite = bool(torch.isfinite(out.float()).all())
            assert finite == (declared == 4)                            # followed, page 6's infinities would show
        got = int(word.item())
        assert got == code, (kernel, declared, got)
        if code:
            with pytest.raises(RuntimeError, match=f"code {code}"):
                ops.error_check(DEV)
        ops.error_check(DEV)                                             # the word was cleared


@pytest.mark.parametrize("kernel", ["prefill_mma_sync", "prefill_tcgen05", "decode", "plain"])
def test_pages_a_window_has_left_are_not_read(kernel):
    """A windowed request gives back the pages its window has passed, and their block-table
    entries stay on the device.  Such a page may already hold another request's values: here it
    holds infinities, and (for another entry) an id outside the pool.  The output is the same
    as with clean pages, and no code is written."""
    from sparseengine_b200.csrc import ops
    hq, hkv, d, page, window = 8, 2, 128, 16, 40
    dtype = torch.float32 if kernel == "plain" else torch.bfloat16
    n, q_len = 200, (1 if kernel in ("decode", "plain") else 37)
    table, rows, _, _, cache = _cache_setup([n], hkv, d, page, dtype)
    k, v = rnd(n, hkv, d, dtype=dtype, seed=1), rnd(n, hkv, d, dtype=dtype, seed=2)
    pos = torch.arange(n, device=DEV)
    pg = table[int(rows[0]), (pos // page).long()].long()
    cache[pg, 0, :, (pos % page).long()] = k
    cache[pg, 1, :, (pos % page).long()] = v
    first_needed = (n - q_len) - window + 1                     # the oldest key the portion's first query sees
    dead = list(range(first_needed // page))                    # table entries wholly before it
    assert len(dead) >= 4
    q = rnd(q_len, hq, d, dtype=dtype, seed=3)

    def run():
        out = torch.zeros_like(q)
        kw = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, page_size=page, scale=d ** -0.5, window=window)
        if kernel in ("decode", "plain"):
            p1 = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
            seq = torch.zeros(1, dtype=torch.int32, device=DEV)
            if kernel == "plain":
                ops.paged_attention_plain(q.view(q_len, -1), cache, table, rows, seq, p1, out.view(q_len, -1), **kw)
            else:
                ops.attn_decode(q.view(q_len, -1), cache, table, rows, seq, p1, out.view(q_len, -1), max_keys=window, **kw)
        else:
            fn = ops.attn_prefill_tc if kernel == "prefill_tcgen05" else ops.attn_prefill
            fn(q.view(q_len, -1), cache, table, rows, torch.tensor([0, q_len], dtype=torch.int32, device=DEV),
               torch.tensor([n], dtype=torch.int32, device=DEV), out.view(q_len, -1), entries=1, max_q_len=q_len, **kw)
        ops.error_check(DEV)
        return out

    clean = run()
    r = int(rows[0])
    for idx in dead[:-1]:
        cache[int(table[r, idx])] = float("inf")                # "another request's" values
    table[r, dead[0]] = 10 ** 6                                 # and an entry that names no page at all
    again = run()
    assert torch.isfinite(again.float()).all()
    assert torch.equal(again, clean)
    qs = torch.zeros(n, hq, d)
    qs[n - q_len:] = q.float().cpu()
    ref = plain_m2.causal_attention(qs, k.float().cpu(), v.float().cpu(), dtype, window)[n - q_len:]
    torch.testing.assert_close(again.float().cpu(), ref, **tol(dtype, 2e-5, 2e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing", ["split_half", "interleaved", "interleaved_to_split_half"])
@pytest.mark.parametrize("tokens", [5, 80])
def test_qk_prep_pairings_frequency_tables_and_amplitude(dtype, pairing, tokens):
    """The position encoding is data to the kernel: any table of frequencies (here a yarn table
    from the plain implementation), a factor on cos and sin, and three ways of pairing dims."""
    from sparseengine_b200.csrc import ops
    hq, hkv, d, rot, page = 3, 1, 64, 48, 8
    scaling = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64}
    inv, amp = plain_m2.rope_frequencies(rot, 1e4, scaling)
    table, rows, positions, token_seq, cache = _cache_setup([tokens], hkv, d, page, dtype, firsts=[100])
    qkv = rnd(tokens, (hq + 2 * hkv) * d, dtype=dtype, seed=8)
    q_out = torch.empty(tokens, hq * d, dtype=dtype, device=DEV)
    ops.qk_prep(qkv, None, None, inv.to(DEV), positions, token_seq, rows, table, cache, q_out, num_heads=hq,
                num_kv_heads=hkv, head_dim=d, rotary_dim=rot, eps=1e-6, rope_scale=amp, page_size=page, pairing=pairing)
    x = qkv.float().cpu()[:, :hq * d].view(tokens, hq, d)
    ref = plain_m2.partial_rotary(x, positions.cpu(), rot, 1e4, dtype, scaling, interleaved=pairing != "split_half")
    if pairing == "interleaved":                        # results go back to the adjacent dims
        r = ref[..., :rot].clone()
        ref[..., 0:rot:2], ref[..., 1:rot:2] = r[..., :rot // 2], r[..., rot // 2:]
    torch.testing.assert_close(q_out.float().cpu().view(tokens, hq, d), ref, **tol(dtype, 3e-5, 2e-2))
    assert amp > 1.0 and torch.equal(q_out.float().cpu().view(tokens, hq, d)[..., rot:], x[..., rot:])
    with pytest.raises(ValueError, match="pairing"):
        ops.qk_prep(qkv, None, None, inv.to(DEV), positions, token_seq, rows, table, cache, q_out, num_heads=hq,
                    num_kv_heads=hkv, head_dim=d, rotary_dim=rot, eps=1e-6, rope_scale=1.0, page_size=page, pairing="x")


def test_size_limits_the_parts_check_are_the_launchers_own():
    """The limits the parts refuse at construction restate what the launchers refuse; and at a
    limit the kernel runs, one past it the launcher says so."""
    from sparseengine_b200.csrc import ops
    for name in ("rmsnorm_max_width", "router_max_experts", "router_max_unaligned_width", "moe_max_experts"):
        assert ops.limit(name) == ops.LIMITS[name], name
    w = ops.LIMITS["rmsnorm_max_width"]
    x, wt = rnd(2, w + 8, seed=1), torch.ones(w + 8, device=DEV)
    y = torch.empty(2, w, device=DEV)
    ops.rmsnorm(x[:, :w].contiguous(), wt[:w].contiguous(), 1e-6, y)
    ref = plain_m2.rms_norm(x[:, :w].cpu(), wt[:w].cpu(), 1e-6, torch.float32)
    torch.testing.assert_close(y.cpu(), ref, atol=1e-5, rtol=1e-5)
    with pytest.raises(ValueError, match="size this kernel does not support"):
        ops.rmsnorm(x, wt, 1e-6, torch.empty_like(x))
    # a router over rows wider than its shared-memory tile: the tiled kernel takes them, for few tokens too
    hidden, experts = 7168, 16
    xr, gate = rnd(3, hidden, seed=2), rnd(experts, hidden, scale=0.05, seed=3)
    ids = torch.empty(3, 2, dtype=torch.int32, device=DEV)
    wts = torch.empty(3, 2, dtype=torch.float32, device=DEV)
    logits = torch.empty(3, experts, device=DEV)
    ops.router(xr, gate, None, ids, wts, top_k=2, logits_out=logits)
    torch.testing.assert_close(logits.cpu(), xr.cpu() @ gate.cpu().t(), atol=1e-4, rtol=1e-4)
    one = torch.empty(1, experts, device=DEV)
    ops.router(xr[:1].contiguous(), gate, None, ids[:1], wts[:1], top_k=2, logits_out=one)
    assert torch.equal(one[0], logits[0])                      # and a token's logits do not depend on the batch


@pytest.mark.parametrize("tokens,hidden,inter,experts,top_k", [
    (8, 64, 64, 2, 1), (40, 128, 136, 2, 2), (300, 256, 192, 3, 2), (333, 200, 72, 5, 3), (700, 3072, 1536, 8, 2),
    (2500, 3072, 1536, 64, 8), (4100, 3072, 1536, 256, 8)])
def test_experts_on_pairs_of_sms(tokens, hidden, inter, experts, top_k):
    """The grouped GEMMs on pairs of SMs (tcgen05.mma.cta_group::2, tiles of 256 x 256: gate and up
    rows of the same features side by side in one accumulator) against the plain implementation's
    experts: tiles of a few rows and of 256, experts without rows, widths that are no multiple of
    the 128-feature block, several items per pair (the accumulators and the exchange buffers
    alternate across items)."""
    from sparseengine_b200.config.specs import MoESpec
    from sparseengine_b200.csrc import ops
    from sparseengine_b200.parts.moe import SparseMoE
    g = torch.Generator(device=DEV).manual_seed(tokens)
    w13 = (torch.randn(experts, 2 * inter, hidden, generator=g, device=DEV) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(experts, hidden, inter, generator=g, device=DEV) * 0.05).to(torch.bfloat16)
    x = torch.randn(tokens, hidden, generator=g, device=DEV).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(experts, generator=g, device=DEV)[:top_k] for _ in range(tokens)]).int()
    if experts >= 5:                                 # an expert without rows: its tokens go to a neighbour they do not have yet
        for t in (ids == 1).any(-1).nonzero().view(-1).tolist():
            spare = next(e for e in range(experts) if e != 1 and e not in ids[t].tolist())
            ids[t][ids[t] == 1] = spare
    wt = torch.rand(tokens, top_k, generator=g, device=DEV)
    part = SparseMoE(MoESpec(hidden_size=hidden, num_experts=experts, top_k=top_k, intermediate_size=inter), torch.bfloat16)
    part.bind({"w13": w13, "w2": w2})
    part.pair_min_rows, part.pair_min_rows_per_expert = 1, 0
    before = ops.calls.get("se_moe_grouped_gemm_pair", 0)
    out = part.run_experts(x, ids, wt)
    ops.error_check(DEV)
    assert ops.calls.get("se_moe_grouped_gemm_pair", 0) == before + 2
    ref = plain_m2.experts(x.float(), ids.long(), wt, w13[:, :inter], w13[:, inter:], w2, torch.bfloat16)
    rms = float(ref.pow(2).mean().sqrt())
    torch.testing.assert_close(out.float(), ref, atol=2e-2 * rms, rtol=2.0 ** -7)
    assert (out.float() - ref).abs().mean() < 2e-3 * rms
    part.pair_min_rows = None                        # and the one-CTA kernel gives the same values to rounding
    one = part.run_experts(x, ids, wt)
    torch.testing.assert_close(out.float(), one.float(), atol=2e-2 * rms, rtol=2.0 ** -7)


@pytest.mark.parametrize("tokens,hidden,experts,top_k", [(256, 3072, 256, 8), (1000, 3072, 256, 8), (300, 1024, 40, 3)])
def test_router_logits_from_tensor_cores_are_32_bit_accurate(tokens, hidden, experts, top_k):
    """Prompt steps take their router logits from the tensor cores: the 32-bit gate as three
    bfloat16 terms, K in chunks of at most 512 whose partial sums are added in 32-bit.  Against a
    64-bit product the error stays under 6e-6 (logits of size 1), and the experts are those of
    the 64-bit scores wherever the gap to the next score is above 1e-5."""
    from sparseengine_b200.config.specs import MoESpec
    from sparseengine_b200.parts.moe import SparseMoE
    g = torch.Generator(device=DEV).manual_seed(3)
    gate = torch.randn(experts, hidden, generator=g, device=DEV) * (1.1 / math.sqrt(hidden))
    bias = torch.randn(experts, generator=g, device=DEV) * 0.05
    x = torch.randn(tokens, hidden, generator=g, device=DEV).to(torch.bfloat16)
    part = SparseMoE(MoESpec(hidden_size=hidden, num_experts=experts, top_k=top_k, intermediate_size=64), torch.bfloat16)
    part.bind({"gate": gate, "selection_bias": bias})
    assert part._split_gate() is not None and tokens >= part.split_router_min_tokens
    ids, w = part.route(x)
    ref_logits = x.double() @ gate.double().t()
    split = part._split_gate()
    chunks, kc, _ = split.shape
    parts = torch.bmm(x.view(tokens, chunks, kc).transpose(0, 1), split, out_dtype=torch.float32)
    logits = parts.view(chunks, tokens, 3, experts).sum(dim=(0, 2))
    assert float((logits.double() - ref_logits).abs().max()) < 6e-6
    p = torch.sigmoid(ref_logits)
    score = p + bias.double()
    srt = score.sort(-1, descending=True)
    gap = srt.values[:, top_k - 1] - srt.values[:, top_k]
    want = srt.indices[:, :top_k].sort(-1).values
    same = (ids.long().sort(-1).values == want).all(-1)
    assert bool(same[gap > 1e-5].all()) and int((gap > 1e-5).sum()) > tokens * 0.9
    sel = p.gather(1, ids.long())
    torch.testing.assert_close(w.double(), sel / sel.sum(-1, keepdim=True), atol=1e-5, rtol=1e-5)
    # few tokens take the kernels with the fixed order of sums: the same experts
    part.split_router_min_tokens = None
    ids2, _ = part.route(x)
    assert bool((ids2.long().sort(-1).values == want)[gap > 1e-5].all())


def test_read_stream_reads_any_size_and_reports_nothing():
    """The measuring aid that reads a tensor through bulk copies into shared memory: whole
    stages only (what is left of a 32 KB stage is not read), any number of stages, no result and
    no error code."""
    from sparseengine_b200.csrc import ops
    for nbytes in (1, 32 * 1024, 5 * 32 * 1024 + 17, 48 * 32 * 1024 * 3 + 32 * 1024, 40 << 20):
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
        ops.read_stream(buf)
        torch.cuda.synchronize()
        ops.error_check(DEV)
    with pytest.raises(ValueError):
        ops.read_stream(torch.zeros(64 * 1024 + 1, dtype=torch.uint8, device=DEV)[1:])      # not 16-byte aligned


_QK_PREP_SCRIPT = r"""
import sys, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
import plain_m2
from sparseengine_b200.csrc import ops
DEV = "cuda:0"
out = {{}}
for name, (hq, hkv, d, rot, page, norm, tokens) in {{"m2": (48, 8, 128, 64, 16, True, 300), "odd": (5, 3, 64, 32, 8, True, 130),
                                                    "plain": (6, 2, 128, 64, 16, False, 200), "full": (4, 4, 64, 64, 4, True, 70)}}.items():
    g = torch.Generator(device=DEV).manual_seed(len(name))
    qkv = (torch.randn(tokens, (hq + 2 * hkv) * d, generator=g, device=DEV) * 2).bfloat16()
    qw = (1 + 0.1 * torch.randn(hq * d, generator=g, device=DEV)).bfloat16() if norm else None
    kw = (1 + 0.1 * torch.randn(hkv * d, generator=g, device=DEV)).bfloat16() if norm else None
    inv = plain_m2.rope_inv_freq(rot, 1e6).to(DEV)
    pages = -(-(tokens + 900) // page) + 1
    table = torch.arange(pages, dtype=torch.int32, device=DEV).flip(0).view(1, -1).contiguous()
    cache = torch.zeros(pages, 2, hkv, page, d, dtype=torch.bfloat16, device=DEV)
    positions = torch.arange(900, 900 + tokens, dtype=torch.int32, device=DEV)
    zeros = torch.zeros(tokens, dtype=torch.int32, device=DEV)
    q_out = torch.empty(tokens, hq * d, dtype=torch.bfloat16, device=DEV)
    ops.qk_prep(qkv, qw, kw, inv, positions, zeros, zeros[:1], table, cache, q_out, num_heads=hq, num_kv_heads=hkv,
                head_dim=d, rotary_dim=rot, eps=1e-6, rope_scale=1.0, page_size=page)
    ops.error_check(DEV)
    out[name + ".q"] = q_out.cpu()
    out[name + ".cache"] = cache.cpu()
torch.save(out, sys.argv[1])
"""


def test_qk_prep_bfloat16_kernel_gives_the_bits_of_the_general_one(tmp_path):
    """Steps of many bfloat16 tokens take a kernel of their own (packed pairs, fewer instructions);
    SE_QK_PREP_GENERIC=1 sends them through the kernel that also serves 32-bit.  The library reads
    the switch once, so each kernel runs in a process of its own; queries and cache must be equal
    bit for bit."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "qk.py"
    script.write_text(_QK_PREP_SCRIPT.format(root=root))
    outs = []
    for generic in ("0", "1"):
        path = str(tmp_path / f"out{generic}.pt")
        subprocess.run([sys.executable, str(script), path], check=True, env=dict(os.environ, SE_QK_PREP_GENERIC=generic))
        outs.append(torch.load(path))
    assert outs[0].keys() == outs[1].keys()
    for k in outs[0]:
        assert torch.equal(outs[0][k], outs[1][k]), k
