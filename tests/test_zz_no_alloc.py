"""The routing build that allocates nothing (``se_moe_route_build_no_alloc``), called
through its exported C symbol the way a program without a tensor framework would call
it: the caller owns the input and every output, the scratch is inside the library.

It must give exactly what the ordinary entry point gives, on two calls in a row (the
second call finds the first call's leftovers in the shared scratch), and it must refuse
sizes beyond its fixed maximum.  The file name sorts last so that a run which stops at
the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

OUTPUTS = ("offsets", "sorted", "inv_pos", "tile_expert", "tile_row0", "num_tiles")


def _buffers(assignments, experts, tile_rows, fill):
    from sparseengine_b200.csrc import ops
    i32 = dict(dtype=torch.int32, device="cuda:0")
    tiles = ops.moe_max_tiles(assignments, experts, tile_rows)
    sizes = {"counts": experts, "rank": assignments, "offsets": experts + 1, "sorted": assignments,
             "inv_pos": assignments, "tile_expert": tiles, "tile_row0": tiles, "num_tiles": 1}
    return {k: torch.full((n,), fill, **i32) for k, n in sizes.items()}


def test_no_alloc_route_build_matches_the_ordinary_one_twice_in_a_row():
    from sparseengine_b200.csrc import ops
    lib = ops.library()
    fn = lib.se_moe_route_build_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 7
    err = lib.se_no_alloc_strerror
    err.restype = ctypes.c_char_p
    err.argtypes = [ctypes.c_int]
    stream = torch.cuda.current_stream().cuda_stream

    # first a large call, then a small one with other experts: stale ranks and counts of the
    # first call lie in the scratch when the second runs
    cases = [(4096, 8, 256, 32, 1), (37, 3, 6, 16, 2)]
    for tokens, top_k, experts, tile_rows, seed in cases:
        g = torch.Generator().manual_seed(seed)
        ids = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(tokens)]).int()
        ids = ids.view(-1).contiguous().to("cuda:0")
        a = ids.numel()
        want = _buffers(a, experts, tile_rows, -7)
        ops.moe_route_build(ids, experts, tile_rows, want)
        got = _buffers(a, experts, tile_rows, -7)
        rc = fn(ids.data_ptr(), a, experts, tile_rows, *[got[k].data_ptr() for k in OUTPUTS], stream)
        assert rc == 0, err(rc)
        torch.cuda.synchronize()
        n = int(want["num_tiles"][0])
        assert int(got["num_tiles"][0]) == n > 0
        for k in ("offsets", "sorted", "inv_pos"):
            assert torch.equal(got[k], want[k]), k
        for k in ("tile_expert", "tile_row0"):
            assert torch.equal(got[k][:n], want[k][:n]), k
        # and the result is a valid routing: a permutation, grouped by expert, stable
        srt = got["sorted"].cpu().long()
        assert sorted(srt.tolist()) == list(range(a))
        by_expert = ids.cpu().long()[srt]
        assert torch.equal(by_expert, by_expert.sort(stable=True).values)


def test_no_alloc_route_build_refuses_sizes_beyond_its_maximum():
    from sparseengine_b200.csrc import ops
    lib = ops.library()
    fn = lib.se_moe_route_build_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 7
    err = lib.se_no_alloc_strerror
    err.restype = ctypes.c_char_p
    err.argtypes = [ctypes.c_int]
    ids = torch.zeros(8, dtype=torch.int32, device="cuda:0")
    out = _buffers(8, 4, 4, 0)
    ptrs = [out[k].data_ptr() for k in OUTPUTS]
    rc = fn(ids.data_ptr(), 65537, 4, 4, *ptrs, 0)
    assert rc == -11 and b"65536" in err(rc)
    rc = fn(ids.data_ptr(), 8, 1025, 4, *ptrs, 0)
    assert rc == -12 and b"1024" in err(rc)
    assert fn(ids.data_ptr(), 8, 4, 0, *ptrs, 0) == -10
    assert fn(ids.data_ptr(), 0, 4, 4, *ptrs, 0) == 0          # nothing to do
    torch.cuda.synchronize()
    assert all(int(v.abs().sum()) == 0 for v in out.values())   # refused calls wrote nothing
