"""Time one hot kernel of the engine alone, at MiniMax M2 layer sizes by default, and
report the achieved fraction of its roofline (bytes it must read over time against the
copy bandwidth, or flops over time against the bf16 peak).

    python -m sparseengine_b200.cli.kernel_bench --kernel experts --tokens 8
    python -m sparseengine_b200.cli.kernel_bench --kernel attention_decode --batch 8 --context 3072
    python -m sparseengine_b200.cli.kernel_bench --kernel attention_prefill --tokens 2048
    python -m sparseengine_b200.cli.kernel_bench --kernel router --tokens 2048
    python -m sparseengine_b200.cli.kernel_bench --kernel dense --tokens 8 --n 8192 --k 3072

The workload is small on purpose (a few GB at most, weights larger than the L2 cache), so
that a profiler capture of it ends quickly.  ``--experts-resident`` experts are allocated
(the routing only uses those); several weight sets are rotated so that no launch finds its
weights in L2.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks() -> dict:
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out.update({k: float(d[k]) for k in ("hbm_gbs", "bf16_tflops") if d.get(k)})
            out["source"] = "measured"
        except Exception:
            pass
    return out


def timed(fn, iters: int, warmup: int = 3) -> float:
    """Milliseconds per call.  The calls are captured into one CUDA graph and the graph is
    timed with CUDA events, so that short kernels are not measured by how fast Python can
    launch them; if capture is not possible the calls are timed launch by launch."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph = None
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        graph = g
    except Exception:
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph is not None:
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
    else:
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_experts(a, dev):
    from ..config.specs import MoESpec
    from ..csrc import ops
    from ..parts.moe import SparseMoE
    e, k = a.experts_resident, a.top_k
    g = torch.Generator(device=dev).manual_seed(1)
    sets = []
    for _ in range(a.weight_sets):
        part = SparseMoE(MoESpec(hidden_size=a.hidden, num_experts=e, top_k=k, intermediate_size=a.inter), torch.bfloat16)
        part.bind({"w13": (torch.randn(e, 2 * a.inter, a.hidden, generator=g, device=dev) * 0.02).bfloat16(),
                   "w2": (torch.randn(e, a.hidden, a.inter, generator=g, device=dev) * 0.02).bfloat16()})
        sets.append(part)
    x = torch.randn(a.tokens, a.hidden, generator=g, device=dev).bfloat16()
    ids = torch.stack([torch.randperm(e, generator=g, device=dev)[:k] for _ in range(a.tokens)]).int()
    wt = torch.rand(a.tokens, k, generator=g, device=dev)
    distinct = len(set(ids.view(-1).tolist()))
    i = [0]

    def run():
        sets[i[0] % len(sets)].run_experts(x, ids, wt)
        i[0] += 1
    ms = timed(run, a.iters)
    ops.error_check(dev)
    by = distinct * 3 * a.inter * a.hidden * 2
    fl = a.tokens * k * 3 * 2 * a.inter * a.hidden
    return ms, by, fl, {"distinct_experts": distinct, "kernels": "route build with row gather, gate/up+SwiGLU, down, combine"}


def _filled_cache(a, dev, kv_lens):
    page = a.page_size
    pages = sum(-(-n // page) for n in kv_lens) + 1
    cache = (torch.randn(pages, 2, a.kv_heads, page, a.head_dim, device=dev) * 0.5).bfloat16()
    width = max(-(-n // page) for n in kv_lens)
    table = torch.zeros(len(kv_lens), width, dtype=torch.int32, device=dev)
    perm = torch.randperm(pages - 1, device=dev).int()
    o = 0
    for r, n in enumerate(kv_lens):
        c = -(-n // page)
        table[r, :c] = perm[o:o + c]
        o += c
    return cache, table


def bench_attention_decode(a, dev):
    from ..csrc import ops
    b = a.batch
    kv = [a.context] * b
    cache, table = _filled_cache(a, dev, kv)
    q = (torch.randn(b, a.heads * a.head_dim, device=dev)).bfloat16()
    out = torch.empty_like(q)
    rows = torch.arange(b, dtype=torch.int32, device=dev)
    pos = torch.full((b,), a.context - 1, dtype=torch.int32, device=dev)

    def run():
        ops.attn_decode(q, cache, table, rows, rows, pos, out, num_heads=a.heads, num_kv_heads=a.kv_heads,
                        head_dim=a.head_dim, page_size=a.page_size, scale=a.head_dim ** -0.5, max_keys=a.context)
    ms = timed(run, a.iters)
    by = b * a.context * 2 * a.kv_heads * a.head_dim * 2
    fl = 4 * b * a.context * a.heads * a.head_dim
    return ms, by, fl, {"splits": ops.attn_decode_plan(b, a.heads, a.kv_heads, a.context)[0]}


def bench_attention_prefill(a, dev):
    from ..csrc import ops
    t = a.tokens
    cache, table = _filled_cache(a, dev, [a.context_prefix + t])
    q = (torch.randn(t, a.heads * a.head_dim, device=dev)).bfloat16()
    out = torch.empty_like(q)
    rows = torch.zeros(1, dtype=torch.int32, device=dev)
    cu = torch.tensor([0, t], dtype=torch.int32, device=dev)
    kvl = torch.tensor([a.context_prefix + t], dtype=torch.int32, device=dev)

    fn = ops.attn_prefill_tc if a.impl == "tcgen05" else ops.attn_prefill

    def run():
        fn(q, cache, table, rows, cu, kvl, out, entries=1, max_q_len=t, num_heads=a.heads,
           num_kv_heads=a.kv_heads, head_dim=a.head_dim, page_size=a.page_size, scale=a.head_dim ** -0.5)
    ms = timed(run, a.iters)
    ops.error_check(dev)
    keys = a.context_prefix * t + t * (t + 1) / 2
    fl = 4 * a.heads * a.head_dim * keys
    by = (a.context_prefix + t) * 2 * a.kv_heads * a.head_dim * 2 + 2 * t * a.heads * a.head_dim * 2
    return ms, by, fl, {"impl": a.impl}


def bench_router(a, dev):
    from ..csrc import ops
    x = torch.randn(a.tokens, a.hidden, device=dev).bfloat16()
    gate = torch.randn(a.experts, a.hidden, device=dev) * 0.1
    bias = torch.randn(a.experts, device=dev) * 0.1
    ids = torch.empty(a.tokens, a.top_k, dtype=torch.int32, device=dev)
    w = torch.empty(a.tokens, a.top_k, dtype=torch.float32, device=dev)
    ms = timed(lambda: ops.router(x, gate, bias, ids, w, top_k=a.top_k), a.iters)
    return ms, a.experts * a.hidden * 4 + a.tokens * a.hidden * 2, 2 * a.tokens * a.hidden * a.experts, {}


def bench_dense(a, dev):
    from ..csrc import ops
    from ..parts.linear import linear
    x = torch.randn(a.tokens, a.k, device=dev).bfloat16()
    sets = max(a.weight_sets, -(-(300 << 20) // (a.n * a.k * 2)))          # more weights than the L2 holds
    ws = [(torch.randn(a.n, a.k, device=dev) * 0.02).bfloat16() for _ in range(sets)]
    out = torch.empty(a.tokens, a.n, dtype=torch.bfloat16, device=dev)
    i = [0]


    def run_lib():
        torch.matmul(x, ws[i[0] % len(ws)].t(), out=out)
        i[0] += 1

    def run_gemv():
        ops.gemv(x, ws[i[0] % len(ws)], out)
        i[0] += 1

    def run_tc():
        ops.gemm_tc_dense(x, ws[i[0] % len(ws)], out, 16 if a.tokens <= 16 else 64 if a.tokens <= 64 else 128)
        i[0] += 1
    ms = timed(run_lib, a.iters)
    ms_tc = timed(run_tc, a.iters)
    extra = {"library_ms": round(ms, 4), "own_tcgen05_ms": round(ms_tc, 4)}
    if ops.gemv_supported(a.tokens, a.n, a.k):
        ms = timed(run_gemv, a.iters)          # what the engine runs for this shape
        extra["own_gemv_ms"] = round(ms, 4)
    return ms, a.n * a.k * 2, 2 * a.tokens * a.n * a.k, extra


def bench_read_stream(a, dev):
    """``--mb`` MB read once by bulk asynchronous copies into shared memory (csrc/read_stream.cu)."""
    from ..csrc import ops
    buf = torch.empty(a.mb << 20, dtype=torch.uint8, device=dev).fill_(1)
    ms = timed(lambda: ops.read_stream(buf), a.iters)
    ops.error_check(dev)
    return ms, buf.numel(), 0, {}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", required=True,
                    choices=["experts", "attention_decode", "attention_prefill", "router", "dense", "read_stream"])
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=3072)
    ap.add_argument("--context-prefix", type=int, default=0)
    ap.add_argument("--hidden", type=int, default=3072)
    ap.add_argument("--inter", type=int, default=1536)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--experts-resident", type=int, default=64)
    ap.add_argument("--weight-sets", type=int, default=2)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--heads", type=int, default=48)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--mb", type=int, default=4096, help="read_stream: bytes to read, in MB")
    ap.add_argument("--impl", default="tcgen05", choices=["tcgen05", "mma_sync"],
                    help="attention_prefill: which of the two tensor-core kernels")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("kernel_bench needs a CUDA device")
    dev = "cuda:0"
    fn = {"experts": bench_experts, "attention_decode": bench_attention_decode,
          "attention_prefill": bench_attention_prefill, "router": bench_router, "dense": bench_dense,
          "read_stream": bench_read_stream}[a.kernel]
    ms, by, fl, extra = fn(a, dev)
    pk = peaks()
    gbs, tfl = by / ms / 1e6, fl / ms / 1e9
    out = {"kernel": a.kernel, "ms": round(ms, 4), "bytes": by, "flops": fl, "GB/s": round(gbs, 1),
           "TFLOP/s": round(tfl, 2), "hbm_frac": round(gbs / pk["hbm_gbs"], 4),
           "bf16_frac": round(tfl / pk["bf16_tflops"], 4), "peaks": pk["source"]}
    out.update(extra)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
