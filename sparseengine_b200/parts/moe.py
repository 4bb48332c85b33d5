"""Feed-forward parts: routed SwiGLU experts and the dense SwiGLU MLP.

Router (32-bit) → routing build (rows sorted by expert) → grouped gate/up GEMM with the
SwiGLU epilogue → grouped down GEMM times the routing weight → sum over the top-k slots
in slot order.  Reference: src/sparseengine/models/minimax_m2.py:140-269,
src/sparseengine/layers/packed_moe.py:138-155 (w13 = gate rows then up rows).
"""
from __future__ import annotations

import os

import torch

from ..config.specs import ParamSpec
from ..csrc import ops
from .base import FeedForward, register_feed_forward


class _RoutedSwiGLU(FeedForward):
    """Shared machinery: given ids [T, k] int32 and weights [T, k] float32, run experts."""

    graph_safe = True

    num_experts: int
    top_k: int
    hidden: int
    inter: int

    # None: tensor cores whenever the sizes allow (bfloat16, row pitches that TMA takes);
    # False: always the CUDA-core kernels (the float32 path uses them in any case).
    use_tensor_cores = None

    # Which tensor-core kernel runs the experts.  One CTA per tile (csrc/gemm_tc.cu) streams the
    # weights and is ahead while an expert has few rows; pairs of SMs on 256 x 256 tiles
    # (csrc/gemm_tc_pair.cu) take fewer bytes per flop from L2 and are ahead once the experts that
    # get rows have about a hundred each (measured at MiniMax M2's sizes, both kernels, 1,024 to
    # 8,192 tokens over 64 and 256 experts: 3 to 15 % faster from 128 rows per expert, 4 % slower
    # at 64).  How many experts get rows is not known on the host without waiting for the device,
    # so the choice goes by what the routing builds of earlier large steps counted (read from a
    # pinned copy that the step queues behind itself; at first every expert is assumed to get rows).
    # The two kernels sum in the same order, so the choice changes speed only.
    pair_min_rows = 2048                   # (token, slot) rows in the step; None: never the pair kernel
    pair_min_rows_per_expert = 100
    route_stats_large = None               # as route_stats, for steps of at least pair_min_rows rows

    def live_experts_estimate(self) -> float:
        host = getattr(self, "_large_host", None)
        if host is None:
            return float(self.num_experts)
        used, builds = int(host[0]), int(host[1])
        return used / builds if builds > 0 else float(self.num_experts)

    def takes_pair_kernel(self, rows: int) -> bool:
        forced = os.environ.get("SE_MOE_PAIR_MIN_ROWS")             # tuning aid: rows from which the pair kernel runs
        if forced:
            return rows >= int(forced)
        if self.pair_min_rows is None or rows < self.pair_min_rows:
            return False
        if not (ops.moe_grouped_gemm_pair_supported(self.hidden, self.inter)
                and ops.moe_grouped_gemm_pair_supported(self.inter, self.hidden)):
            return False
        return rows >= self.pair_min_rows_per_expert * self.live_experts_estimate()

    def tensor_cores_usable(self, x) -> bool:
        if self.use_tensor_cores is False or x.dtype != torch.bfloat16:
            return False
        return ops.gemm_tc_supported(self.hidden, self.inter) and ops.gemm_tc_supported(self.inter, self.hidden)

    # Two 64-bit counters on the device, created with the first step: [0] the experts that got at
    # least one row, summed over routing builds, [1] the routing builds.  The routing build
    # counts them where its per-expert counts already are (no launch of its own, also inside
    # replayed CUDA graphs); a benchmark reads the difference around a timed region to know how
    # many experts' weights a step had to read.
    route_stats = None

    def run_experts(self, x, ids, weights):
        tokens = x.shape[0]
        a = tokens * self.top_k
        dev = x.device
        tc = self.tensor_cores_usable(x)
        pair = tc and self.takes_pair_kernel(a)
        tile_rows = (ops.PAIR_TILE_ROWS if pair else ops.moe_tile_rows_tc(a, self.num_experts)) if tc else ops.moe_plain_tile_rows()
        max_tiles = ops.moe_max_tiles(a, self.num_experts, tile_rows)
        i32 = dict(dtype=torch.int32, device=dev)
        ws = {"counts": torch.empty(self.num_experts, **i32), "rank": torch.empty(a, **i32),
              "offsets": torch.empty(self.num_experts + 1, **i32), "sorted": torch.empty(a, **i32),
              "inv_pos": torch.empty(a, **i32), "tile_expert": torch.empty(max_tiles, **i32),
              "tile_row0": torch.empty(max_tiles, **i32), "num_tiles": torch.empty(1, **i32)}
        # the tensor-core GEMM reads the activation rows in expert order
        xs = torch.empty(a, self.hidden, dtype=x.dtype, device=dev) if tc else None
        if self.route_stats is None:
            self.route_stats = torch.zeros(2, dtype=torch.int64, device=dev)
            self.route_stats_large = torch.zeros(2, dtype=torch.int64, device=dev)
        large = tc and self.pair_min_rows is not None and a >= self.pair_min_rows
        settled = ops.moe_route_build(ids, self.num_experts, tile_rows, ws, gather=(x, xs, self.top_k) if tc else None,
                                      stats=self.route_stats_large if large else self.route_stats)
        if large:        # what this build counted reaches the host behind this step, for later steps' choice
            if getattr(self, "_large_host", None) is None:
                self._large_host = torch.zeros(2, dtype=torch.int64).pin_memory()
            self._large_host.copy_(self.route_stats_large, non_blocking=True)
        act = torch.empty(a, self.inter, dtype=x.dtype, device=dev)
        y = torch.empty(a, self.hidden, dtype=x.dtype, device=dev)
        if pair:
            ops.moe_grouped_gemm_pair(0, xs, self.w13, ws, None, act, experts=self.num_experts, max_tiles=max_tiles,
                                      n_out=self.inter, k_dim=self.hidden)
            ops.moe_grouped_gemm_pair(1, act, self.w2, ws, weights, y, experts=self.num_experts, max_tiles=max_tiles,
                                      n_out=self.hidden, k_dim=self.inter)
        elif tc:
            # the second product starts while the first still runs: the lists are older than both
            ops.moe_grouped_gemm_tc(0, xs, self.w13, ws, None, act, experts=self.num_experts, max_tiles=max_tiles,
                                    n_out=self.inter, k_dim=self.hidden, nt=tile_rows, lists_settled=settled)
            ops.moe_grouped_gemm_tc(1, act, self.w2, ws, weights, y, experts=self.num_experts, max_tiles=max_tiles,
                                    n_out=self.hidden, k_dim=self.inter, nt=tile_rows, lists_settled=True)
        else:
            ops.moe_grouped_gemm_plain(0, x, self.w13, ws, None, act, max_tiles=max_tiles, n_out=self.inter,
                                       k_dim=self.hidden, top_k=self.top_k)
            ops.moe_grouped_gemm_plain(1, act, self.w2, ws, weights, y, max_tiles=max_tiles, n_out=self.hidden,
                                       k_dim=self.inter, top_k=self.top_k)
        out = torch.empty(tokens, self.hidden, dtype=x.dtype, device=dev)
        ops.moe_combine(y, ws["inv_pos"], out, self.top_k)
        return out


class SparseMoE(_RoutedSwiGLU):
    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not supported (only 'silu')")
        if spec.score_fn not in ops.SCORE_FN:
            raise ValueError(f"score function {spec.score_fn!r} is not supported")
        if not 0 < spec.top_k <= spec.num_experts:
            raise ValueError("top_k must be in [1, num_experts]")
        most = min(ops.LIMITS["router_max_experts"], ops.LIMITS["moe_max_experts"])
        if spec.num_experts > most:
            raise ValueError(f"{spec.num_experts} experts are not supported (at most {most}: the selection and the "
                             "routing build keep per-expert tables in shared memory)")
        if spec.hidden_size % 4 and spec.hidden_size > ops.LIMITS["router_max_unaligned_width"]:
            raise ValueError(f"a router over rows of {spec.hidden_size} elements is not supported: widths that are no "
                             f"multiple of 4 go up to {ops.LIMITS['router_max_unaligned_width']}")
        if spec.hidden_size <= 0 or spec.intermediate_size <= 0:
            raise ValueError("hidden_size and intermediate_size must be positive")
        self.num_experts, self.top_k = spec.num_experts, spec.top_k
        self.hidden, self.inter = spec.hidden_size, spec.intermediate_size
        self.selection_bias = None

    def bind(self, tensors):
        super().bind(tensors)
        self._gate_split = None          # derived from the gate

    def parameters(self):
        s = self.spec
        out = {"gate": ParamSpec((s.num_experts, s.hidden_size), "float32"),
               "w13": ParamSpec((s.num_experts, 2 * s.intermediate_size, s.hidden_size)),
               "w2": ParamSpec((s.num_experts, s.hidden_size, s.intermediate_size))}
        if s.selection_bias:
            out["selection_bias"] = ParamSpec((s.num_experts,), "float32", "bias")
        return out

    # Debugging aid: set to a list and every call appends the chosen expert ids (a CPU
    # copy, [tokens, top_k]), so that a test can follow the router through a near-tie.
    capture = None

    # Prompt steps of at least this many tokens (bfloat16) take their router logits from the tensor
    # cores; fewer tokens, and every decode step, take the CUDA-core kernels, whose sums run in one
    # fixed order whatever the batch.  None: never.
    split_router_min_tokens = 256
    SPLIT_ROUTER_CHUNK = 512      # longest run of K that is accumulated in tensor-core precision

    def _split_gate(self):
        """The 32-bit gate as three bfloat16 terms (gate = hi + mid + lo exactly to 2^-24 of its
        size), laid out [chunks, K per chunk, 3 * experts] for one batched product, or None if the
        width does not cut into chunks.  The activations are bfloat16, so every product
        x * term is exact in 32-bit; the tensor cores' accumulator loses a little with every add,
        so K is cut into chunks of at most 512 whose partial sums are added on the CUDA cores in
        32-bit.  Measured at MiniMax M2's sizes against a 64-bit product: largest error 3.1e-6,
        mean 4.1e-7 (the library's 32-bit product, which the reference uses here
        (src/sparseengine/models/minimax_m2.py:166), has 1.2e-5 and 7.7e-7; the fixed-order kernel
        6.9e-7 and 1.0e-7)."""
        if getattr(self, "_gate_split", None) is None:
            h = self.hidden
            chunks = next((c for c in range(1, h + 1) if h % c == 0 and h // c <= self.SPLIT_ROUTER_CHUNK
                           and (h // c) % 8 == 0), None)
            if chunks is None:
                self._gate_split = False
            else:
                g = self.gate
                hi = g.to(torch.bfloat16)
                rest = g - hi.float()
                mid = rest.to(torch.bfloat16)
                lo = (rest - mid.float()).to(torch.bfloat16)
                split = torch.cat([hi, mid, lo], 0)                                   # [3E, H]
                self._gate_split = split.view(3 * self.num_experts, chunks, h // chunks).permute(1, 2, 0).contiguous()
        return self._gate_split if self._gate_split is not False else None

    def route(self, x):
        tokens = x.shape[0]
        ids = torch.empty(tokens, self.top_k, dtype=torch.int32, device=x.device)
        weights = torch.empty(tokens, self.top_k, dtype=torch.float32, device=x.device)
        s = self.spec
        split = None
        if (x.dtype == torch.bfloat16 and self.split_router_min_tokens is not None
                and tokens >= self.split_router_min_tokens):
            split = self._split_gate()
        if split is not None:
            chunks, kc, _ = split.shape
            parts = torch.bmm(x.view(tokens, chunks, kc).transpose(0, 1), split, out_dtype=torch.float32)
            # the selection adds the parts itself (chunk by chunk, term by term)
            ops.router_select(parts.view(chunks, tokens, 3, self.num_experts), self.selection_bias, ids, weights,
                              top_k=self.top_k, score_fn=s.score_fn, renormalize=s.renormalize,
                              routed_scale=s.routed_scale)
        else:
            ops.router(x, self.gate, self.selection_bias, ids, weights, top_k=self.top_k, score_fn=s.score_fn,
                       renormalize=s.renormalize, routed_scale=s.routed_scale)
        if self.capture is not None:
            self.capture.append(ids.cpu())
        return ids, weights

    # Most rows routed and run at once (the reference's mlp_chunk_size,
    # src/sparseengine/models/minimax_m2.py:254-268); the engine sets it from its options.
    chunk_rows = 16384

    def forward(self, x, step):
        if x.shape[0] <= self.chunk_rows:
            ids, weights = self.route(x)
            return self.run_experts(x, ids, weights)
        outs = []
        for a in range(0, x.shape[0], self.chunk_rows):
            xc = x[a:a + self.chunk_rows]
            ids, weights = self.route(xc)
            outs.append(self.run_experts(xc, ids, weights))
        return torch.cat(outs, 0)


class DenseMLP(_RoutedSwiGLU):
    """SwiGLU MLP = one expert every token selects with weight 1."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not supported (only 'silu')")
        self.num_experts, self.top_k = 1, 1
        self.hidden, self.inter = spec.hidden_size, spec.intermediate_size

    def parameters(self):
        s = self.spec
        return {"w13": ParamSpec((1, 2 * s.intermediate_size, s.hidden_size)),
                "w2": ParamSpec((1, s.hidden_size, s.intermediate_size))}

    def forward(self, x, step):
        tokens = x.shape[0]
        ids = torch.zeros(tokens, 1, dtype=torch.int32, device=x.device)
        weights = torch.ones(tokens, 1, dtype=torch.float32, device=x.device)
        return self.run_experts(x, ids, weights)


register_feed_forward("moe", SparseMoE)
register_feed_forward("dense_mlp", DenseMLP)
