"""Grouped-query attention over the paged cache.

qkv projection → (optional) whole-projection QK RMSNorm → position encoding → K/V into
their page → attention over the request's pages → output projection.  Order of effects
as in the reference (src/sparseengine/models/minimax_m2.py:334-359): this step's keys are
written before attention reads the cache.
"""
from __future__ import annotations

import torch

from ..config.specs import ParamSpec
from ..csrc import ops
from .base import KVRequest, Mixer, make_position, register_mixer
from .linear import linear
from .position import RotaryArgs, as_rotary_args


class PagedAttention(Mixer):
    graph_safe = True
    # a step's entries are a grid dimension of the prompt-portion kernels
    max_step_entries = ops.LIMITS["grid_dim_yz"]

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError("num_heads must be a positive multiple of num_kv_heads")
        if s.head_dim <= 0 or s.head_dim % 16 or s.head_dim > ops.LIMITS["attention_max_head_dim"]:
            raise ValueError(f"head_dim {s.head_dim} is not supported (multiples of 16 up to "
                             f"{ops.LIMITS['attention_max_head_dim']})")
        if s.num_heads > ops.LIMITS["grid_dim_yz"]:
            raise ValueError(f"{s.num_heads} query heads are not supported (at most {ops.LIMITS['grid_dim_yz']}: "
                             "heads are a grid dimension of the attention kernels)")
        if s.qk_norm not in (None, "whole_projection"):
            raise ValueError(f"qk_norm {s.qk_norm!r} is not supported")
        if s.window is not None and s.window <= 0:
            raise ValueError("window must be positive (None: all keys)")
        self.position = make_position(s.position, dtype) if s.position is not None else None
        rot = getattr(s.position, "rotary_dim", 0) if s.position is not None else 0
        if rot > s.head_dim:
            raise ValueError(f"the position encoding rotates {rot} dims, a head has {s.head_dim}")
        self.q_norm = self.k_norm = None

    def parameters(self):
        s = self.spec
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        out = {"qkv": ParamSpec((q + 2 * kv, s.hidden_size)), "o": ParamSpec((s.hidden_size, q))}
        if s.qk_norm is not None:
            out["q_norm"] = ParamSpec((q,), "act", "norm")
            out["k_norm"] = ParamSpec((kv,), "act", "norm")
        return out

    def kv_request(self):
        return KVRequest(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def forward(self, x, step, slot):
        s = self.spec
        tokens = x.shape[0]
        # the position part first: whatever it launches to make its table then lies before the
        # projection, and q/k preparation, which starts as the projection's dependent, may read the
        # table while the projection still runs
        rope = (as_rotary_args(self.position.kernel_args(x.device)) if self.position is not None
                else RotaryArgs(None, 0))
        qkv = linear(x, self.qkv)
        q = torch.empty(tokens, s.num_heads * s.head_dim, dtype=x.dtype, device=x.device)
        ops.qk_prep(qkv, self.q_norm, self.k_norm, rope.inv_freq, step.positions, step.token_seq, step.seq_rows,
                    slot.table, slot.kv, q, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads,
                    head_dim=s.head_dim, rotary_dim=rope.rotary_dim, eps=s.qk_norm_eps, rope_scale=rope.scale,
                    page_size=slot.page_size, write_cache=slot.write_cache, pairing=rope.pairing,
                    step_inputs_settled=True)       # the projection before it does not write the positions
        attn = torch.empty_like(q)
        self.attend(q, attn, step, slot, after_qk_prep=True)
        return linear(attn, self.o)

    # The split-key kernel (one CTA per token, KV head and key split) reads a request's keys once
    # per token, the prompt-portion kernels once per 256 (token, head) rows but without splitting
    # the keys.  So portions go to the latter: steps of more than `decode_kernel_max_tokens`
    # tokens, and smaller steps whose longest entry has at least `portion_min_tokens` tokens and
    # that average at least `portion_min_average` tokens per entry (measured at M2 sizes: a
    # 512-token portion after an 8,192-token prefix takes 1.39 ms per layer instead of 3.79, a
    # 32-token one 0.87 instead of 1.08; eight decoding requests beside a 64-token portion 0.86
    # instead of 0.91).  The three numbers are defaults measured at those sizes on a B200; the
    # engine option ``kernel_tuning`` sets them per engine (results do not depend on them).
    decode_kernel_max_tokens = 512
    portion_min_tokens = 16
    portion_min_average = 8

    def takes_portion_kernel(self, step) -> bool:
        if step.num_tokens > self.decode_kernel_max_tokens:
            return True
        return (step.max_q_len >= self.portion_min_tokens
                and step.num_tokens >= self.portion_min_average * step.num_seqs)
    use_tensor_cores = None      # False: always the plain kernel

    def attend(self, q, out, step, slot, after_qk_prep=False):
        """``after_qk_prep``: the kernel launched last is the one that wrote this step's keys and
        ``q``; the split-key kernel then looks its place in the block table up while it still runs."""
        s = self.spec
        if (self.use_tensor_cores is not False and q.dtype == torch.bfloat16
                and ops.attn_decode_supported(s.head_dim, s.num_heads, s.num_kv_heads)):
            if not self.takes_portion_kernel(step):
                max_keys = step.max_kv_len if s.window is None else min(step.max_kv_len, s.window)
                ops.attn_decode(q, slot.kv, slot.table, step.seq_rows, step.token_seq, step.positions, out,
                                num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim,
                                page_size=slot.page_size, scale=s.scale, window=s.window, max_keys=max_keys,
                                step_inputs_settled=after_qk_prep)
            else:
                # prompt portions: tcgen05 + tensor memory for head size 128, m16n8k16 tiles otherwise
                fn = (ops.attn_prefill_tc if ops.attn_prefill_tc_supported(s.head_dim, s.num_heads, s.num_kv_heads)
                      else ops.attn_prefill)
                fn(q, slot.kv, slot.table, step.seq_rows, step.cu_q, step.kv_len, out, entries=step.num_seqs,
                   max_q_len=step.max_q_len, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads,
                   head_dim=s.head_dim, page_size=slot.page_size, scale=s.scale, window=s.window)
            return
        ops.paged_attention_plain(q, slot.kv, slot.table, step.seq_rows, step.token_seq, step.positions, out,
                                  num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim,
                                  page_size=slot.page_size, scale=s.scale, window=s.window)


register_mixer("attention", PagedAttention)
