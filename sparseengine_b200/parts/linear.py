"""Dense projections ``y = x · Wᵀ`` (no bias), 32-bit accumulation.

The reference runs these through a library GEMM (``F.linear``:
src/sparseengine/layers/linear.py:174-191, src/sparseengine/layers/embed_head.py:80), and so
does this module (cuBLAS through ``torch.matmul``), except for up to 8 rows in bfloat16
(decode), where the product is a stream over the weights and this library's own kernel
(csrc/gemv.cu) reads them once at memory speed.  In float32 the reduced-precision
matrix modes are switched off for the whole process, so a float32 product is a true
32-bit product.
"""
from __future__ import annotations

import torch

from ..csrc import ops

torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


USE_GEMV = True     # False: the library product for every shape
# Beyond this many output features the library product is taken for few rows too (measured at
# MiniMax M2's sizes: the LM head, 200,064 features, is ahead there).  An engine option
# (``kernel_tuning={"gemv_max_out_features": n}``) sets it.
GEMV_MAX_OUT = 16384
# ... and from this many rows on (measured in whole decode steps of 8 layers at MiniMax M2's sizes:
# 8 rows 2,735 µs with this kernel against 2,789 with the library, 9 rows 3,134 against 3,060,
# 16 rows 4,503 against 4,423: the kernel's second 8-row tile costs more than the library's
# product, which for 17 to 128 rows takes 11 µs per projection).  ``gemv_max_rows`` sets it.
GEMV_MAX_ROWS = 8


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [rows, in], w [out, in] → [rows, out]; CUDA tensors of one dtype only."""
    if not (x.is_cuda and w.is_cuda):
        raise ValueError("linear needs CUDA tensors (there is no CPU path)")
    if x.dtype != w.dtype:
        raise TypeError(f"linear: activation {x.dtype} and weight {w.dtype} differ")
    if (USE_GEMV and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous() and w.is_contiguous()
            and w.shape[0] <= GEMV_MAX_OUT and x.shape[0] <= GEMV_MAX_ROWS
            and ops.gemv_supported(x.shape[0], w.shape[0], x.shape[1])):
        # a handful of rows (decode): this library's weight-streaming kernel
        if out is None:
            out = torch.empty(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
        return ops.gemv(x, w, out)
    if out is None:
        return torch.matmul(x, w.t())
    return torch.matmul(x, w.t(), out=out)
