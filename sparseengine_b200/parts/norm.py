"""RMSNorm with an optional fused residual add (kernel: csrc/elementwise.cu).

Reference: src/sparseengine/layers/layernorm.py:120-159.
"""
from __future__ import annotations

import torch

from ..config.specs import ParamSpec
from ..csrc import ops
from .base import Norm, register_norm


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if not 0 < spec.size <= ops.LIMITS["rmsnorm_max_width"]:
            raise ValueError(f"RMSNorm width {spec.size} is not supported: the kernel takes rows of 1 to "
                             f"{ops.LIMITS['rmsnorm_max_width']} elements")
        if not spec.eps > 0:
            raise ValueError("RMSNorm eps must be positive")

    def parameters(self):
        return {"weight": ParamSpec((self.spec.size,), "act", "norm")}

    def forward(self, x, residual=None):
        out = torch.empty_like(x)
        if residual is None:
            ops.rmsnorm(x, self.weight, self.spec.eps, out)
            return out, x
        new_residual = torch.empty_like(x)
        ops.rmsnorm(x, self.weight, self.spec.eps, out, residual=residual, residual_out=new_residual)
        return out, new_residual


register_norm("rms", RMSNorm)
