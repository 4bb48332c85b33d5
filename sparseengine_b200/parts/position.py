"""Rotary position encoding: owns the inverse-frequency table; the rotation itself is
fused into the attention mixer's q/k preparation kernel (csrc/qk_prep.cu).

inv_freq_j = theta^(-2j/R), computed in 32-bit exactly as the reference does
(src/sparseengine/layers/rotary_embedding.py:15-24); angle = position * inv_freq.
A position encoding part exposes ``kernel_args()`` → (inv_freq tensor or None,
rotary_dim, scale); another pairing or scaling is another ``kind``.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if spec.pairing != "split_half":
            raise ValueError(f"rotary pairing {spec.pairing!r} is not supported (only 'split_half')")
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError("rotary_dim must be positive and even")
        self._inv_freq = None

    def inv_freq(self, device) -> torch.Tensor:
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            r = self.spec.rotary_dim
            inv = 1.0 / (self.spec.theta ** (torch.arange(0, r, 2, dtype=torch.float32) / r))
            self._inv_freq = inv.to(device)
        return self._inv_freq

    def kernel_args(self, device):
        return self.inv_freq(device), self.spec.rotary_dim, float(self.spec.scaling)


register_position("rotary", RotaryEncoding)
