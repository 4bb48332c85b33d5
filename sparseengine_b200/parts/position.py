"""Rotary position encoding: owns the table of rotation frequencies; the rotation itself is
fused into the attention mixer's q/k preparation kernel (csrc/qk_prep.cu).

What the kernel is given is data (:class:`RotaryArgs`): one frequency per rotated pair, the
number of rotated dims, a factor on cos and sin, and which dims form a pair.  Everything an
architecture's configuration says about scaled frequencies is worked into the table here, on
the host, once: the kernel computes ``angle = position * inv_freq[j]`` in 32-bit and nothing
else.  Base table: inv_freq_j = theta^(-2j/R) in 32-bit
(src/sparseengine/layers/rotary_embedding.py:15-24).  Scaled tables, by ``frequency_scaling``
(the configuration's ``rope_scaling`` / ``rope_parameters`` entries; accepted types and their
required keys as src/sparseengine/models/rope.py:70-129, formulas as
src/sparseengine/layers/rotary_embedding.py:26-101):

* ``linear``: every frequency divided by ``factor``;
* ``llama3``: wavelengths beyond ``original/low_freq_factor`` are divided by ``factor``, those
  under ``original/high_freq_factor`` are kept, and the band between is blended;
* ``yarn``: frequencies are blended between kept (fast dims) and divided by ``factor`` (slow
  dims) over the ramp between the dims that make ``beta_fast`` and ``beta_slow`` turns within
  the original context; cos and sin are multiplied by an attention factor
  (``attention_factor``, else from ``mscale``/``mscale_all_dim``, else 0.1·ln(factor) + 1).

A position encoding of another kind registers a class whose ``kernel_args(device)`` returns
a :class:`RotaryArgs` (or the triple ``(inv_freq, rotary_dim, scale)``, split-half pairing).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .base import PositionEncoding, register_position

PAIRINGS = ("split_half", "interleaved", "interleaved_to_split_half")


@dataclass
class RotaryArgs:
    """What the q/k preparation kernel needs of a position encoding."""
    inv_freq: Optional[torch.Tensor]      # float32 [rotary_dim / 2] on the device; None: nothing is rotated
    rotary_dim: int                       # leading dims of each head that are rotated
    scale: float = 1.0                    # multiplies cos and sin
    pairing: str = "split_half"           # one of PAIRINGS


def as_rotary_args(args) -> RotaryArgs:
    if isinstance(args, RotaryArgs):
        return args
    inv_freq, rotary_dim, scale = args
    return RotaryArgs(inv_freq, int(rotary_dim), float(scale))


def _need(params: dict, key: str, kind: str) -> float:
    if key not in params:
        raise ValueError(f"{kind} frequency scaling needs {key!r}")
    v = float(params[key])
    if not math.isfinite(v):
        raise ValueError(f"{kind} frequency scaling: {key} must be finite, got {params[key]!r}")
    return v


def _yarn_amplitude(factor: float, multiplier: float = 1.0) -> float:
    return 1.0 if factor <= 1.0 else 0.1 * multiplier * math.log(factor) + 1.0


def scaled_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]) -> tuple:
    """``(inv_freq float32 [rotary_dim/2] on the CPU, factor on cos and sin)``."""
    exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim
    inv = 1.0 / (theta ** exponent)
    if not scaling:
        return inv, 1.0
    kind = str(scaling.get("rope_type", scaling.get("type", "default"))).lower()
    if kind == "default":
        return inv, 1.0
    if kind not in ("linear", "llama3", "yarn"):
        raise ValueError(f"frequency scaling {kind!r} is not supported (linear, llama3 and yarn are; "
                         "types that depend on the sequence length are not)")
    factor = _need(scaling, "factor", kind)
    if factor < 1.0:
        raise ValueError(f"{kind} frequency scaling: factor must be at least 1, got {factor}")
    if kind == "linear":
        return inv / factor, 1.0
    original = _need(scaling, "original_max_position_embeddings", kind)
    if original <= 0:
        raise ValueError(f"{kind} frequency scaling: original_max_position_embeddings must be positive")
    if kind == "llama3":
        low, high = _need(scaling, "low_freq_factor", kind), _need(scaling, "high_freq_factor", kind)
        if not 0 < low < high:
            raise ValueError(f"llama3 frequency scaling needs 0 < low_freq_factor < high_freq_factor, got {low}, {high}")
        wavelength = 2 * math.pi / inv
        long_wave, short_wave = original / low, original / high
        slowed = torch.where(wavelength > long_wave, inv / factor, inv)
        blend = (original / wavelength - low) / (high - low)
        blended = (1 - blend) * slowed / factor + blend * slowed
        between = (wavelength >= short_wave) & (wavelength <= long_wave)
        return torch.where(between, blended, slowed), 1.0
    # yarn
    fast, slow = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))
    if not (math.isfinite(fast) and math.isfinite(slow) and fast > slow > 0):
        raise ValueError(f"yarn frequency scaling needs beta_fast > beta_slow > 0, got {fast}, {slow}")

    def dim_of(turns: float) -> float:      # the (fractional) dim that makes `turns` turns in the original context
        return rotary_dim * math.log(original / (turns * 2 * math.pi)) / (2 * math.log(theta))

    first, last = dim_of(fast), dim_of(slow)
    if bool(scaling.get("truncate", True)):
        first, last = math.floor(first), math.ceil(last)
    first, last = max(first, 0), min(last, rotary_dim - 1)
    if first == last:
        last += 0.001
    ramp = torch.clamp((torch.arange(rotary_dim // 2, dtype=torch.float32) - first) / (last - first), 0, 1)
    kept = 1 - ramp
    inv = inv / factor * (1 - kept) + inv * kept
    amplitude = scaling.get("attention_factor")
    if amplitude is None:
        m, m_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
        amplitude = (_yarn_amplitude(factor, float(m)) / _yarn_amplitude(factor, float(m_all)) if m and m_all
                     else _yarn_amplitude(factor))
    amplitude = float(amplitude)
    if not (math.isfinite(amplitude) and amplitude > 0):
        raise ValueError(f"yarn frequency scaling: the attention factor must be positive and finite, got {amplitude}")
    return inv, amplitude


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if spec.pairing not in PAIRINGS:
            raise ValueError(f"rotary pairing {spec.pairing!r} is not supported; known: {list(PAIRINGS)}")
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError("rotary_dim must be positive and even")
        if not spec.theta > 0:
            raise ValueError("theta must be positive")
        scaling = dict(spec.frequency_scaling) if spec.frequency_scaling else None
        self._table, amplitude = scaled_frequencies(spec.rotary_dim, spec.theta, scaling)
        self._scale = float(spec.scaling) * amplitude
        self._inv_freq = None

    def inv_freq(self, device) -> torch.Tensor:
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            self._inv_freq = self._table.to(device)
        return self._inv_freq

    def kernel_args(self, device) -> RotaryArgs:
        return RotaryArgs(self.inv_freq(device), self.spec.rotary_dim, self._scale, self.spec.pairing)


register_position("rotary", RotaryEncoding)
