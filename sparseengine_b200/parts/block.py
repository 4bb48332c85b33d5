"""Arrangement of a layer's parts in a block.

``pre_norm``: the model carries ``(hidden, residual)``; the first block takes
``residual = hidden``; afterwards each norm call adds the last sublayer's output to the
residual (32-bit add, rounded to the activation dtype) and normalises the unrounded sum
(src/sparseengine/models/minimax_m2.py:381-397).  Another arrangement registers under
another name in ``ARRANGEMENTS``: a class built from ``(LayerSpec, dtype)`` with ``parts()``
(name -> part: the model lists parameters and cache needs from it; the part named ``mixer`` is
the one that may ask for pages or state), ``forward(hidden, residual, step, slot)`` ->
``(hidden, residual)``, and an attribute ``mixer``.  Parts beyond the four of ``pre_norm`` come
from ``LayerSpec.extra``.
"""
from __future__ import annotations

from .base import make_feed_forward, make_mixer, make_norm


class PreNormBlock:
    def __init__(self, spec, dtype):
        self.spec = spec
        self.mixer = make_mixer(spec.mixer, dtype)
        self.feed_forward = make_feed_forward(spec.feed_forward, dtype)
        self.mixer_norm = make_norm(spec.mixer_norm, dtype)
        self.feed_forward_norm = make_norm(spec.feed_forward_norm, dtype)

    def parts(self) -> dict:
        return {"mixer": self.mixer, "feed_forward": self.feed_forward, "mixer_norm": self.mixer_norm,
                "feed_forward_norm": self.feed_forward_norm}

    def forward(self, hidden, residual, step, slot):
        x, residual = self.mixer_norm.forward(hidden, residual)
        hidden = self.mixer.forward(x, step, slot)
        x, residual = self.feed_forward_norm.forward(hidden, residual)
        hidden = self.feed_forward.forward(x, step)
        return hidden, residual


ARRANGEMENTS = {"pre_norm": PreNormBlock}


def make_block(spec, dtype):
    if spec.arrangement not in ARRANGEMENTS:
        raise ValueError(f"unknown block arrangement {spec.arrangement!r}; known: {sorted(ARRANGEMENTS)}")
    return ARRANGEMENTS[spec.arrangement](spec, dtype)
