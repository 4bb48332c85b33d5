"""Interfaces of the parts a layer is assembled from, and their registries.

A part is built from its spec record (``sparseengine_b200.config.specs``) and the
engine's activation dtype; it declares its parameters (:meth:`Part.parameters`), gets
them bound once they are loaded (:meth:`Part.bind`) and runs on the tokens of one step.
No part knows which model it is in: sizes and constants come from the spec only.

Registries map a spec's ``kind`` to the class that implements it:
``MIXERS`` (``forward(x, step, slot) -> y``), ``FEED_FORWARDS`` (``forward(x, step) -> y``),
``NORMS`` (``forward(x, residual=None) -> (y, residual)``) and ``POSITIONS`` (built by a
mixer from its spec's ``position`` field).  Registering a new kind needs no change to
the framework: call :func:`register_mixer` (or its siblings) before the model is built.

What a mixer may ask of the cache manager:

* :meth:`Mixer.kv_request` → :class:`KVRequest`: paged keys and values, all keys or a
  window of them; layers whose requests are equal share one group of pages;
* :meth:`Mixer.state_request` → :class:`StateRequest`: a per-request state of fixed
  size, zeroed when a request is admitted.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..config.specs import ParamSpec


@dataclass(frozen=True)
class KVRequest:
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: every key is kept; n: only the last n


@dataclass(frozen=True)
class StateRequest:
    shape: tuple                     # per request
    dtype: torch.dtype = torch.float32


@dataclass
class LayerSlot:
    """What one visit of the execution order may touch besides its weights."""
    kv: Optional[torch.Tensor] = None        # [pages, 2, kv heads, page_size, head_dim] of its cache layer
    table: Optional[torch.Tensor] = None     # [rows, max pages] int32 block table of its group
    page_size: int = 0
    write_cache: bool = True
    state: Optional[torch.Tensor] = None     # [rows, *StateRequest.shape]


@dataclass
class StepContext:
    """Device-side description of one step's batch (int32 tensors) plus host copies.

    Token ``i`` belongs to batch entry ``token_seq[i]`` and sits at absolute position
    ``positions[i]`` of its request; entry ``j`` owns cache/state row ``seq_rows[j]``,
    brings ``q_lens[j]`` tokens starting at ``q_starts[j]`` and has ``kv_lens[j]`` tokens
    in the cache once this step's keys are written.
    """
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_seq: torch.Tensor
    seq_rows: torch.Tensor
    cu_q: torch.Tensor               # [num_seqs + 1]
    kv_len: torch.Tensor             # [num_seqs]
    q_lens: list = field(default_factory=list)       # host
    q_starts: list = field(default_factory=list)     # host
    kv_lens: list = field(default_factory=list)      # host
    rows: list = field(default_factory=list)         # host copy of seq_rows
    dtype: torch.dtype = torch.float32
    extras: dict = field(default_factory=dict)       # scratch shared by parts within a step
    max_kv_bound: Optional[int] = None               # an upper bound to plan launches with, if set

    @property
    def state_rows(self) -> torch.Tensor:
        """Entry ``j``'s row in every per-request state tensor (``LayerSlot.state[row]``), on the
        device.  A mixer with state of its own that indexes its state with this tensor and finds
        its tokens through ``token_seq`` / ``cu_q`` / ``positions`` reads nothing from the host,
        and may declare itself ``graph_safe``.  (The same rows index the block tables.)"""
        return self.seq_rows

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    @property
    def max_kv_len(self) -> int:
        """Most keys any entry has; launch plans use ``max_kv_bound`` when it is set (a
        replayed CUDA graph is planned for a bound, not for the step's exact lengths)."""
        if self.max_kv_bound is not None:
            return self.max_kv_bound
        return max(self.kv_lens) if self.kv_lens else 0


class Part:
    """Base of every part: owns parameters, bound after loading.

    ``graph_safe``: the part's ``forward`` may be captured into a CUDA graph and replayed
    for other steps of the same shape, i.e. everything that changes from step to step is
    read on the device from the step's tensors, nothing from host-side lists.  The
    built-in parts are; a part that does not say so keeps its model out of graphs."""

    graph_safe = False

    def __init__(self, spec: Any, dtype: torch.dtype):
        self.spec = spec
        self.dtype = dtype

    def parameters(self) -> dict:
        """``{local name: ParamSpec}``."""
        return {}

    def bind(self, tensors: dict) -> None:
        """Receive the loaded parameters (device tensors, final dtype)."""
        for name, t in tensors.items():
            setattr(self, name, t)


class Norm(Part):
    def forward(self, x, residual=None):
        """Return ``(normed, new_residual)``; without a residual, ``new_residual = x``."""
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Mixer(Part):
    # most entries (requests) one step may bring, if the mixer's kernels bound it (None: any)
    max_step_entries = None

    def kv_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, x: torch.Tensor, step: StepContext, slot: LayerSlot) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        raise NotImplementedError


MIXERS: dict = {}
FEED_FORWARDS: dict = {}
NORMS: dict = {}
POSITIONS: dict = {}


def register_mixer(kind: str, cls) -> None:
    MIXERS[kind] = cls


def register_feed_forward(kind: str, cls) -> None:
    FEED_FORWARDS[kind] = cls


def register_norm(kind: str, cls) -> None:
    NORMS[kind] = cls


def register_position(kind: str, cls) -> None:
    POSITIONS[kind] = cls


def _make(registry: dict, what: str, spec: Any, dtype: torch.dtype):
    kind = getattr(spec, "kind", None)
    if kind not in registry:
        raise ValueError(f"no {what} registered for kind {kind!r}; known: {sorted(registry)}")
    return registry[kind](spec, dtype)


def make_mixer(spec, dtype):
    return _make(MIXERS, "mixer", spec, dtype)


def make_feed_forward(spec, dtype):
    return _make(FEED_FORWARDS, "feed-forward", spec, dtype)


def make_norm(spec, dtype):
    return _make(NORMS, "norm", spec, dtype)


def make_position(spec, dtype):
    return _make(POSITIONS, "position encoding", spec, dtype)


__all__ = ["KVRequest", "StateRequest", "LayerSlot", "StepContext", "Part", "Norm", "PositionEncoding",
           "Mixer", "FeedForward", "ParamSpec", "register_mixer", "register_feed_forward", "register_norm",
           "register_position", "make_mixer", "make_feed_forward", "make_norm", "make_position",
           "MIXERS", "FEED_FORWARDS", "NORMS", "POSITIONS"]
