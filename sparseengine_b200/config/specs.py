"""Typed descriptions of the parts a model is assembled from.

A model is data: a list of :class:`LayerSpec` (which mixer, feed-forward, norm and
position encoding a layer has, with every size and constant as a field) and an
execution order, a list of :class:`ScheduleEntry` that may name a layer twice or let
an entry read the cache another entry wrote.  Nothing here knows an architecture's
name; architecture builders (``sparseengine_b200.models``) turn a ``config.json``
into these records, and ``sparseengine_b200.parts`` turns the records into parts.

The reference keeps the same facts spread over ``ModelSpec``
(src/sparseengine/models/spec.py:11-211), ``RuntimeLayout``
(src/sparseengine/models/layout.py:77-357) and per-op ``*OpSpec`` records
(src/sparseengine/operators/moe_router.py:19-42, src/sparseengine/operators/moe.py:23-82).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence


@dataclass(frozen=True)
class Source:
    """One checkpoint tensor that fills a slice of a parameter.

    ``index`` addresses the destination along the leading dimensions of the parameter:
    an ``int`` selects (and drops) a dimension, a ``(start, length)`` pair narrows it;
    the remaining dimensions are taken whole.
    """
    name: str
    index: tuple = ()


@dataclass(frozen=True)
class ParamSpec:
    """A parameter a part owns.

    ``dtype`` is ``"act"`` (the engine's activation dtype: bfloat16 or float32) or
    ``"float32"`` (kept in 32-bit whatever the engine dtype, e.g. router weights).
    ``init`` names the random-weights distribution: ``"matrix"`` N(0, std),
    ``"norm"`` 1 + N(0, norm_std), ``"bias"`` N(0, bias_std).
    """
    shape: tuple
    dtype: str = "act"
    init: str = "matrix"
    sources: tuple = ()          # tuple[Source, ...]; filled by the architecture builder


@dataclass(frozen=True)
class RotarySpec:
    kind: str = "rotary"
    rotary_dim: int = 0
    theta: float = 10000.0
    # which dims form rotated pair i: "split_half" (i, i + rotary_dim/2), "interleaved"
    # (2i, 2i+1), "interleaved_to_split_half" (reads 2i, 2i+1; writes i, i + rotary_dim/2)
    pairing: str = "split_half"
    scaling: float = 1.0          # multiplies cos and sin (beside what frequency_scaling brings)
    # the configuration's frequency-scaling entries (linear, llama3, yarn) as a sorted tuple of
    # (key, value) pairs, or None; worked into the frequency table on the host
    frequency_scaling: Optional[tuple] = None


@dataclass(frozen=True)
class RMSNormSpec:
    kind: str = "rms"
    size: int = 0
    eps: float = 1e-6


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged key/value cache."""
    kind: str = "attention"
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    qk_norm: Optional[str] = None     # None | "whole_projection"
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None      # keys p-window+1..p; None = all keys
    position: Optional[Any] = None    # a position-encoding spec (e.g. RotarySpec)


@dataclass(frozen=True)
class MoESpec:
    """Routed SwiGLU experts."""
    kind: str = "moe"
    hidden_size: int = 0
    num_experts: int = 0
    top_k: int = 0
    intermediate_size: int = 0
    score_fn: str = "sigmoid"         # "sigmoid" | "softmax"
    selection_bias: bool = True       # bias added for selection only
    renormalize: bool = True
    routed_scale: float = 1.0
    activation: str = "silu"


@dataclass(frozen=True)
class DenseMLPSpec:
    """A dense SwiGLU feed-forward (one always-selected expert)."""
    kind: str = "dense_mlp"
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its parts and the name of their arrangement in a block.

    The built-in arrangement ``pre_norm`` takes a mixer and a feed-forward between two norms.
    An arrangement with further parts (a norm after each sublayer, a second feed-forward beside
    the first, ...) finds their specs under ``extra`` by the names it gives them, builds them with
    the same registries, and lists them in its ``parts()``; their checkpoint tensors go into
    ``sources`` under "<part name>.<parameter>" like everyone's."""
    mixer: Any
    feed_forward: Any
    mixer_norm: Any
    feed_forward_norm: Any
    arrangement: str = "pre_norm"
    extra: dict = field(default_factory=dict)       # part name -> spec, for arrangements with more parts
    # part-local parameter name -> tuple[Source, ...]; keys are "<part>.<param>" with
    # part in {"mixer", "feed_forward", "mixer_norm", "feed_forward_norm"}.
    sources: dict = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleEntry:
    """One visit of the execution order.

    ``layer`` indexes ``ModelSpec.layers`` (weights).  ``cache`` names the cache layer
    this visit attends over, ``None`` for "a cache layer of its own".  With
    ``write_cache=False`` the visit writes nothing and only reads what the entry that
    owns ``cache`` wrote earlier in the same step (key/value sharing between layers).
    """
    layer: int
    cache: Optional[int] = None
    write_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    layers: Sequence[LayerSpec]
    order: Sequence[ScheduleEntry]
    final_norm: Any
    final_norm_source: str = "model.norm.weight"
    embed_source: str = "model.embed_tokens.weight"
    head_source: Optional[str] = "lm_head.weight"   # None = tied to the embedding
    embed_scale: float = 1.0                        # the embedded tokens are multiplied by this (in the activation type)
    logit_softcap: Optional[float] = None           # c: logits become c * tanh(logits / c), in 32-bit
    ignored_prefixes: tuple = ()                    # checkpoint names skipped at load
    ignored_rule: Optional[Any] = None              # name -> bool: further names skipped at load
    stored_dtype: str = "bfloat16"
