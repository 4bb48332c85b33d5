"""A model assembled from a :class:`ModelSpec`: embedding, blocks in their execution
order, final norm, LM head.  Architecture-agnostic.

The loop mirrors src/sparseengine/models/qwen3.py:291-328 (embed → layers → final fused
add+norm) and src/sparseengine/layers/embed_head.py:75-84 (LM head on selected rows
only); here the rows are whatever the caller asks for, and the final norm also runs on
those rows only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config.specs import ModelSpec, ParamSpec, Source
from ..csrc import ops
from ..parts.base import KVRequest, StateRequest, StepContext, make_norm
from ..parts.block import PreNormBlock, make_block
from ..parts.linear import linear


@dataclass
class Param:
    """A parameter with its owner and the checkpoint tensors that fill it."""
    owner: object
    name: str            # attribute on the owner
    qualified: str       # unique name for messages, e.g. "layers.3.mixer.qkv"
    spec: ParamSpec
    sources: tuple       # tuple[Source, ...]
    tensor: Optional[torch.Tensor] = None


@dataclass(frozen=True)
class EntryCache:
    """Where a schedule entry keeps keys/values and state."""
    group: Optional[int]         # index into CacheLayout.groups
    cache_layer: Optional[int]   # layer index inside the group's storage
    write: bool
    state: Optional[int]         # index into CacheLayout.states


@dataclass(frozen=True)
class CacheLayout:
    groups: tuple        # tuple[(KVRequest, number of cache layers)]
    states: tuple        # tuple[StateRequest], one per schedule entry that has state
    entries: tuple       # tuple[EntryCache], one per schedule entry


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"engine dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.blocks = [make_block(ls, dtype) for ls in spec.layers]
        self.final_norm = make_norm(spec.final_norm, dtype)
        self.embed = None
        self.head = None
        self.profile = None     # a dict: CUDA-event pairs per part are collected in it (a debugging aid)
        for i, e in enumerate(spec.order):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.blocks)}")
            if e.cache is not None and not 0 <= e.cache < i:
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache}, which is not earlier")
        self.layout = self._cache_layout()

    # ---- parameters --------------------------------------------------------------------
    def params(self) -> list[Param]:
        s = self.spec
        out = [Param(self, "embed", "embed", ParamSpec((s.vocab_size, s.hidden_size)), (Source(s.embed_source),))]
        if s.head_source is not None:
            out.append(Param(self, "head", "head", ParamSpec((s.vocab_size, s.hidden_size)),
                             (Source(s.head_source),)))
        for name, p in self.final_norm.parameters().items():
            out.append(Param(self.final_norm, name, f"final_norm.{name}", p, (Source(s.final_norm_source),)))
        for i, (block, ls) in enumerate(zip(self.blocks, s.layers)):
            for part_name, part in block.parts().items():
                for name, p in part.parameters().items():
                    key = f"{part_name}.{name}"
                    if key not in ls.sources:
                        raise ValueError(f"layer {i}: no checkpoint source given for parameter {key!r}")
                    out.append(Param(part, name, f"layers.{i}.{key}", p, tuple(ls.sources[key])))
        return out

    def bind(self, params: list[Param]) -> None:
        by_owner: dict = {}
        for p in params:
            if p.tensor is None:
                raise ValueError(f"parameter {p.qualified} was not loaded")
            by_owner.setdefault(id(p.owner), (p.owner, {}))[1][p.name] = p.tensor
        for owner, tensors in by_owner.values():
            if owner is self:
                for n, t in tensors.items():
                    setattr(self, n, t)
            else:
                owner.bind(tensors)
        if self.spec.head_source is None:
            self.head = self.embed

    def param_dtype(self, p: ParamSpec) -> torch.dtype:
        return torch.float32 if p.dtype == "float32" else self.dtype

    # ---- cache needs -------------------------------------------------------------------
    def _cache_layout(self) -> CacheLayout:
        groups: list = []          # [KVRequest, count]
        states: list = []
        entries: list = []
        for e in self.spec.order:
            mixer = self.blocks[e.layer].mixer
            kv = mixer.kv_request()
            st = mixer.state_request()
            group = layer = None
            if kv is not None:
                if e.cache is not None:
                    owner = entries[e.cache]
                    if owner.group is None or groups[owner.group][0] != kv:
                        raise ValueError("a schedule entry can only share a cache of the same shape and window")
                    group, layer = owner.group, owner.cache_layer
                else:
                    for gi, (req, _) in enumerate(groups):
                        if req == kv:
                            group = gi
                            break
                    else:
                        groups.append([kv, 0])
                        group = len(groups) - 1
                    layer = groups[group][1]
                    groups[group][1] += 1
            state = None
            if st is not None:
                states.append(st)
                state = len(states) - 1
            write = e.write_cache and e.cache is None
            entries.append(EntryCache(group, layer, write if kv is not None else False, state))
        return CacheLayout(tuple((g[0], g[1]) for g in groups), tuple(states), tuple(entries))

    def _timed_block(self, block, hidden, residual, step, slot):
        """The pre-norm block part by part with a CUDA event pair around each part."""
        def timed(name, fn, *a):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a)
            e1.record()
            self.profile.setdefault(name, []).append((e0, e1))
            return out
        if not isinstance(block, PreNormBlock):
            return timed("block", block.forward, hidden, residual, step, slot)
        x, residual = timed("mixer_norm", block.mixer_norm.forward, hidden, residual)
        hidden = timed("mixer", block.mixer.forward, x, step, slot)
        x, residual = timed("feed_forward_norm", block.feed_forward_norm.forward, hidden, residual)
        hidden = timed("feed_forward", block.feed_forward.forward, x, step)
        return hidden, residual

    # ---- forward -----------------------------------------------------------------------
    def forward(self, step: StepContext, slots: list, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every schedule entry; return logits
        ``[len(want_rows), vocab]`` in the activation dtype, or ``None`` if no row is wanted."""
        s = self.spec
        hidden = torch.empty(step.num_tokens, s.hidden_size, dtype=self.dtype, device=step.token_ids.device)
        ops.embed_gather(self.embed, step.token_ids, hidden)
        if s.embed_scale != 1.0:
            hidden.mul_(s.embed_scale)
        residual = None
        for entry, slot in zip(s.order, slots):
            block = self.blocks[entry.layer]
            if self.profile is None:
                hidden, residual = block.forward(hidden, residual, step, slot)
            else:
                hidden, residual = self._timed_block(block, hidden, residual, step, slot)
        if want_rows is None or want_rows.numel() == 0:
            return None
        n = want_rows.numel()
        h = torch.empty(n, s.hidden_size, dtype=self.dtype, device=hidden.device)
        ops.gather_rows(hidden, want_rows, h)
        if residual is not None:
            r = torch.empty_like(h)
            ops.gather_rows(residual, want_rows, r)
            h, _ = self.final_norm.forward(h, r)
        else:
            h, _ = self.final_norm.forward(h)
        logits = linear(h, self.head)
        if s.logit_softcap is not None:
            c = float(s.logit_softcap)
            logits = (torch.tanh(logits.float() / c) * c).to(logits.dtype)
        return logits
