"""The step function: one batch of (request, its next tokens) → logits at the wanted
places.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.  Only
the tokens given are run; everything earlier comes from the cache.  Sampling is not
done here.  The reference's runner takes either prompt chunks or decode tokens per step
and samples inside (src/sparseengine/engine/model_runner.py:2572-2660; inputs built in
src/sparseengine/engine/cache_manager/standard.py:2065-2206); this one takes any mix and
returns logits.

Per step: reserve pages (all or nothing) → pack the step's metadata into one pinned
int32 buffer → one host-to-device copy → apply block-table updates → model forward →
commit the tokens to the cache manager.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..csrc import ops
from ..parts.base import StepContext
from .model import Model


@dataclass
class StepEntry:
    """A request's next tokens in this step and the places (indices into ``tokens``)
    whose logits are wanted."""
    seq_id: object
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


class _Staging:
    """A small ring of pinned host buffers, each guarded by an event so that a buffer is
    not rewritten while its copy may still be in flight."""

    def __init__(self, depth: int = 4):
        self.depth = depth
        self.bufs = [None] * depth
        self.events = [None] * depth
        self.i = 0

    def get(self, n: int):
        i = self.i
        self.i = (i + 1) % self.depth
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.bufs[i] is None or self.bufs[i].numel() < n:
            self.bufs[i] = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=True)
        return i, self.bufs[i]

    def mark(self, i: int):
        if self.events[i] is None:
            self.events[i] = torch.cuda.Event()
        self.events[i].record()


@dataclass
class _DecodeGraph:
    graph: object
    meta: torch.Tensor            # persistent device copy of the step's packed metadata
    logits: torch.Tensor          # static output of the captured forward
    kernels: int = 0              # kernels of this library that one replay launches


class ModelRunner:
    KV_BUCKET = 512               # decode graphs are planned for context lengths rounded up to this
    MAX_GRAPHS = 64               # captured graphs kept (least recently used go first)

    def __init__(self, model: Model, cache: CacheManager, device="cuda:0", decode_graphs: bool = True):
        self.model = model
        self.cache = cache
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        for b in model.blocks:
            most = getattr(b.parts().get("mixer"), "max_step_entries", None)
            if most is not None and cache.max_rows > most:
                raise ValueError(f"{cache.max_rows} resident requests are not supported: a step takes at most {most} "
                                 f"entries ({type(b.parts()['mixer']).__name__})")
        self.slots = [cache.slot_for(e) for e in model.layout.entries]
        self._staging = _Staging()
        self.steps = 0
        self.tokens = 0
        # Decode-only steps (every entry brings one token) replay a CUDA graph per
        # (batch size, context bucket); anything else runs launch by launch.
        parts = [p for b in model.blocks for p in b.parts().values()] + [model.final_norm]
        self.decode_graphs = bool(decode_graphs) and all(getattr(p, "graph_safe", False) for p in parts)
        self._graphs: dict = {}
        self._graph_pool = None
        self.graph_replays = 0
        self.validate = False          # host-side checks of every step's indices (a debugging aid)

    # ---- life cycle of a request -------------------------------------------------------
    def admit(self, seq_id) -> None:
        self.cache.admit(seq_id)

    def release(self, seq_id) -> None:
        self.cache.release(seq_id)

    # ---- the step ------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], token_feedback: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch.  Returns logits ``[wanted, vocab]`` (activation dtype) in the
        order of the entries and of each entry's ``want``, or ``None`` if nothing is wanted.

        ``token_feedback``: for a step of single tokens, an int32 device tensor with the entries'
        tokens in their order (the ids a sampler has just written): the step is then queued
        without the host knowing them; the entries' own ``tokens`` are placeholders.

        Raises :class:`OutOfPages` (and changes nothing) if the pages do not suffice.
        The returned tensor may be overwritten by the next step."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        vocab = self.model.spec.vocab_size
        seen = set()
        for e in entries:
            if e.seq_id in seen:
                raise ValueError(f"request {e.seq_id!r} appears twice in one step")
            seen.add(e.seq_id)
            if not self.cache.has(e.seq_id):
                raise ValueError(f"request {e.seq_id!r} was not admitted")
            if min(e.tokens) < 0 or max(e.tokens) >= vocab:
                raise ValueError(f"request {e.seq_id!r}: token id outside [0, {vocab})")
            if any(not 0 <= w < len(e.tokens) for w in e.want):
                raise ValueError(f"request {e.seq_id!r}: wanted place outside its tokens")
        done = []
        try:
            for e in entries:
                self.cache.reserve(e.seq_id, len(e.tokens))
                done.append(e.seq_id)
        except (OutOfPages, ValueError):
            for s in done:
                self.cache.cancel(s)
            raise

        try:
            if self.validate:
                self._check_invariants(entries)
            if self.decode_graphs and all(len(e.tokens) == 1 for e in entries):
                logits = self._step_graph(entries, token_feedback)
            else:
                logits = None
            if logits is None:
                if token_feedback is not None:       # no graph for this step: the host has to see the tokens after all
                    for e, t in zip(entries, token_feedback.tolist()):
                        e.tokens = [int(t)]
                step, want_rows, updates = self._pack(entries)
                with torch.cuda.device(self.device):
                    for g, (upd, n) in zip(self.cache.groups, updates):
                        if n:
                            ops.table_update(g.table, upd, n, g.pool.num_pages)
                    logits = self.model.forward(step, self.slots, want_rows)
        except BaseException:
            # the step did not happen: give back what was reserved for it
            # (cf. src/sparseengine/engine/llm_engine.py:1826-1857)
            for e in entries:
                self.cache.cancel(e.seq_id)
            raise
        for e in entries:
            self.cache.commit(e.seq_id, len(e.tokens))
        self.steps += 1
        self.tokens += sum(len(e.tokens) for e in entries)
        return logits

    def _check_invariants(self, entries) -> None:
        """Host-side validation of what the kernels will index with: every position a step
        reads or writes has a page, pages are inside their pool, no page belongs to two
        requests, lengths stay under the limit (the reference's debug bounds checks,
        src/sparseengine/layers/attention_backend.py:155-215)."""
        self.cache.check()
        for e in entries:
            row, start = self.cache.row(e.seq_id), self.cache.length(e.seq_id)
            end = start + len(e.tokens)
            if end > self.cache.max_seq_len:
                raise AssertionError(f"request {e.seq_id!r} would exceed the maximum length")
            for g in self.cache.groups:
                lo = 0 if g.window is None else max(0, start - g.window + 1)
                idx = np.arange(lo // g.page_size, -(-end // g.page_size))
                pages = g.table_host[row, idx]
                if (pages < 0).any() or (pages >= g.pool.num_pages).any():
                    raise AssertionError(f"request {e.seq_id!r}: block table has no valid page for positions {lo}..{end - 1}")

    # ---- decode steps as replayed CUDA graphs ------------------------------------------
    def _step_graph(self, entries, token_feedback=None):
        """Run a decode-only step through a captured graph.  Returns the logits of the wanted
        rows, or ``None`` if this step cannot use a graph (too many block-table updates
        pending, or capture is not possible), in which case nothing has been done."""
        n = len(entries)
        groups = self.cache.groups
        if any(len(g.pending) > n for g in groups):
            return None
        q_starts = [self.cache.length(e.seq_id) for e in entries]
        bound = -(-(max(q_starts) + 1) // self.KV_BUCKET) * self.KV_BUCKET
        key = (n, bound)
        # fixed layout for n entries: ids, positions, token->entry, rows, cu_q, kv_len, wanted rows,
        # then per group one count word and up to n update triples
        sizes = [n, n, n, n, n + 1, n, n] + [4, 3 * n] * len(groups)
        offs = np.concatenate(([0], np.cumsum([-(-s // 4) * 4 for s in sizes]))).astype(np.int64)
        total = int(offs[-1])
        slot, host = self._staging.get(total)
        h = host.numpy()
        rows = [self.cache.row(e.seq_id) for e in entries]
        h[offs[0]:offs[0] + n] = [e.tokens[0] for e in entries]
        h[offs[1]:offs[1] + n] = q_starts
        h[offs[2]:offs[2] + n] = np.arange(n, dtype=np.int32)
        h[offs[3]:offs[3] + n] = rows
        h[offs[4]:offs[4] + n + 1] = np.arange(n + 1, dtype=np.int32)
        h[offs[5]:offs[5] + n] = [s + 1 for s in q_starts]
        h[offs[6]:offs[6] + n] = np.arange(n, dtype=np.int32)
        for gi in range(len(groups)):
            u = self.cache.drain_updates(gi)
            h[offs[7 + 2 * gi]] = len(u)
            if u:
                h[offs[8 + 2 * gi]:offs[8 + 2 * gi] + 3 * len(u)] = np.asarray(u, dtype=np.int32).reshape(-1)

        with torch.cuda.device(self.device):
            entry = self._graphs.get(key)
            meta = entry.meta if entry is not None else torch.empty(total, dtype=torch.int32, device=self.device)
            meta.copy_(host[:total], non_blocking=True)
            self._staging.mark(slot)
            if token_feedback is not None:
                meta[int(offs[0]):int(offs[0]) + n].copy_(token_feedback[:n])

            def view(i, length):
                return meta[int(offs[i]):int(offs[i]) + length]

            def forward():
                step = StepContext(
                    num_tokens=n, num_seqs=n, token_ids=view(0, n), positions=view(1, n), token_seq=view(2, n),
                    seq_rows=view(3, n), cu_q=view(4, n + 1), kv_len=view(5, n), q_lens=[1] * n,
                    q_starts=list(q_starts), kv_lens=[s + 1 for s in q_starts], rows=list(rows),
                    dtype=self.model.dtype, max_kv_bound=bound)
                for gi, g in enumerate(groups):
                    ops.table_update_dyn(g.table, view(8 + 2 * gi, 3 * n), view(7 + 2 * gi, 1), n, g.pool.num_pages)
                return self.model.forward(step, self.slots, view(6, n))

            if entry is None:
                logits = forward()                       # this step's work, launch by launch
                try:
                    graph = torch.cuda.CUDAGraph()
                    if self._graph_pool is None:
                        self._graph_pool = torch.cuda.graph_pool_handle()
                    torch.cuda.synchronize(self.device)
                    before = ops.launch_count
                    with torch.cuda.graph(graph, pool=self._graph_pool):
                        static_logits = forward()        # recorded, not run
                    recorded = ops.launch_count - before
                    ops.launch_count = before            # nothing ran during capture
                    self._graphs[key] = _DecodeGraph(graph, meta, static_logits, recorded)
                    while len(self._graphs) > self.MAX_GRAPHS:          # dicts keep insertion order
                        self._graphs.pop(next(iter(self._graphs)))
                except Exception as exc:                 # capture is an optimisation only
                    self.decode_graphs = False
                    print(f"[sparseengine_b200] CUDA graph capture failed ({exc!r}); decode runs without graphs",
                          flush=True)
            else:
                self._graphs[key] = self._graphs.pop(key)               # most recently used last
                entry.graph.replay()
                self.graph_replays += 1
                ops.launch_count += entry.kernels
                logits = entry.logits
        want = [i for i, e in enumerate(entries) for _ in e.want]
        if not want:
            return logits[:0]
        if want == list(range(n)):
            return logits
        return logits[torch.tensor(want, device=self.device)]

    def _pack(self, entries):
        n = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        t = sum(q_lens)
        q_starts = [self.cache.length(e.seq_id) for e in entries]
        rows = [self.cache.row(e.seq_id) for e in entries]
        kv_lens = [s + q for s, q in zip(q_starts, q_lens)]
        want = []
        base = 0
        for e, q in zip(entries, q_lens):
            want.extend(base + w for w in e.want)
            base += q
        upd = [self.cache.drain_updates(g) for g in range(len(self.cache.groups))]

        # layout of the packed buffer (all int32)
        sizes = [t, t, t, n, n + 1, n, len(want)] + [3 * len(u) for u in upd]
        offs = np.concatenate(([0], np.cumsum([-(-s // 4) * 4 for s in sizes]))).astype(np.int64)
        total = int(offs[-1])
        slot, host = self._staging.get(total)
        h = host.numpy()
        tok = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        h[offs[0]:offs[0] + t] = tok
        h[offs[1]:offs[1] + t] = np.concatenate([np.arange(s, s + q, dtype=np.int32) for s, q in zip(q_starts, q_lens)])
        h[offs[2]:offs[2] + t] = np.repeat(np.arange(n, dtype=np.int32), q_lens)
        h[offs[3]:offs[3] + n] = rows
        h[offs[4]:offs[4] + n + 1] = np.concatenate(([0], np.cumsum(q_lens))).astype(np.int32)
        h[offs[5]:offs[5] + n] = kv_lens
        if want:
            h[offs[6]:offs[6] + len(want)] = want
        for i, u in enumerate(upd):
            if u:
                h[offs[7 + i]:offs[7 + i] + 3 * len(u)] = np.asarray(u, dtype=np.int32).reshape(-1)
        with torch.cuda.device(self.device):
            dev = torch.empty(total, dtype=torch.int32, device=self.device)
            dev.copy_(host[:total], non_blocking=True)
            self._staging.mark(slot)

        def view(i, length):
            return dev[int(offs[i]):int(offs[i]) + length]

        step = StepContext(
            num_tokens=t, num_seqs=n, token_ids=view(0, t), positions=view(1, t), token_seq=view(2, t),
            seq_rows=view(3, n), cu_q=view(4, n + 1), kv_len=view(5, n), q_lens=q_lens, q_starts=q_starts,
            kv_lens=kv_lens, rows=rows, dtype=self.model.dtype)
        want_rows = view(6, len(want)) if want else None
        updates = [(view(7 + i, 3 * len(u)), len(u)) for i, u in enumerate(upd)]
        return step, want_rows, updates
