"""The cache manager: paged keys/values with a block table per request, one group of
pages per kind of layer, and fixed-size per-request state slots.

* A **group** serves all cache layers whose mixers asked for the same thing
  (:class:`~sparseengine_b200.parts.base.KVRequest`: heads, head size, window).  It owns
  a page pool, a storage tensor ``[cache layers, pages, 2, kv heads, page_size, head_dim]``
  and a block table ``[rows, max pages per request]`` (int32, on the device, with a host
  mirror).  Page ``table[row, i]`` holds the request's positions
  ``i*page_size .. (i+1)*page_size-1`` in every cache layer of the group.
* A request is **admitted** (gets a row and zeroed state slots), **reserves** pages for
  its next tokens before a step (all groups or none), **commits** them after the step
  (a windowed group then gives back the pages no later query can see) and is
  **released** when it ends (everything returns to the pools).
* **State slots**: ``state[i][row]`` is a tensor of fixed shape per request for schedule
  entries whose mixer declared a :class:`StateRequest`.  The dense-cache attention of
  MiniMax M2 declares none; the slots exist for mixers with state of their own.

Block-table changes are queued as ``(row, index, page)`` triples; the step function
uploads them with the rest of the step's metadata and a kernel applies them.

Reference: src/sparseengine/engine/cache_manager/standard.py:106-170 (rows, slot stack),
:1752-1859 (allocation at prepare_step, rollback), :1950-1999 (free_seq);
src/sparseengine/engine/recurrent_state_manager.py (per-row fixed-size state).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from .pages import OutOfPages, PagePool


@dataclass
class _Request:
    row: int
    length: int = 0
    pages: list = field(default_factory=list)       # per group: {table index: page}
    reserved: int = 0                                # tokens reserved and not yet committed


class CacheGroup:
    def __init__(self, request, cache_layers: int, num_pages: int, page_size: int, max_rows: int,
                 max_pages_per_seq: int, dtype, device, allocate: bool):
        self.request = request
        self.cache_layers = cache_layers
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.table_host = np.full((max_rows, max_pages_per_seq), -1, dtype=np.int32)
        self.pending: list = []      # (row, index, page)
        self.storage = None
        self.table = None
        if allocate:
            self.storage = torch.zeros(cache_layers, num_pages, 2, request.num_kv_heads, page_size,
                                       request.head_dim, dtype=dtype, device=device)
            self.table = torch.zeros(max_rows, max_pages_per_seq, dtype=torch.int32, device=device)

    @property
    def window(self) -> Optional[int]:
        return self.request.window

    def bytes_per_page(self, itemsize: int) -> int:
        r = self.request
        return self.cache_layers * 2 * r.num_kv_heads * self.page_size * r.head_dim * itemsize


class CacheManager:
    def __init__(self, layout, *, page_size: int, num_pages, max_rows: int, max_seq_len: int,
                 dtype=torch.float32, device="cpu", allocate: bool = True, reserved_state_bytes: int = 0):
        """``layout`` is a model's :class:`CacheLayout`; ``num_pages`` an int (every group)
        or a list with one entry per group.  ``reserved_state_bytes`` adds one more slot of
        that many bytes per request (``reserved_state[row]``, zeroed at admission) that no
        part of the dense-cache path uses: it is the room a sparse cache method would keep
        its per-request metadata in."""
        if page_size <= 0 or max_rows <= 0 or max_seq_len <= 0:
            raise ValueError("page_size, max_rows and max_seq_len must be positive")
        self.layout = layout
        self.page_size = int(page_size)
        self.max_rows = int(max_rows)
        self.max_seq_len = int(max_seq_len)
        self.max_pages_per_seq = -(-self.max_seq_len // self.page_size)
        counts = list(num_pages) if isinstance(num_pages, (list, tuple)) else [num_pages] * len(layout.groups)
        if len(counts) != len(layout.groups):
            raise ValueError("num_pages needs one entry per cache group")
        self.groups = [CacheGroup(req, n_layers, int(c), self.page_size, self.max_rows, self.max_pages_per_seq,
                                  dtype, device, allocate)
                       for (req, n_layers), c in zip(layout.groups, counts)]
        self.states = []
        for st in layout.states:
            self.states.append(torch.zeros((self.max_rows, *st.shape), dtype=st.dtype, device=device)
                               if allocate else None)
        self.reserved_state = None
        if reserved_state_bytes > 0 and allocate:
            self.reserved_state = torch.zeros(self.max_rows, int(reserved_state_bytes), dtype=torch.uint8, device=device)
        self._free_rows = list(range(self.max_rows - 1, -1, -1))
        self._requests: dict = {}

    # ---- queries -----------------------------------------------------------------------
    @property
    def free_rows(self) -> int:
        return len(self._free_rows)

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.free

    def has(self, seq_id) -> bool:
        return seq_id in self._requests

    def length(self, seq_id) -> int:
        return self._requests[seq_id].length

    def row(self, seq_id) -> int:
        return self._requests[seq_id].row

    def live(self) -> list:
        return list(self._requests)

    def pages_needed(self, seq_id, n_tokens: int, length: Optional[int] = None) -> list[int]:
        """New pages per group to hold ``n_tokens`` more tokens of the request (``seq_id``
        may be unknown yet, then ``length`` counts as given, default 0)."""
        if length is None:
            r = self._requests.get(seq_id)
            length = (r.length + r.reserved) if r is not None else 0
        p = self.page_size
        return [-(-(length + n_tokens) // p) - (-(-length // p)) for _ in self.groups]

    def pages_for_tokens(self, n_tokens: int) -> int:
        return -(-n_tokens // self.page_size)

    def can_reserve(self, wants) -> bool:
        """``wants``: iterable of ``(seq_id, n_tokens)``; True if all fit at once."""
        need = [0] * len(self.groups)
        new_rows = 0
        seen: dict = {}
        for seq_id, n in wants:
            r = self._requests.get(seq_id)
            base = seen.get(seq_id, (r.length + r.reserved) if r is not None else 0)
            if r is None and seq_id not in seen:
                new_rows += 1
            for g, k in enumerate(self.pages_needed(seq_id, n, base)):
                need[g] += k
            seen[seq_id] = base + n
        return new_rows <= self.free_rows and all(n <= g.pool.free for n, g in zip(need, self.groups))

    # ---- life cycle --------------------------------------------------------------------
    def admit(self, seq_id) -> int:
        if seq_id in self._requests:
            raise ValueError(f"request {seq_id!r} is already admitted")
        if not self._free_rows:
            raise OutOfPages(f"no free row for request {seq_id!r} ({self.max_rows} rows)")
        row = self._free_rows.pop()
        self._requests[seq_id] = _Request(row=row, pages=[{} for _ in self.groups])
        for st in self.states:
            if st is not None:
                st[row].zero_()
        if self.reserved_state is not None:
            self.reserved_state[row].zero_()
        return row

    def reserve(self, seq_id, n_tokens: int) -> None:
        """Take the pages the request's next ``n_tokens`` tokens need, in every group, or
        none at all (:class:`OutOfPages`)."""
        r = self._requests[seq_id]
        if n_tokens <= 0:
            raise ValueError("a reservation needs at least one token")
        start = r.length + r.reserved
        if start + n_tokens > self.max_seq_len:
            raise ValueError(f"request {seq_id!r} would reach {start + n_tokens} tokens, the limit is "
                             f"{self.max_seq_len}")
        p = self.page_size
        first, last = -(-start // p), -(-(start + n_tokens) // p)
        taken = []
        try:
            for g in self.groups:
                taken.append(g.pool.take(last - first))
        except OutOfPages:
            for g, pages in zip(self.groups, taken):
                g.pool.give(pages)
            raise
        for gi, (g, pages) in enumerate(zip(self.groups, taken)):
            for idx, page in zip(range(first, last), pages):
                r.pages[gi][idx] = page
                g.table_host[r.row, idx] = page
                g.pending.append((r.row, idx, page))
        r.reserved += n_tokens

    def commit(self, seq_id, n_tokens: int) -> None:
        """The step wrote ``n_tokens`` of the reserved tokens.  A windowed group gives
        back every page whose positions no later query can see."""
        r = self._requests[seq_id]
        if n_tokens > r.reserved:
            raise ValueError("commit of more tokens than were reserved")
        r.reserved -= n_tokens
        r.length += n_tokens
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            first_needed = max(0, r.length - g.window + 1)     # the next query's oldest key
            dead = [idx for idx in r.pages[gi] if (idx + 1) * self.page_size <= first_needed]
            if dead:
                g.pool.give([r.pages[gi].pop(idx) for idx in dead])
                for idx in dead:
                    g.table_host[r.row, idx] = -1

    def cancel(self, seq_id) -> None:
        """Undo reservations that were not committed (a step that did not run)."""
        r = self._requests[seq_id]
        if not r.reserved:
            return
        keep = -(-r.length // self.page_size)
        for gi, g in enumerate(self.groups):
            extra = [idx for idx in r.pages[gi] if idx >= keep]
            g.pool.give([r.pages[gi].pop(idx) for idx in extra])
            for idx in extra:
                g.table_host[r.row, idx] = -1
            g.pending = [u for u in g.pending if not (u[0] == r.row and u[1] >= keep)]
        r.reserved = 0

    def release(self, seq_id) -> None:
        """The request ended: its pages and its row go back."""
        r = self._requests.pop(seq_id, None)
        if r is None:
            raise ValueError(f"request {seq_id!r} is not held (released twice?)")
        for gi, g in enumerate(self.groups):
            g.pool.give(list(r.pages[gi].values()))
            g.table_host[r.row, :] = -1
            g.pending = [u for u in g.pending if u[0] != r.row]
        self._free_rows.append(r.row)

    def drain_updates(self, group: int) -> list:
        g = self.groups[group]
        out, g.pending = g.pending, []
        return out

    # ---- views -------------------------------------------------------------------------
    def slot_for(self, entry_cache):
        """The :class:`LayerSlot` of one schedule entry."""
        from ..parts.base import LayerSlot
        slot = LayerSlot()
        if entry_cache.group is not None:
            g = self.groups[entry_cache.group]
            slot.kv = g.storage[entry_cache.cache_layer] if g.storage is not None else None
            slot.table = g.table
            slot.page_size = g.page_size
            slot.write_cache = entry_cache.write
        if entry_cache.state is not None:
            slot.state = self.states[entry_cache.state]
        return slot

    def check(self) -> None:
        """Raise if a page is lost or held twice (used by tests)."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = [p for r in self._requests.values() for p in r.pages[gi].values()]
            if len(held) != len(set(held)):
                raise AssertionError("a page is held by two requests")
            if len(held) != g.pool.held:
                raise AssertionError(f"group {gi}: {g.pool.held} pages held by the pool, {len(held)} by requests")
        rows = [r.row for r in self._requests.values()]
        if len(rows) != len(set(rows)) or len(rows) + len(self._free_rows) != self.max_rows:
            raise AssertionError("rows do not balance")
