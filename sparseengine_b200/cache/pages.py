"""A pool of fixed-size pages with a last-in-first-out free list.

Pages that are given back are the first to be taken again, so a small pool reuses
pages at once.  Every page is either free or held exactly once: taking more than is
free fails without taking any, giving back a page that is not held is an error.
The reference's nearest objects are the slot stack of its dense manager
(src/sparseengine/engine/cache_manager/standard.py:128-129,1637-1653) and
``PhysicalPageAllocator`` (src/sparseengine/engine/cache_manager/storage/page_allocator.py:6-68).
"""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """Not enough free pages (or rows) for what was asked; nothing was taken."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))   # pop() gives page 0 first
        self._held = bytearray(self.num_pages)
        self._used_before = bytearray(self.num_pages)
        self.taken_total = 0
        self.reused_total = 0      # pages taken that some request had held before

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int) -> list[int]:
        if n < 0:
            raise ValueError("cannot take a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = 1
            self.reused_total += self._used_before[p]
            self._used_before[p] = 1
        self.taken_total += n
        return out

    def give(self, pages) -> None:
        pages = list(pages)
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not of this pool")
            if not self._held[p]:
                raise ValueError(f"page {p} is given back but not held")
            self._held[p] = 0
        # the last page given back is the next one taken
        self._free.extend(pages)

    def check(self) -> None:
        """Raise if the pool's books do not balance (used by tests)."""
        if len(set(self._free)) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        if any(self._held[p] for p in self._free):
            raise AssertionError("a free page is marked held")
        if sum(self._held) + len(self._free) != self.num_pages:
            raise AssertionError("pages were lost")
