"""Host-side bookkeeping of the cache: pages, request slots, block tables.

Nothing here touches the device.  ``KVCacheManager`` in ``kv_cache.py`` pairs these tables
with the device tensors.

* ``PagePool``: a LIFO free list over pages ``1..num_pages`` (page 0 is never handed out: a
  zero in a block table means "no page", as index 0 does in lily/mem_cache/memory_pool.py:1-7).
  LIFO, so that a page given back is the next one handed out and stale contents meet new
  requests early.  A page freed twice, or one that was never handed out, raises.
* ``SlotPool``: request slots ``1..max_requests`` (slot 0 stays empty so that padded rows of a
  captured decode graph can point at it, lily/mem_cache/memory_pool.py:21-30).
* ``BlockTable``: for one request in one cache group, the page that holds each run of
  ``page_size`` positions.  In a group with a window, pages wholly behind the window are
  given back while the request lives; their entries become 0 and are never read again.
"""

from __future__ import annotations

import itertools

from typing import Dict, List, Optional


class OutOfPages(RuntimeError):
    """The pool cannot supply the pages a step needs (the scheduler decides what happens next)."""


class OutOfSlots(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages, 0, -1))      # pop() hands out 1, 2, 3, ...
        self._held = bytearray(num_pages + 1)

    @property
    def available(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = 1
        return out

    def free(self, pages) -> None:
        for p in pages:
            if not (1 <= p <= self.num_pages) or not self._held[p]:
                raise RuntimeError(f"page {p} freed but not held")
            self._held[p] = 0
            self._free.append(p)

    def held(self) -> int:
        return self.num_pages - len(self._free)


class SlotPool:
    def __init__(self, max_requests: int):
        self.max_requests = max_requests
        self._free: List[int] = list(range(max_requests, 0, -1))
        self._held = bytearray(max_requests + 1)

    @property
    def available(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.max_requests} request slots are in use")
        s = self._free.pop()
        self._held[s] = 1
        return s

    def free(self, slot: int) -> None:
        if not (1 <= slot <= self.max_requests) or not self._held[slot]:
            raise RuntimeError(f"request slot {slot} freed but not held")
        self._held[slot] = 0
        self._free.append(slot)


class BlockTable:
    """Pages of one request in one group.  ``pages[i]`` holds positions
    ``[i * page_size, (i + 1) * page_size)``; 0 after the window has passed them."""

    __slots__ = ("pages", "first_live", "stamp")
    _stamps = itertools.count(1)

    def __init__(self):
        self.pages: List[int] = []
        self.first_live = 0          # index of the first page not yet given back
        self.stamp = next(BlockTable._stamps)      # a new number whenever the table changes; no two tables share one

    def touch(self) -> None:
        self.stamp = next(BlockTable._stamps)

    def live_pages(self) -> List[int]:
        return [p for p in self.pages[self.first_live:] if p]


def pages_for(length: int, page_size: int) -> int:
    return -(-length // page_size)


class GroupTables:
    """All block tables of one cache group, over one page pool."""

    def __init__(self, num_pages: int, page_size: int, window: Optional[int] = None):
        self.pool = PagePool(num_pages)
        self.page_size = page_size
        self.window = window
        self.tables: Dict[int, BlockTable] = {}

    def open(self, slot: int) -> None:
        if slot in self.tables:
            raise RuntimeError(f"slot {slot} is already open")
        self.tables[slot] = BlockTable()

    def pages_needed(self, slot: int, new_len: int) -> int:
        """Pages that must be taken from the pool for the request to hold ``new_len`` positions."""
        return max(0, pages_for(new_len, self.page_size) - len(self.tables[slot].pages))

    def grow(self, slot: int, new_len: int) -> None:
        t = self.tables[slot]
        need = pages_for(new_len, self.page_size) - len(t.pages)
        if need > 0:
            t.pages.extend(self.pool.alloc(need))
            t.touch()

    def pass_window(self, slot: int, seq_len: int) -> int:
        """Gives back the pages no later query can see: with ``seq_len`` positions cached, the
        next query sits at ``seq_len`` or later and sees keys ``> seq_len - window`` only."""
        if self.window is None:
            return 0
        t = self.tables[slot]
        first_needed = max(0, seq_len - self.window + 1) // self.page_size
        first_needed = min(first_needed, len(t.pages))
        gone = [p for p in t.pages[t.first_live:first_needed] if p]
        for i in range(t.first_live, first_needed):
            t.pages[i] = 0
        if first_needed > t.first_live:
            t.touch()
        t.first_live = max(t.first_live, first_needed)
        self.pool.free(gone)
        return len(gone)

    def close(self, slot: int) -> None:
        t = self.tables.pop(slot)
        self.pool.free(t.live_pages())
