"""Host-side bookkeeping of the cache: slots, pages, block tables.  No GPU here.

A *slot* belongs to one live sequence: a row of every group's block table, a
length, and a row of the fixed-size state region.  A *page* holds `page_size`
consecutive positions of one sequence for every layer of one group.  Slots
and pages are handed out lowest-first from LIFO stacks and given back when
the sequence ends, so that later sequences use them again.

Upstream keeps one table per layer with the batch size frozen at
construction, maps pages lazily, never gives a page back and never checks for
exhaustion (src/kvcache.h:40-61,117-122; src/src-cuda/kvcache.cu:46-55).
"""
from __future__ import annotations

from typing import Optional

import numpy as np


class CacheError(RuntimeError):
    """The cache cannot do what was asked: it is full, or a slot was misused."""


class SlotAllocator:
    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise CacheError(f"a cache needs at least one slot, not {n_slots}")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))     # pop() gives the lowest
        self._live: set[int] = set()

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"all {self.n_slots} slots are in use")
        s = self._free.pop()
        self._live.add(s)
        return s

    def free(self, slot: int) -> None:
        if slot not in self._live:
            raise CacheError(f"slot {slot} is not in use (freed twice, or never given out)")
        self._live.remove(slot)
        self._free.append(slot)

    def is_live(self, slot: int) -> bool:
        return slot in self._live

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def live(self) -> frozenset:
        return frozenset(self._live)


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, not {n_pages}")
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self._out = np.zeros(n_pages, dtype=bool)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"all {self.n_pages} cache pages are in use")
        p = self._free.pop()
        self._out[p] = True
        return p

    def give(self, page: int) -> None:
        if page < 0 or page >= self.n_pages or not self._out[page]:
            raise CacheError(f"page {page} is not in use (given back twice, or never taken)")
        self._out[page] = False
        self._free.append(page)


class GroupTable:
    """Block table of one group of layers: which pool page holds each logical page of each slot.

    With a `window` of w keys, positions that no later query can see (those
    below length - w + 1 once a step is done) are dropped page by page and
    their pages go back to the pool."""

    def __init__(self, n_pages: int, page_size: int, max_slots: int, max_pages_per_seq: int,
                 window: Optional[int] = None):
        self.page_size = page_size
        self.window = window
        self.pool = PagePool(n_pages)
        self.table = np.full((max_slots, max_pages_per_seq), -1, dtype=np.int32)
        self.first_page = np.zeros(max_slots, dtype=np.int64)   # logical pages below are dropped
        self.end_page = np.zeros(max_slots, dtype=np.int64)     # logical pages below are mapped (or dropped)
        self.dirty: set[int] = set()

    def pages_needed(self, slot: int, new_len: int) -> int:
        want_end = -(-new_len // self.page_size)
        return max(0, want_end - int(self.end_page[slot]))

    def reserve(self, slot: int, new_len: int) -> None:
        """Map pages so that positions below `new_len` have a home.  The caller has checked the pool."""
        want_end = -(-new_len // self.page_size)
        if want_end > self.table.shape[1]:
            raise CacheError(f"a sequence of {new_len} positions needs {want_end} pages; the block table "
                             f"holds {self.table.shape[1]} per sequence")
        for lp in range(int(self.end_page[slot]), want_end):
            self.table[slot, lp] = self.pool.take()
            self.dirty.add(slot)
        self.end_page[slot] = max(int(self.end_page[slot]), want_end)

    def trim(self, slot: int, length: int) -> None:
        """After a step that brought the sequence to `length`: drop pages wholly out of the window."""
        if self.window is None:
            return
        keep_from = max(0, length - self.window + 1) // self.page_size
        for lp in range(int(self.first_page[slot]), min(keep_from, int(self.end_page[slot]))):
            self.pool.give(int(self.table[slot, lp]))
            self.table[slot, lp] = -1
            self.dirty.add(slot)
        self.first_page[slot] = max(int(self.first_page[slot]), min(keep_from, int(self.end_page[slot])))

    def release(self, slot: int) -> None:
        for lp in range(int(self.first_page[slot]), int(self.end_page[slot])):
            self.pool.give(int(self.table[slot, lp]))
            self.table[slot, lp] = -1
        if self.end_page[slot] > self.first_page[slot]:
            self.dirty.add(slot)
        self.first_page[slot] = 0
        self.end_page[slot] = 0

    def pages_of(self, slot: int) -> list[int]:
        return [int(p) for p in self.table[slot, int(self.first_page[slot]):int(self.end_page[slot])]]
