"""Host-side bookkeeping of the cache: which pages and which slots are free, and who holds what.

A page holds the keys and values of ``PAGE`` consecutive positions of one sequence; a slot is a sequence's handle
(its row of the page table, its fixed-size state, its length). Nothing here touches the device, so the rules that
matter - no page or slot is lost, held twice or freed twice - are testable without a GPU.

(The reference keeps one sequence in one contiguous buffer, ``kindi/nanbeige.py:587-594``, and rounds its length to
256 positions, ``:245``; pages of 64 positions give many sequences of unknown final length one pool to share.)
"""
from __future__ import annotations

from typing import Dict, List, Optional

PAGE = 64


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """no free page (or slot) is left: the live sequences hold more than the cache was sized for"""


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


class FreeList:
    """ids 0..n-1; ``take`` hands out the most recently freed id first, so that reuse is exercised early"""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))
        self._held = [False] * n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull("no free %s left (all %d are held)" % (self.what, self.n))
        i = self._free.pop()
        if self._held[i]:
            raise CacheError("%s %d was on the free list while held" % (self.what, i))
        self._held[i] = True
        return i

    def give(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheError("%s %d does not exist (there are %d)" % (self.what, i, self.n))
        if not self._held[i]:
            raise CacheError("%s %d is freed twice (or was never taken)" % (self.what, i))
        self._held[i] = False
        self._free.append(i)

    def held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def check(self) -> None:
        """every id is either free once or held, never both, never neither"""
        seen = [0] * self.n
        for i in self._free:
            seen[i] += 1
        for i in range(self.n):
            if seen[i] + (1 if self._held[i] else 0) != 1:
                raise CacheError("%s %d: on the free list %d times, held=%s" % (self.what, i, seen[i], self._held[i]))


class PageMap:
    """The pages of one group of cache entries: per slot, the page of each block of ``PAGE`` positions.

    ``window`` None keeps all pages of a sequence; otherwise pages that lie wholly before the last ``window``
    positions are given back as the sequence grows."""

    def __init__(self, n_pages: int, n_slots: int, window: Optional[int] = None):
        self.pool = FreeList(n_pages, "cache page")
        self.window = window
        self.rows: List[Dict[int, int]] = [dict() for _ in range(n_slots)]     # slot -> {block index: page}
        self.n_blocks: List[int] = [0] * n_slots                                # blocks mapped so far, per slot
        self.dirty: List[tuple] = []                                            # (slot, block, page or -1)

    def ensure(self, slot: int, new_len: int) -> None:
        """map pages for every position below new_len that the slot may still read or write"""
        row = self.rows[slot]
        first = self.n_blocks[slot]
        need = pages_for(new_len)
        got: List[int] = []
        try:
            for b in range(first, need):
                pg = self.pool.take()
                got.append(b)
                row[b] = pg
                self.dirty.append((slot, b, pg))
            self.n_blocks[slot] = max(first, need)
        except CacheFull:
            for b in got:
                self.pool.give(row.pop(b))
                self.dirty.append((slot, b, -1))
            raise

    def trim(self, slot: int, length: int) -> None:
        """give back the pages that no later query of this sequence can read (window groups only)"""
        if self.window is None:
            return
        first_needed = length - self.window + 1
        if first_needed <= 0:
            return
        row = self.rows[slot]
        for b in [b for b in row if (b + 1) * PAGE <= first_needed]:
            self.pool.give(row.pop(b))
            self.dirty.append((slot, b, -1))

    def release(self, slot: int) -> None:
        row = self.rows[slot]
        for b, pg in row.items():
            self.pool.give(pg)
            self.dirty.append((slot, b, -1))
        row.clear()
        self.n_blocks[slot] = 0

    def take_dirty(self) -> List[tuple]:
        d, self.dirty = self.dirty, []
        return d

    def check(self) -> None:
        self.pool.check()
        owner: Dict[int, int] = {}
        for s, row in enumerate(self.rows):
            for b, pg in row.items():
                if pg in owner:
                    raise CacheError("cache page %d is held by slots %d and %d" % (pg, owner[pg], s))
                if not self.pool.held(pg):
                    raise CacheError("cache page %d is mapped by slot %d but marked free" % (pg, s))
                owner[pg] = s
        if len(owner) != self.pool.n_held:
            raise CacheError("%d cache pages are held but %d are mapped: pages were lost"
                             % (self.pool.n_held, len(owner)))
