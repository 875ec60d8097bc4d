"""The cache of a running engine: a slot per sequence, keys and values per cache entry, fixed-size state.

Cache entries (one per schedule entry that owns a cache) are grouped by what they need: entries that keep the same
number of key/value heads of the same size over the same span (all positions, or a window) share one group, and
each group has storage of its own: a pool of pages ``[entry][page][k|v][kv head][position in page][head_dim]`` and
a page table ``[slot][block]`` on the device. Entries that ask for a fixed-size state get a 32-bit tensor
``[slot][...]`` that is zeroed when a slot is taken.

Lengths are per sequence. A slot is taken when a sequence starts and given back when it ends; pages and slots that
were given back are handed out again first. The reference's counterpart is one sequence's buffers
(``kindi/nanbeige.py:587-594``) and, for its hybrid engine, recurrent state beside keys and values
(``kindi/engine.py:228-232,306-308``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import KVNeed, StateNeed
from .pages import PAGE, CacheError, FreeList, PageMap, pages_for


@dataclass
class KVGroup:
    need: KVNeed
    entries: List[int]                 # cache entry indices, in pool order
    pool: torch.Tensor                 # [len(entries), pool pages, 2, n_kv, PAGE, head_dim]
    table: torch.Tensor                # int32 [n_slots, n_pages] on the device, -1 = not mapped
    pages: PageMap
    n_pool_pages: int                  # pages of this group's pool (a window group needs fewer than a full one)


class SequenceCache:
    def __init__(self, needs: Sequence, *, max_tokens: int, n_slots: int, dtype: torch.dtype, device,
                 max_step_tokens: Optional[int] = None):
        """``needs[i]`` is the KVNeed / StateNeed / None of cache entry i. ``max_tokens`` is the most tokens all
        live sequences hold together, each sequence's count rounded up to a page. ``max_step_tokens``: the most new
        tokens one step stores (None: unknown, as many as the cache holds); it bounds what a window group has to
        keep, because pages behind the window are given back after every step."""
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_pages = max(1, pages_for(max_tokens))
        self.n_slots = max(1, min(n_slots, self.n_pages))
        self.max_step_tokens = max_step_tokens
        self.slots = FreeList(self.n_slots, "sequence slot")
        self.length: List[int] = [0] * self.n_slots
        self.groups: List[KVGroup] = []
        self._where: Dict[int, Tuple[int, int]] = {}          # cache entry -> (group index, index in group)
        self.state: Dict[int, torch.Tensor] = {}
        by_need: Dict[KVNeed, List[int]] = {}
        for i, need in enumerate(needs):
            if isinstance(need, KVNeed):
                by_need.setdefault(need, []).append(i)
            elif isinstance(need, StateNeed):
                self.state[i] = torch.zeros((self.n_slots,) + tuple(need.shape), dtype=torch.float32,
                                            device=self.device)
            elif need is not None:
                raise TypeError("cache entry %d asks for %r; a part's cache_need must be KVNeed, StateNeed or None"
                                % (i, need))
        for need, entries in by_need.items():
            n_pool = self.group_pages(need, self.n_pages, self.n_slots, max_step_tokens)
            pool = torch.zeros((len(entries), n_pool, 2, need.n_kv_heads, PAGE, need.head_dim), dtype=dtype,
                               device=self.device)
            table = torch.full((self.n_slots, self.n_pages), -1, dtype=torch.int32, device=self.device)
            g = KVGroup(need, entries, pool, table, PageMap(n_pool, self.n_slots, need.window), n_pool)
            for j, e in enumerate(entries):
                self._where[e] = (len(self.groups), j)
            self.groups.append(g)

    # ------------------------------------------------------------------ sizes
    @staticmethod
    def group_pages(need: KVNeed, n_pages: int, n_slots: int, max_step_tokens: Optional[int]) -> int:
        """pages of a group's pool. All keys: what the cache holds. A window: each sequence keeps the pages its window
        touches (two more than the window fills: it starts and ends inside pages), and while a step runs also the
        pages of its new tokens (each sequence's share again starts and ends inside pages); never more than a
        full group"""
        if need.window is None or max_step_tokens is None:
            return n_pages
        return min(n_pages, n_slots * (pages_for(need.window) + 4) + pages_for(max_step_tokens))

    @staticmethod
    def bytes_needed(needs: Sequence, max_tokens: int, n_slots: int, dtype: torch.dtype,
                     max_step_tokens: Optional[int] = None) -> int:
        n_pages = max(1, pages_for(max_tokens))
        n_slots = max(1, min(n_slots, n_pages))
        el = torch.empty((), dtype=dtype).element_size()
        total = 0
        seen = set()
        for need in needs:
            if isinstance(need, KVNeed):
                total += (SequenceCache.group_pages(need, n_pages, n_slots, max_step_tokens) * 2 * need.n_kv_heads
                          * PAGE * need.head_dim * el)
                if need not in seen:
                    seen.add(need)
                    total += min(n_slots, n_pages) * n_pages * 4
            elif isinstance(need, StateNeed):
                total += min(n_slots, n_pages) * int(np.prod(need.shape)) * 4
        return total

    def kv_bytes_per_token(self) -> int:
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.entries) * 2 * g.need.n_kv_heads * g.need.head_dim * el for g in self.groups)

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        s = self.slots.take()
        self.length[s] = 0
        for t in self.state.values():
            t[s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        self.slots.give(slot)
        for g in self.groups:
            g.pages.release(slot)
        self.length[slot] = 0

    def reserve(self, slot: int, new_len: int) -> None:
        """map pages so that positions below new_len can be written and read. Raises CacheFull when a group has no
        page left; pages mapped before that stay with the slot (they are given back with it)"""
        if not self.slots.held(slot):
            raise CacheError("slot %d is not in use" % slot)
        for g in self.groups:
            g.pages.ensure(slot, new_len)

    def commit(self, slot: int, new_len: int) -> None:
        """the step that stored positions up to new_len has been issued"""
        self.length[slot] = new_len
        for g in self.groups:
            g.pages.trim(slot, new_len)

    def flush(self) -> None:
        """bring the device page tables up to date (before a step's kernels are launched)"""
        for g in self.groups:
            dirty = g.pages.take_dirty()
            if not dirty:
                continue
            last: Dict[Tuple[int, int], int] = {}
            for s, b, pg in dirty:
                last[(s, b)] = pg
            n = len(last)
            if self.device.type != "cuda":
                idx = torch.tensor([s * self.n_pages + b for (s, b) in last], dtype=torch.int64)
                val = torch.tensor(list(last.values()), dtype=torch.int32)
                g.table.view(-1).index_copy_(0, idx, val)
                continue
            # one copy from pinned memory (places, then pages) instead of two from pageable memory, each of which
            # would hold the host up for tens of microseconds before the step's first kernel
            stage = self._stage(2 * n)
            stage[:n] = torch.tensor([s * self.n_pages + b for (s, b) in last], dtype=torch.int64)
            stage[n:2 * n] = torch.tensor(list(last.values()), dtype=torch.int64)
            dev = stage[:2 * n].to(self.device, non_blocking=True)
            self._stage_free.record()
            g.table.view(-1).index_copy_(0, dev[:n], dev[n:].to(torch.int32))

    def _stage(self, n: int) -> torch.Tensor:
        """pinned int64 staging memory of at least n elements, free to be written (the copy out of it that was issued
        last has finished)"""
        buf = getattr(self, "_stage_buf", None)
        if buf is None:
            self._stage_free = torch.cuda.Event()
        else:
            self._stage_free.synchronize()
        if buf is None or buf.numel() < n:
            buf = self._stage_buf = torch.empty(max(256, 2 * n), dtype=torch.int64, pin_memory=True)
        return buf

    # ------------------------------------------------------------------ views for the parts
    def kv_view(self, entry: int):
        """(pool of this entry [pool pages, 2, n_kv, PAGE, head_dim], page table, number of pages of the pool)"""
        gi, j = self._where[entry]
        g = self.groups[gi]
        return g.pool[j], g.table, g.n_pool_pages

    def state_view(self, entry: int) -> torch.Tensor:
        return self.state[entry]

    def tokens_held(self) -> int:
        return max((g.pages.pool.n_held for g in self.groups), default=0) * PAGE

    def check(self) -> None:
        self.slots.check()
        for g in self.groups:
            g.pages.check()
            for s in range(self.n_slots):
                if not self.slots.held(s) and g.pages.rows[s]:
                    raise CacheError("free slot %d still maps %d pages" % (s, len(g.pages.rows[s])))
