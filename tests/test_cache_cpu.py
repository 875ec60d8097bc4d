"""The cache's bookkeeping: no slot or page is lost, held twice or freed twice; windows give pages back; reuse."""
import random

import pytest
import torch

from kindi_b200.cache.pages import PAGE, CacheError, CacheFull, FreeList, PageMap, pages_for
from kindi_b200.cache.sequence_cache import SequenceCache
from kindi_b200.parts.base import KVNeed, StateNeed


def test_free_list_rules():
    f = FreeList(3, "thing")
    a, b, c = f.take(), f.take(), f.take()
    assert sorted((a, b, c)) == [0, 1, 2]
    with pytest.raises(CacheFull):
        f.take()
    f.give(b)
    with pytest.raises(CacheError):
        f.give(b)                                    # freed twice
    with pytest.raises(CacheError):
        f.give(7)                                    # never existed
    assert f.take() == b                             # what was freed last is used again first
    f.check()


def test_page_map_random_walk_loses_nothing():
    rng = random.Random(0)
    pm = PageMap(n_pages=40, n_slots=6)
    length = [0] * 6
    for _ in range(2000):
        s = rng.randrange(6)
        if rng.random() < 0.15:
            pm.release(s)
            length[s] = 0
        else:
            new = length[s] + rng.randrange(1, 90)
            try:
                pm.ensure(s, new)
                length[s] = new
            except CacheFull:
                pass
        pm.check()
        assert pm.pool.n_held == sum(pages_for(n) for n in length)
    for s in range(6):
        pm.release(s)
    pm.check()
    assert pm.pool.n_held == 0 and pm.pool.n_free == 40


def test_failed_reservation_changes_nothing():
    pm = PageMap(n_pages=3, n_slots=2)
    pm.ensure(0, 2 * PAGE)
    with pytest.raises(CacheFull):
        pm.ensure(1, 2 * PAGE + 1)
    pm.check()
    assert pm.pool.n_held == 2 and not pm.rows[1]
    pm.ensure(1, PAGE)
    assert pm.pool.n_held == 3


def test_window_gives_pages_back():
    pm = PageMap(n_pages=8, n_slots=1, window=100)
    pm.ensure(0, 500)
    assert pm.pool.n_held == 8
    pm.trim(0, 500)                 # the next query sits at 500 and reads 401..500: pages 0..5 hold positions < 384
    assert sorted(pm.rows[0]) == [6, 7] and pm.pool.n_held == 2
    pm.ensure(0, 600)
    assert sorted(pm.rows[0]) == [6, 7, 8, 9]
    pm.trim(0, 600)
    assert sorted(pm.rows[0]) == [7, 8, 9]
    pm.check()
    w1 = PageMap(n_pages=4, n_slots=1, window=1)
    w1.ensure(0, PAGE)
    w1.trim(0, PAGE)
    assert not w1.rows[0]
    w1.ensure(0, PAGE + 1)          # the next block, not block 0 again
    assert list(w1.rows[0]) == [1]


def test_sequence_cache_groups_slots_and_state():
    needs = [KVNeed(2, 16), KVNeed(2, 16, 40), KVNeed(2, 16), StateNeed((3, 4)), None, KVNeed(1, 32)]
    c = SequenceCache(needs, max_tokens=10 * PAGE, n_slots=4, dtype=torch.float32, device="cpu")
    assert len(c.groups) == 3                                           # full 2x16, window 2x16, full 1x32
    assert [g.entries for g in c.groups] == [[0, 2], [1], [5]]
    assert c.groups[0].pool.shape == (2, 10, 2, 2, PAGE, 16)
    assert c.state_view(3).shape == (4, 3, 4)
    pool0, table0, n = c.kv_view(2)
    assert pool0.shape == (10, 2, 2, PAGE, 16) and table0.shape == (4, 10) and n == 10
    s = c.alloc_slot()
    c.state_view(3)[s] += 5.0
    c.reserve(s, 3 * PAGE + 1)
    c.commit(s, 3 * PAGE + 1)
    c.flush()
    assert (c.groups[0].table[s] >= 0).sum() == 4
    assert (c.groups[1].table[s] >= 0).sum() == 2        # the window group kept the pages of positions 154..193
    c.check()
    with pytest.raises(CacheError):
        c.reserve(3 if s != 3 else 2, 10)                                # a slot that is not in use
    c.free_slot(s)
    with pytest.raises(CacheError):
        c.free_slot(s)
    c.flush()
    assert (c.groups[0].table >= 0).sum() == 0
    s2 = c.alloc_slot()
    assert s2 == s and float(c.state_view(3)[s2].abs().sum()) == 0.0     # reused, state zeroed
    c.check()
    assert c.kv_bytes_per_token() == (2 * 2 * 2 * 16 + 1 * 2 * 2 * 16 + 1 * 2 * 1 * 32) * 4


def test_cache_full_is_reported():
    c = SequenceCache([KVNeed(1, 16)], max_tokens=2 * PAGE, n_slots=4, dtype=torch.float32, device="cpu")
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve(a, PAGE)
    c.reserve(b, PAGE)
    with pytest.raises(CacheFull):
        c.reserve(a, PAGE + 1)
    c.check()


def test_window_group_keeps_a_pool_of_the_window_plus_a_step():
    """a group whose entries only ever read a window holds far fewer pages than a group that keeps every key, and
    sequences can still grow to the cache's full length in steps of at most max_step_tokens new tokens"""
    needs = [KVNeed(1, 16), KVNeed(1, 16, 100)]
    c = SequenceCache(needs, max_tokens=40000, n_slots=2, dtype=torch.float32, device="cpu", max_step_tokens=256)
    full, win = c.groups
    assert full.n_pool_pages == 625 and win.n_pool_pages == 2 * (2 + 4) + 4
    assert win.pool.shape[1] == win.n_pool_pages and c.kv_view(1)[2] == win.n_pool_pages
    assert SequenceCache.bytes_needed(needs, 40000, 2, torch.float32, 256) < \
        0.52 * SequenceCache.bytes_needed(needs, 40000, 2, torch.float32)
    rng = random.Random(1)
    a, b = c.alloc_slot(), c.alloc_slot()
    la = lb = 0
    while la + lb < 39000:
        na = rng.choice((1, 1, 63, 64, 65, 128, 200))
        nb = min(256 - na, rng.choice((1, 1, 56, 7)))
        c.reserve(a, la + na)
        c.reserve(b, lb + nb)
        c.flush()
        la, lb = la + na, lb + nb
        c.commit(a, la)
        c.commit(b, lb)
        held = {p for p in c.groups[1].table[a].tolist() if p >= 0}
        assert all(0 <= p < win.n_pool_pages for p in held)
        rows_a = c.groups[1].pages.rows[a]       # the next query (position la) reads la - 99 .. la
        assert (la - 1) // PAGE in rows_a and max(0, la - 99) // PAGE in rows_a
    c.check()
    c.free_slot(a)
    c.free_slot(b)
    c.check()
    assert win.pages.pool.n_held == 0 and full.pages.pool.n_held == 0
