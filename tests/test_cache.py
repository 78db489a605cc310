"""Slots, pages, block tables and the state region (CPU: the cache with its storage on the host)."""
import numpy as np
import pytest
import torch

from garlic_inference_b200.cache import (CacheError, GroupTable, KVRequirement, PagedCache, PagePool,
                                         SlotAllocator, StateRequirement)


def test_slots_lowest_first_reuse_and_misuse():
    s = SlotAllocator(3)
    assert [s.alloc(), s.alloc(), s.alloc()] == [0, 1, 2]
    with pytest.raises(CacheError, match="all 3 slots"):
        s.alloc()
    s.free(1)
    with pytest.raises(CacheError, match="freed twice"):
        s.free(1)
    with pytest.raises(CacheError, match="not in use"):
        s.free(7)
    assert s.alloc() == 1 and s.n_free == 0 and s.live == {0, 1, 2}


def test_pages_never_lost_or_held_twice():
    rng = np.random.default_rng(0)
    pool = PagePool(17)
    held = []
    for _ in range(2000):
        if held and (rng.random() < 0.5 or pool.n_free == 0):
            pool.give(held.pop(int(rng.integers(len(held)))))
        else:
            p = pool.take()
            assert p not in held
            held.append(p)
        assert pool.n_free + len(held) == 17
    with pytest.raises(CacheError, match="given back twice"):
        pool.give(next(p for p in range(17) if p not in held))
    while pool.n_free:
        held.append(pool.take())
    with pytest.raises(CacheError, match="all 17"):
        pool.take()
    assert sorted(held) == list(range(17))


def test_group_table_maps_pages_and_trims_the_window():
    g = GroupTable(n_pages=8, page_size=4, max_slots=2, max_pages_per_seq=8, window=6)
    assert g.pages_needed(0, 9) == 3
    g.reserve(0, 9)
    assert g.pages_of(0) == [0, 1, 2] and g.dirty == {0}
    g.trim(0, 9)                       # next query is position 9 and sees keys 4..9: page 0 is out
    assert g.pages_of(0) == [1, 2] and g.table[0, 0] == -1 and g.pool.n_free == 6
    g.reserve(0, 10)                   # still inside page 2
    assert g.pages_of(0) == [1, 2]
    g.reserve(0, 13)
    assert g.pages_of(0) == [1, 2, 0]  # the page given back is used again
    g.release(0)
    assert g.pool.n_free == 8 and (g.table[0] == -1).all() and g.pages_needed(0, 1) == 1
    full = GroupTable(n_pages=8, page_size=4, max_slots=2, max_pages_per_seq=2)
    with pytest.raises(CacheError, match="block table"):
        full.reserve(0, 9)


def _cache(**kw):
    reqs = [KVRequirement(2, 8), KVRequirement(2, 8), KVRequirement(2, 8, window=10), StateRequirement((3, 2)), None]
    args = dict(max_tokens=256, max_positions=128, dtype=torch.float32, device="cpu", page_size=16)
    args.update(kw)
    return PagedCache(reqs, **args)


def test_groups_have_storage_of_their_own():
    c = _cache()
    assert len(c.groups) == 2 and c.n_pages == 16 and c.max_slots == 4 and c.max_pages_per_seq == 8
    full, win = c.kv_view(0), c.kv_view(2)
    assert full.window is None and win.window == 10
    assert full.k_pool.shape == (16, 2, 16, 8)
    assert c.kv_view(1).block_table.data_ptr() == full.block_table.data_ptr()      # same group, one table
    assert win.block_table.data_ptr() != full.block_table.data_ptr()
    assert c.kv_view(1).k_pool.data_ptr() != full.k_pool.data_ptr()
    assert c.kv_view(3) is None and c.kv_view(4) is None
    assert c.state_view(3).shape == (4 + 1, 3, 2) and c.state_bytes_per_slot == 24     # a row per slot and a spare
    assert c.bytes_per_token() == 2 * 3 * 2 * 8 * 4


def test_step_bookkeeping_unequal_lengths_and_reuse():
    c = _cache()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.prepare([a, b], [37, 5])
    assert c.groups[0].table[a, :3].tolist() != [-1, -1, -1] and int(c.groups[0].table[a, 3]) == -1
    c.commit([a, b], [37, 5])
    assert (c.length(a), c.length(b)) == (37, 5)
    # the windowed group dropped what position 37's query cannot see (keys below 28 -> page 0)
    assert int(c.groups[1].host.table[a, 0]) == -1 and int(c.groups[1].host.table[a, 1]) >= 0
    assert int(c.groups[0].host.table[a, 0]) >= 0
    pages_a = set(c.groups[0].host.pages_of(a))
    c.state_view(3)[a] = 7.0
    c.free_slot(a)
    assert c.groups[0].host.pool.n_free == 16 - 1 and c.groups[1].host.pool.n_free == 16 - 1
    a2 = c.alloc_slot()
    assert a2 == a and c.length(a2) == 0 and float(c.state_view(3)[a2].abs().sum()) == 0.0
    c.prepare([a2], [20])
    assert set(c.groups[0].host.pages_of(a2)) <= pages_a | set(range(16))
    assert c.groups[0].table[a2, 0] >= 0          # the device table follows the host's
    with pytest.raises(CacheError, match="not in use"):
        c.free_slot(3)
    c.free_slot(a2)
    with pytest.raises(CacheError, match="not in use"):
        c.free_slot(a2)


def test_exhaustion_and_limits_raise_before_anything_changes():
    c = _cache(max_tokens=128)          # 8 pages of 16, 2 slots
    a, b = c.alloc_slot(), c.alloc_slot()
    with pytest.raises(CacheError, match="all 2 slots"):
        c.alloc_slot()
    c.prepare([a], [100])
    c.commit([a], [100])
    free_before = [g.host.pool.n_free for g in c.groups]
    with pytest.raises(CacheError, match="cache is full"):
        c.prepare([a, b], [1, 40])      # b needs 3 pages, 1 is free
    assert [g.host.pool.n_free for g in c.groups] == free_before and c.length(b) == 0
    with pytest.raises(CacheError, match="limit is 128"):
        c.prepare([a], [29])
    with pytest.raises(CacheError, match="twice"):
        c.prepare([a, a], [1, 1])
    with pytest.raises(CacheError, match="not in use"):
        c.prepare([5], [1])


def test_many_batches_lose_no_page_and_no_slot():
    rng = np.random.default_rng(1)
    c = _cache(max_tokens=512, max_positions=128)
    for _ in range(50):
        n = int(rng.integers(1, c.max_slots + 1))
        slots = [c.alloc_slot() for _ in range(n)]
        lens = [int(rng.integers(1, 60)) for _ in slots]
        c.prepare(slots, lens)
        c.commit(slots, lens)
        for _ in range(int(rng.integers(0, 20))):
            c.prepare(slots, [1] * n)
            c.commit(slots, [1] * n)
        held = [p for g in c.groups[:1] for s in slots for p in g.host.pages_of(s)]
        assert len(held) == len(set(held)), "a page is held twice"
        for s in slots:
            c.free_slot(s)
        assert c.slots.n_free == c.max_slots
        assert all(g.host.pool.n_free == g.host.pool.n_pages for g in c.groups)
        assert all((g.host.table == -1).all() for g in c.groups)
