"""KV-page residency state machine on a bookkeeping-only pool (no GPU): the behaviours the reference pins for
its weight residency manager (tests/test_memory_governor.py:86-146) carried over to page groups."""
import pytest

import lokahi_b200 as L


def make(budget, n_seqs=3, pages=4, group_pages=4):
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=1, head_dim=8, num_pages=64, max_seqs=8,
                                       max_pages_per_seq=16, page_size=4, device=-1, host_pages=64))
    res = L.KVPageResidency(pool, budget_pages=budget, group_pages=group_pages)
    seqs = []
    for _ in range(n_seqs):
        s = pool.alloc_sequence()
        pool.append(0, None, None, n_new=pages * 4, seq_ids=[s], start_pos=[0])
        seqs.append(s)
    return pool, res, seqs


def test_never_evicts_a_pinned_group():
    pool, res, (a, b, c) = make(budget=8)
    res.track(a)
    res.pin(a, 0, 4)
    res.track(b)
    res.track(c)                                   # 12 pages tracked, budget 8: the oldest unpinned group goes
    snap = res.snapshot()
    assert (a, 0) in snap.resident_groups and (c, 0) in snap.resident_groups and snap.parked_groups == ((b, 0),)
    assert snap.resident_pages <= snap.budget_pages and snap.evictions == 1
    assert (pool.page_table(b) <= -2).all() and (pool.page_table(a) >= 0).all()
    res.release(a, 0, 4)


def test_ensure_resident_brings_back_and_evicts_lru():
    pool, res, (a, b, c) = make(budget=8)
    for s in (a, b, c):
        res.track(s)                               # a is parked when c arrives
    assert res.snapshot().parked_groups == ((a, 0),)
    assert res.ensure_resident(a, 0, 4) == 1       # b is now the least recently used
    snap = res.snapshot()
    assert snap.parked_groups == ((b, 0),) and snap.stalls == 1 and snap.prefetches == 1
    assert res.ensure_resident(a, 1, 2) == 0       # already resident: a hit
    assert (pool.page_table(a) >= 0).all()
    with pytest.raises(KeyError, match="not tracked"):
        res.ensure_resident(5, 0, 1)


def test_budget_shrink_evicts_oldest_unpinned_groups_and_refuses_pinned():
    pool, res, (a, b, c) = make(budget=12)
    for s in (a, b, c):
        res.track(s)
    res.pin(a, 0, 4)
    res.release(a, 0, 4)                           # a becomes the most recently used
    assert res.resize_budget(8) == ((b, 0),)
    snap = res.snapshot()
    assert snap.budget_pages == 8 and snap.resident_groups == ((a, 0), (c, 0))
    res.pin(a, 0, 4)
    res.pin(c, 0, 4)
    before = res.snapshot()
    with pytest.raises(L.BudgetExceededError, match="pinned"):
        res.resize_budget(4)
    assert res.snapshot() == before
    with pytest.raises(L.BudgetExceededError):
        res.ensure_resident(b, 0, 4)               # no room: both residents are pinned; nothing changes
    assert res.snapshot() == before
    res.release(a, 0, 4)
    res.release(c, 0, 4)
    with pytest.raises(RuntimeError, match="not pinned"):
        res.release(a, 0, 4)


def test_groups_follow_a_growing_sequence():
    pool, res, (a,) = make(budget=16, n_seqs=1, pages=3, group_pages=2)
    res.track(a)
    assert res.snapshot().resident_groups == ((a, 0), (a, 1)) and res.snapshot().resident_pages == 3
    pool.append(0, None, None, n_new=8, seq_ids=[a], start_pos=[12])      # two more pages
    res.track(a)
    snap = res.snapshot()
    assert snap.resident_groups == ((a, 0), (a, 1), (a, 2)) and snap.resident_pages == 5
    assert res.evict(a, 0) and not res.evict(a, 0)
    assert res.snapshot().parked_pages == 2
    res.forget(a)
    assert res.snapshot().resident_groups == ()
    with pytest.raises(ValueError, match="positive"):
        L.KVPageResidency(pool, budget_pages=0)
