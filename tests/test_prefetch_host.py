"""Look-ahead over parked KV page groups on a bookkeeping-only pool (no GPU): the behaviours the reference pins
for its weight prefetch scheduler (tests/test_memory_governor.py:146-213) carried over to page groups."""
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
        res.track(s)
        seqs.append(s)
    return pool, res, seqs


class Recorder:
    def __init__(self):
        self.events = []

    def record_operation(self, name, duration_ms, **kw):
        self.events.append((name, kw.get("cache_status")))


def test_pipeline_loads_the_next_group_ahead_of_its_use():
    """A loop over three sequences with room for two: the first is a cold miss, the others were prefetched while
    the previous one was in use (test_memory_governor.py:146-178)."""
    pool, res, seqs = make(budget=8)
    for s in seqs:                                  # start with everything parked
        res.evict(s, 0)
    assert res.snapshot().resident_pages == 0
    rec = Recorder()
    pf = L.KVPagePrefetcher(res, tracer=rec)
    full = L.TensorTracer()                        # the same calls must fit the reference tracer's signature
    pf2_pool, pf2_res, pf2_seqs = make(budget=8)
    for s in pf2_seqs:
        pf2_res.evict(s, 0)
    with L.KVPagePrefetcher(pf2_res, tracer=full).acquire(pf2_seqs[0], 0, phase="decode"):
        pass
    kinds = [(e.name, e.cache_status, e.group_id) for e in full.events]
    assert ("kv_page_acquire", "cold_miss", f"{pf2_seqs[0]}:0") in kinds
    load = [e for e in full.events if e.name == "kv_page_load"][0]
    assert load.kind == "operation" and load.phase == "decode" and load.bytes_transferred == 4 * (1 * 2 * 1 * 4 * 8 * 2)   # pages x (layers, K|V, heads, page, dim, bf16)
    statuses = []
    for i, s in enumerate(seqs):
        with pf.acquire(s, 0, phase="decode") as lease:
            statuses.append(lease.cache_status)
            if i + 1 < len(seqs):
                assert pf.prefetch(seqs[i + 1], 0, phase="decode")
                assert res.state(seqs[i + 1], 0) is L.GroupState.LOADING
            assert (pool.page_table(s) >= 0).all()
    snap = pf.snapshot()
    assert statuses[0] == "cold_miss" and set(statuses[1:]) <= {"prefetch_ready", "prefetch_wait"}
    assert snap.cold_misses == 1 and snap.prefetch_ready_hits + snap.prefetch_waits == 2 and snap.prefetch_skips == 0
    assert snap.pages_loaded == 12 and snap.stall_time_ms >= 0.0
    assert res.snapshot().resident_pages <= res.snapshot().budget_pages
    assert ("kv_page_acquire", "cold_miss") in rec.events and ("kv_page_load", "demand") in rec.events


def test_single_group_budget_skips_the_look_ahead_but_still_runs():
    """Budget for one group only: the look-ahead is refused (budget_skip) while the current group is pinned and
    every group is then loaded on demand (test_memory_governor.py:180-197)."""
    pool, res, (a, b, _) = make(budget=4, n_seqs=3)
    for s in (a, b):
        if res.is_resident(s, 0):
            res.evict(s, 0)
    pf = L.KVPagePrefetcher(res)
    with pf.acquire(a, 0, phase="prefill"):
        before = res.snapshot()
        assert pf.prefetch(b, 0, phase="prefill") is False
        assert res.snapshot() == before                       # a refused reservation changes nothing
    with pf.acquire(b, 0, phase="prefill") as lease:
        assert lease.cache_status == "cold_miss"
    snap = pf.snapshot()
    assert snap.prefetch_skips == 1 and snap.cold_misses == 2


def test_evicted_completed_prefetch_is_reloaded_on_demand():
    """A prefetched group that was evicted again before its first pin is loaded once more by acquire
    (test_memory_governor.py:199-213)."""
    pool, res, (a, b, c) = make(budget=8)
    for s in (a, b, c):
        if res.is_resident(s, 0):
            res.evict(s, 0)
    pf = L.KVPagePrefetcher(res)
    assert pf.prefetch(a, 0)
    orig_pin, fired = res.pin, []

    def evict_before_first_pin(seq, first, n):                 # what a competing reservation would have done
        if not fired:
            fired.append(True)
            assert res.evict(seq, first // res.group_pages)
        return orig_pin(seq, first, n)

    res.pin = evict_before_first_pin
    with pf.acquire(a, 0) as lease:
        assert lease.cache_status == "prefetch_evicted_reload"
        assert (pool.page_table(a) >= 0).all()
    snap = pf.snapshot()
    assert snap.cold_misses == 1 and snap.pages_loaded == 8    # loaded twice, 4 pages each time
    assert res.snapshot().prefetches == 2


def test_demand_that_cannot_fit_raises_and_changes_nothing():
    pool, res, (a, b, _) = make(budget=4, n_seqs=3)
    for s in (a, b):
        if res.is_resident(s, 0):
            res.evict(s, 0)
    pf = L.KVPagePrefetcher(res)
    lease = pf.acquire(a, 0)
    before = res.snapshot()
    with pytest.raises(L.BudgetExceededError, match="pinned"):
        pf.acquire(b, 0)
    assert res.snapshot() == before
    lease.release()
    lease.release()                                            # idempotent, like WeightLease.release
    with pf.acquire(b, 0) as l2:
        assert l2.cache_status == "cold_miss"
    with pf.acquire(b, 0) as l3:
        assert l3.cache_status == "resident_hit"
    assert pf.snapshot().resident_hits == 1
