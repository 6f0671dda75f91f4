"""Look-ahead for parked KV pages: bring a group back before the step that needs it, and account for the stalls.

The reference has this for weight groups (``PrefetchScheduler``, src/ollm/scheduling/prefetch_scheduler.py:64-257:
``prefetch`` reserves budget and loads on a worker thread, ``acquire`` pins a group and reports how it was found
-- ``resident_hit``, ``prefetch_ready``, ``prefetch_wait``, ``cold_miss``, ``prefetch_evicted_reload`` (recorded through the tracer's ``record_operation`` with the
reference's keyword arguments: ``group_id``, ``cache_status``, ``bytes_transferred``, ``bandwidth_bytes_per_second``) -- a
reservation that does not fit is a ``budget_skip``, and a snapshot carries the counters and the measured stall
time).  Here the unit is a group of KV page-table slots (``KVPageResidency``) and there is no worker thread: the
copy back from pinned host memory is a kernel on the pool's copy stream, so "in flight" means enqueued there and
"ready" means that stream has drained (``PagedPool.transfers_done``).  The cache statuses, the counters and the
failure rule (a demand that cannot fit raises ``BudgetExceededError`` and changes nothing) follow the reference.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from threading import RLock
from typing import Any, Dict, Optional, Tuple

from .residency import BudgetExceededError, GroupState, KVPageResidency


@dataclass(frozen=True)
class KVPrefetchSnapshot:
    resident_hits: int
    cold_misses: int
    prefetch_ready_hits: int
    prefetch_waits: int
    prefetch_skips: int
    pages_loaded: int
    load_time_ms: float
    stall_time_ms: float


class KVPageLease:
    """A pinned group; leaving the ``with`` block (or ``release``) unpins it (prefetch_scheduler.py:36-61)."""

    def __init__(self, prefetcher: "KVPagePrefetcher", seq: int, group_index: int, cache_status: str):
        self.prefetcher, self.seq, self.group_index, self.cache_status = prefetcher, seq, group_index, cache_status
        self._released = False

    def release(self) -> None:
        if not self._released:
            self.prefetcher._release(self.seq, self.group_index)
            self._released = True

    def __enter__(self) -> "KVPageLease":
        return self

    def __exit__(self, exc_type, exc_value, traceback) -> None:
        self.release()


class KVPagePrefetcher:
    def __init__(self, residency: KVPageResidency, *, tracer: Optional[Any] = None, wait_timeout_ms: int = 10000):
        self.residency = residency
        self.pool = residency.pool
        self.tracer = tracer
        self.wait_timeout_ms = int(wait_timeout_ms)
        c = self.pool.cfg
        self._page_bytes = (c.num_layers * 2 * c.num_kv_heads * c.page_size * c.head_dim *
                            (2 if "bfloat16" in str(c.dtype) else 4))       # one page id covers all layers, K and V
        self._inflight: Dict[Tuple[int, int], float] = {}       # group -> time its copy was enqueued
        self._lock = RLock()
        self._resident_hits = self._cold_misses = self._ready_hits = self._waits = self._skips = 0
        self._pages_loaded = 0
        self._load_ms = self._stall_ms = 0.0

    # -- helpers ------------------------------------------------------------------------------------------
    def _trace(self, name: str, duration_ms: float, **kw: Any) -> None:
        if self.tracer is not None:
            self.tracer.record_operation(name, duration_ms, **kw)

    def _slots(self, seq: int, group_index: int) -> Tuple[int, int]:
        gp = self.residency.group_pages
        n_pages = len(self.pool.page_table(seq))
        first = group_index * gp
        return first, max(0, min(gp, n_pages - first))

    def _finish(self, key: Tuple[int, int], phase: str, status: str) -> None:
        """Wait (bounded) for the copy stream, order the compute stream after it, commit every landed group."""
        started = time.perf_counter()
        self.pool.wait_resident(self.wait_timeout_ms)
        self.pool.sync_transfers()
        now = time.perf_counter()
        with self._lock:
            for k, t_enq in list(self._inflight.items()):
                if self.residency.state(*k) is GroupState.LOADING:
                    self.residency.commit(*k)
                    n = self._slots(*k)[1]
                    self._pages_loaded += n
                    self._load_ms += (now - t_enq) * 1000.0
                    nbytes = n * self._page_bytes
                    secs = now - t_enq
                    self._trace("kv_page_load", secs * 1000.0, phase=phase, group_id=f"{k[0]}:{k[1]}",
                                cache_status=status if k == key else "prefetch", bytes_transferred=nbytes,
                                bandwidth_bytes_per_second=(nbytes / secs if secs > 0 else None))
                del self._inflight[k]
        del started

    # -- the two calls of a decode loop ----------------------------------------------------------------------
    def prefetch(self, seq: int, group_index: int, *, phase: str = "decode") -> bool:
        """Reserve room for a parked group and enqueue its copy back; False (a ``budget_skip``) if it cannot fit."""
        key = (seq, group_index)
        with self._lock:
            if self.residency.is_resident(seq, group_index) or key in self._inflight:
                return True
            if not self.residency.reserve(seq, group_index):
                self._skips += 1
                self._trace("kv_page_prefetch", 0.0, phase=phase, group_id=f"{key[0]}:{key[1]}", cache_status="budget_skip")
                return False
            self._inflight[key] = time.perf_counter()
            return True

    def acquire(self, seq: int, group_index: int, *, phase: str = "decode") -> KVPageLease:
        """Pin a group for the attention call that is about to read it, waiting for a copy in flight or loading
        it on demand.  The compute stream is ordered after the copy before this returns."""
        started = time.perf_counter()
        key = (seq, group_index)
        first, n = self._slots(seq, group_index)
        with self._lock:
            inflight = key in self._inflight
        if inflight:
            ready = self.pool.transfers_done()
            self._finish(key, phase, "prefetch")
            status = "prefetch_ready" if ready else "prefetch_wait"
            with self._lock:
                if ready:
                    self._ready_hits += 1
                else:
                    self._waits += 1
            try:
                self.residency.pin(seq, first, n)
            except KeyError:
                # another reservation evicted this unpinned group between its landing and the pin: correctness
                # must not depend on the order of completion, so load it again under the same budget
                self._demand(seq, group_index, first, n, phase, "prefetch_evicted_reload")
                status = "prefetch_evicted_reload"
        elif self.residency.is_resident(seq, group_index):
            self.residency.pin(seq, first, n)
            status = "resident_hit"
            with self._lock:
                self._resident_hits += 1
        else:
            self._demand(seq, group_index, first, n, phase, "demand")
            status = "cold_miss"
        stall = (time.perf_counter() - started) * 1000.0
        with self._lock:
            self._stall_ms += stall
        self._trace("kv_page_acquire", stall, phase=phase, group_id=f"{key[0]}:{key[1]}", cache_status=status)
        return KVPageLease(self, seq, group_index, status)

    def _demand(self, seq: int, group_index: int, first: int, n: int, phase: str, status: str) -> None:
        key = (seq, group_index)
        if not self.residency.reserve(seq, group_index):
            snap = self.residency.snapshot()
            raise BudgetExceededError(
                f"cannot acquire group {key} ({n} pages) inside a budget of {snap.budget_pages} pages; "
                f"pinned={list(snap.pinned_groups)}")
        with self._lock:
            self._inflight[key] = time.perf_counter()
            self._cold_misses += 1
        self._finish(key, phase, status)
        self.residency.pin(seq, first, n)

    def _release(self, seq: int, group_index: int) -> None:
        first, n = self._slots(seq, group_index)
        self.residency.release(seq, first, n)

    def snapshot(self) -> KVPrefetchSnapshot:
        with self._lock:
            return KVPrefetchSnapshot(self._resident_hits, self._cold_misses, self._ready_hits, self._waits, self._skips,
                                      self._pages_loaded, self._load_ms, self._stall_ms)
