"""Residency state for KV pages: which page groups stay in HBM, which are parked in pinned host memory.

The reference has this machinery for *weights* (``ResidencyManager``, src/ollm/scheduling/residency_manager.py:
40-297: a byte budget, LRU order, pin counts, ``resize_budget`` and a snapshot) and only a design note for KV
blocks (docs/STRATA_ENGINE_ARCHITECTURE.md:696-723).  This is the same state machine applied to KV pages on top
of ``PagedPool.evict`` / ``PagedPool.prefetch``: the unit is a *group* of consecutive page-table slots of one
sequence, the budget is a number of device pages, victims are the least recently used unpinned resident groups,
pinned groups (attention in flight) are never evicted, and a request that cannot be met leaves everything as
it was and raises ``BudgetExceededError``.  All policy is host-side bookkeeping; the bytes move through the
pool's copy kernel on its own stream.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from threading import RLock
from typing import Dict, List, Tuple


class BudgetExceededError(RuntimeError):
    """The pinned or requested groups do not fit inside the device-page budget."""


class GroupState(str, Enum):
    RESIDENT = "resident"
    PARKED = "parked"
    LOADING = "loading"       # device pages reserved, copy back from the host enqueued but not yet confirmed


@dataclass
class _Group:
    seq: int
    index: int
    first_slot: int
    n_slots: int
    state: GroupState
    last_used: int
    pin_count: int = 0


@dataclass(frozen=True)
class KVResidencySnapshot:
    budget_pages: int
    resident_pages: int
    parked_pages: int
    pinned_pages: int
    resident_groups: Tuple[Tuple[int, int], ...]
    parked_groups: Tuple[Tuple[int, int], ...]
    pinned_groups: Tuple[Tuple[int, int], ...]
    evictions: int
    prefetches: int
    stalls: int               # ensure_resident calls that had to bring at least one group back
    loading_groups: Tuple[Tuple[int, int], ...] = ()


class KVPageResidency:
    def __init__(self, pool, budget_pages: int, group_pages: int = 64):
        if budget_pages <= 0:
            raise ValueError("budget_pages must be positive")
        if group_pages <= 0:
            raise ValueError("group_pages must be positive")
        self.pool = pool
        self.budget_pages = int(budget_pages)
        self.group_pages = int(group_pages)
        self._groups: Dict[Tuple[int, int], _Group] = {}
        self._tick = 0
        self._lock = RLock()
        self._evictions = self._prefetches = self._stalls = 0

    # -- bookkeeping ---------------------------------------------------------------------------------
    def _next_tick(self) -> int:
        self._tick += 1
        return self._tick

    def _resident_pages(self) -> int:
        """Device pages held: resident groups plus those reserved for a copy in flight."""
        return sum(g.n_slots for g in self._groups.values() if g.state is not GroupState.PARKED)

    def track(self, seq: int) -> None:
        """Register (or extend) the groups of a sequence from its current page-table row; new pages are resident."""
        with self._lock:
            n_pages = len(self.pool.page_table(seq))
            for idx in range(-(-n_pages // self.group_pages)):
                first = idx * self.group_pages
                n = min(self.group_pages, n_pages - first)
                g = self._groups.get((seq, idx))
                if g is None:
                    self._groups[(seq, idx)] = _Group(seq, idx, first, n, GroupState.RESIDENT, self._next_tick())
                elif g.n_slots != n:
                    if g.state is GroupState.PARKED:
                        raise RuntimeError(f"group {(seq, idx)} grew while parked")
                    g.n_slots = n
            self._make_room(0)

    def forget(self, seq: int) -> None:
        with self._lock:
            for key in [k for k in self._groups if k[0] == seq]:
                if self._groups[key].pin_count:
                    raise RuntimeError(f"cannot forget pinned group {key}")
                del self._groups[key]

    def _groups_of(self, seq: int, first_slot: int, n_slots: int) -> List[_Group]:
        lo, hi = first_slot // self.group_pages, (first_slot + n_slots - 1) // self.group_pages
        out = []
        for idx in range(lo, hi + 1):
            g = self._groups.get((seq, idx))
            if g is None:
                raise KeyError(f"group {(seq, idx)} is not tracked")
            out.append(g)
        return out

    def _victims(self, need_pages: int, exclude) -> List[_Group]:
        """LRU unpinned resident groups whose eviction brings the resident set to budget - need_pages."""
        over = self._resident_pages() + need_pages - self.budget_pages
        victims: List[_Group] = []
        if over <= 0:
            return victims
        candidates = sorted((g for g in self._groups.values()
                             if g.state is GroupState.RESIDENT and g.pin_count == 0 and (g.seq, g.index) not in exclude),
                            key=lambda g: g.last_used)
        for g in candidates:
            if over <= 0:
                break
            victims.append(g)
            over -= g.n_slots
        if over > 0:
            raise BudgetExceededError(
                f"need {need_pages} more device pages inside a budget of {self.budget_pages}; pinned or requested "
                f"groups leave {over} pages too many")
        return victims

    def _make_room(self, need_pages: int, exclude=()) -> None:
        for g in self._victims(need_pages, set(exclude)):
            self.pool.evict(g.seq, g.first_slot, g.n_slots)
            g.state = GroupState.PARKED
            self._evictions += 1

    # -- the calls a decode loop makes -----------------------------------------------------------------------
    def ensure_resident(self, seq: int, first_slot: int, n_slots: int) -> int:
        """Bring the groups covering the slots back to HBM (evicting LRU groups if the budget needs it) and
        mark them used.  Returns the number of groups that had to be fetched."""
        with self._lock:
            groups = self._groups_of(seq, first_slot, n_slots)
            parked = [g for g in groups if g.state is GroupState.PARKED]
            loading = [g for g in groups if g.state is GroupState.LOADING]      # reserved earlier, copy in flight
            keys = {(g.seq, g.index) for g in groups}
            self._make_room(sum(g.n_slots for g in parked), exclude=keys)     # raises before anything moves
            for g in parked:
                self.pool.prefetch(g.seq, g.first_slot, g.n_slots)
                self._prefetches += 1
            for g in groups:
                g.state = GroupState.RESIDENT
                g.last_used = self._next_tick()
            if parked or loading:
                self._stalls += 1
                self.pool.sync_transfers()
            return len(parked)

    # -- reserve / commit: the asynchronous half (residency_manager.py:78-150) -------------------------------
    def is_resident(self, seq: int, group_index: int) -> bool:
        with self._lock:
            g = self._groups.get((seq, group_index))
            return g is not None and g.state is GroupState.RESIDENT

    def state(self, seq: int, group_index: int) -> GroupState:
        with self._lock:
            g = self._groups.get((seq, group_index))
            if g is None:
                raise KeyError(f"group {(seq, group_index)} is not tracked")
            return g.state

    def reserve(self, seq: int, group_index: int) -> bool:
        """Make room for a parked group and enqueue its copy back without waiting for it.  Returns False, with
        nothing changed, when the budget cannot hold it beside the pinned and loading groups (the reference's
        ``reserve`` returning False -> "budget_skip", prefetch_scheduler.py:146-156)."""
        with self._lock:
            g = self._groups.get((seq, group_index))
            if g is None:
                raise KeyError(f"group {(seq, group_index)} is not tracked")
            if g.state is not GroupState.PARKED:
                return True
            try:
                self._make_room(g.n_slots, exclude={(seq, group_index)})
            except BudgetExceededError:
                return False
            self.pool.prefetch(g.seq, g.first_slot, g.n_slots)
            g.state = GroupState.LOADING
            self._prefetches += 1
            return True

    def commit(self, seq: int, group_index: int) -> None:
        """The copy of a reserved group has completed: it is resident (and, unpinned, evictable) from now on."""
        with self._lock:
            g = self._groups.get((seq, group_index))
            if g is None or g.state is not GroupState.LOADING:
                raise KeyError(f"group {(seq, group_index)} has no reservation")
            g.state = GroupState.RESIDENT
            g.last_used = self._next_tick()

    def pin(self, seq: int, first_slot: int, n_slots: int) -> None:
        with self._lock:
            groups = self._groups_of(seq, first_slot, n_slots)
            for g in groups:
                if g.state is not GroupState.RESIDENT:
                    raise KeyError(f"group {(g.seq, g.index)} is not resident")
            for g in groups:
                g.pin_count += 1
                g.last_used = self._next_tick()

    def release(self, seq: int, first_slot: int, n_slots: int) -> None:
        with self._lock:
            groups = self._groups_of(seq, first_slot, n_slots)
            for g in groups:
                if g.pin_count <= 0:
                    raise RuntimeError(f"group {(g.seq, g.index)} is not pinned")
            for g in groups:
                g.pin_count -= 1
                g.last_used = self._next_tick()

    def evict(self, seq: int, group_index: int) -> bool:
        with self._lock:
            g = self._groups.get((seq, group_index))
            if g is None or g.state is not GroupState.RESIDENT or g.pin_count > 0:
                return False
            self.pool.evict(g.seq, g.first_slot, g.n_slots)
            g.state = GroupState.PARKED
            self._evictions += 1
            return True

    def resize_budget(self, budget_pages: int) -> Tuple[Tuple[int, int], ...]:
        """Change the device-page budget; shrinking parks LRU unpinned groups.  Fails without any change when
        the pinned groups alone exceed the request (residency_manager.py:209-262)."""
        if budget_pages <= 0:
            raise ValueError("budget_pages must be positive")
        with self._lock:
            pinned = sum(g.n_slots for g in self._groups.values() if g.pin_count > 0 and g.state is GroupState.RESIDENT)
            if pinned > budget_pages:
                raise BudgetExceededError(
                    f"cannot shrink the budget to {budget_pages} pages; pinned groups require {pinned} pages")
            old = self.budget_pages
            self.budget_pages = int(budget_pages)
            try:
                victims = self._victims(0, set())
            except BudgetExceededError:
                self.budget_pages = old
                raise
            for g in victims:
                self.pool.evict(g.seq, g.first_slot, g.n_slots)
                g.state = GroupState.PARKED
                self._evictions += 1
            return tuple((g.seq, g.index) for g in victims)

    def snapshot(self) -> KVResidencySnapshot:
        with self._lock:
            res = [g for g in self._groups.values() if g.state is GroupState.RESIDENT]
            par = [g for g in self._groups.values() if g.state is GroupState.PARKED]
            pin = [g for g in self._groups.values() if g.pin_count > 0]
            load = [g for g in self._groups.values() if g.state is GroupState.LOADING]
            key = lambda g: (g.seq, g.index)
            return KVResidencySnapshot(
                budget_pages=self.budget_pages, resident_pages=sum(g.n_slots for g in res),
                parked_pages=sum(g.n_slots for g in par), pinned_pages=sum(g.n_slots for g in pin),
                resident_groups=tuple(sorted(map(key, res))), parked_groups=tuple(sorted(map(key, par))),
                pinned_groups=tuple(sorted(map(key, pin))), evictions=self._evictions, prefetches=self._prefetches,
                stalls=self._stalls, loading_groups=tuple(sorted(map(key, load))))
