"""The cache manager: groups of layer runs, a block table per request and group, and state slots.

Every mixer says what it needs to keep between steps (`CacheNeed`): keys and values for
all earlier positions, for a window of them, a state of fixed size, or nothing. Layer runs
with the same need form a *group*; a group of keys and values has a page pool of its own
and every request has one block table per group (position p of the request lives in page
`table[p // page_size]`, row `p % page_size`: docs/24-paged-kv-cache.md:59-72 of the
reference, which has a single group because its layers always move together, :395-397).
A windowed group gives pages back as soon as the window has passed them; the others keep
theirs until the request ends. A fixed-state group has storage [slots, ...] and each
request one slot.

Before a step, `reserve(request, start, n)` makes sure pages exist for positions
[start, start + n) in every group (the reference's `beginWrite`,
src/main/java/org/robomiri/jllm/kv/KvSequence.java:116-146); it takes all of them or none
and raises `PoolExhausted`. After the step `commit(request, length)` records the new
length and releases what a window has passed. `close` gives everything back.

The manager is host bookkeeping; the device memory of a group is made by the `allocate`
callable it is given (None in tests that need no device).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

from .pages import PageBookkeepingError, PagePool, PoolExhausted, StateSlotPool

RELEASED = -1  # table entry of a page that a window has passed


@dataclass(frozen=True)
class CacheNeed:
    """What one layer run keeps between steps. Base = nothing."""


@dataclass(frozen=True)
class PagedKeysValues(CacheNeed):
    kv_heads: int
    head_dim: int
    window: int = 0                        # 0 = every earlier position, else the last `window`


@dataclass(frozen=True)
class FixedState(CacheNeed):
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass
class PagedGroup:
    need: PagedKeysValues
    runs: List[int]                        # schedule indices of the member layer runs
    pool: PagePool
    storage: object = None                 # [len(runs), 2, pages, kv_heads, page_size, head_dim]

    def keys_values(self, run: int):
        """(K, V) of one member run: each [pages, kv_heads, page_size, head_dim]."""
        i = self.runs.index(run)
        return self.storage[i, 0], self.storage[i, 1]


@dataclass
class StateGroup:
    need: FixedState
    runs: List[int]
    storage: object = None                 # [len(runs), slots, *shape]

    def state(self, run: int):
        return self.storage[self.runs.index(run)]


@dataclass
class RequestCache:
    request: Hashable
    state_slot: int
    length: int = 0
    tables: List[List[int]] = field(default_factory=list)  # one per paged group
    epoch: int = 0                         # changes whenever a table changed otherwise than by growing at its end


class CacheManager:
    def __init__(self, needs: Sequence[Optional[CacheNeed]], page_size: int, num_pages: int, max_requests: int,
                 allocate: Optional[Callable] = None):
        """`needs[i]` is the need of schedule entry i (None for a run that keeps nothing or reads another's cache)."""
        if page_size < 1:
            raise ValueError(f"page_size={page_size} must be at least 1")
        self.page_size = page_size
        self.num_pages = num_pages
        self.paged: List[PagedGroup] = []
        self.fixed: List[StateGroup] = []
        self.group_of_run: Dict[int, Tuple[str, int]] = {}
        for run, need in enumerate(needs):
            if need is None or type(need) is CacheNeed:
                continue
            if isinstance(need, PagedKeysValues):
                for gi, g in enumerate(self.paged):
                    if g.need == need:
                        g.runs.append(run)
                        break
                else:
                    gi = len(self.paged)
                    self.paged.append(PagedGroup(need, [run], PagePool(num_pages, f"group{gi}")))
                self.group_of_run[run] = ("paged", gi)
            elif isinstance(need, FixedState):
                for gi, g in enumerate(self.fixed):
                    if g.need == need:
                        g.runs.append(run)
                        break
                else:
                    gi = len(self.fixed)
                    self.fixed.append(StateGroup(need, [run]))
                self.group_of_run[run] = ("fixed", gi)
            else:
                raise TypeError(f"layer run {run}: unknown cache need {need!r}")
        self.slots = StateSlotPool(max_requests)
        self._epochs = itertools.count(1)
        self.requests: Dict[Hashable, RequestCache] = {}
        if allocate is not None:
            for g in self.paged:
                g.storage = allocate((len(g.runs), 2, num_pages, g.need.kv_heads, page_size, g.need.head_dim), "kv")
            for g in self.fixed:
                g.storage = allocate((len(g.runs), max_requests) + tuple(g.need.shape), g.need.dtype)

    # ---- what a layer run reads and writes ----------------------------------------------------------------
    def paged_group_of(self, run: int) -> int:
        kind, gi = self.group_of_run[run]
        if kind != "paged":
            raise KeyError(f"layer run {run} keeps no keys and values")
        return gi

    def keys_values(self, run: int):
        return self.paged[self.paged_group_of(run)].keys_values(run)

    def state(self, run: int):
        kind, gi = self.group_of_run[run]
        if kind != "fixed":
            raise KeyError(f"layer run {run} keeps no fixed-size state")
        return self.fixed[gi].state(run)

    # ---- requests ---------------------------------------------------------------------------------------
    def open(self, request: Hashable) -> RequestCache:
        if request in self.requests:
            raise ValueError(f"request {request!r} is open already")
        rc = RequestCache(request, self.slots.alloc(request), 0, [[] for _ in self.paged], next(self._epochs))
        self.requests[request] = rc
        return rc

    def is_open(self, request: Hashable) -> bool:
        return request in self.requests

    def length(self, request: Hashable) -> int:
        return self.requests[request].length

    def _first_needed_page(self, g: PagedGroup, length: int) -> int:
        """Pages below this index hold only positions that no later query of the request can see."""
        if g.need.window <= 0:
            return 0
        return max(0, length + 1 - g.need.window) // self.page_size

    def pages_missing(self, request: Hashable, start: int, n: int) -> List[int]:
        """How many pages each paged group would have to take for positions [start, start + n)."""
        rc = self.requests.get(request)
        out = []
        for gi, g in enumerate(self.paged):
            have = len(rc.tables[gi]) if rc is not None else 0
            if rc is not None and start < rc.length:
                have = min(have, -(-start // self.page_size))
            out.append(max(0, -(-(start + n) // self.page_size) - have))
        return out

    def can_reserve(self, request: Hashable, start: int, n: int) -> bool:
        return all(m <= g.pool.num_free for m, g in zip(self.pages_missing(request, start, n), self.paged))

    def reserve(self, request: Hashable, start: int, n: int) -> None:
        """Pages for positions [start, start + n) in every group, all or none; positions from `start`
        on that an earlier step wrote are dropped first (a rewind)."""
        rc = self.requests[request]
        if start < 0 or n < 1:
            raise ValueError(f"reserve: start={start} n={n}")
        if start > rc.length:
            raise ValueError(f"request {request!r} holds {rc.length} positions, a step cannot start at {start}")
        if start < rc.length:
            self.truncate(request, start)
        taken: List[Tuple[int, int]] = []
        want_pages = -(-(start + n) // self.page_size)
        try:
            for gi, g in enumerate(self.paged):
                table = rc.tables[gi]
                while len(table) < want_pages:
                    page = g.pool.alloc(request)
                    table.append(page)
                    taken.append((gi, page))
        except PoolExhausted:
            rc.epoch = next(self._epochs)
            for gi, page in reversed(taken):
                popped = rc.tables[gi].pop()
                if popped != page:
                    raise PageBookkeepingError("rollback of a failed reserve lost track of a page")
                self.paged[gi].pool.free(page, request)
            raise

    def commit(self, request: Hashable, length: int) -> List[Tuple[int, int]]:
        """The request now holds `length` positions. Returns the (group, page) pairs given back
        because a window has passed them."""
        rc = self.requests[request]
        if length < rc.length:
            raise ValueError(f"commit cannot shorten a request ({rc.length} -> {length}); use truncate")
        rc.length = length
        released = []
        for gi, g in enumerate(self.paged):
            if length > len(rc.tables[gi]) * self.page_size:
                raise PageBookkeepingError(f"request {request!r} committed {length} positions beyond its pages")
            for i in range(min(self._first_needed_page(g, length), len(rc.tables[gi]))):
                page = rc.tables[gi][i]
                if page != RELEASED:
                    g.pool.free(page, request)
                    rc.tables[gi][i] = RELEASED
                    released.append((gi, page))
        if released:
            rc.epoch = next(self._epochs)
        return released

    def truncate(self, request: Hashable, length: int) -> None:
        """Forget positions >= length: pages wholly past it go back (KvSequence.java:149-157). A windowed
        group cannot go back behind pages it has given up already."""
        rc = self.requests[request]
        if length >= rc.length:
            return
        keep = -(-length // self.page_size)
        for gi, g in enumerate(self.paged):    # first look, then touch: a refused rewind changes nothing
            if g.need.window > 0 and self._first_needed_page(g, rc.length) > self._first_needed_page(g, length):
                if any(p == RELEASED for p in rc.tables[gi][self._first_needed_page(g, length):keep]):
                    raise ValueError(f"request {request!r}: a windowed group has released pages that a rewind "
                                     f"to {length} needs; recompute from the start")
        rc.epoch = next(self._epochs)
        for gi, g in enumerate(self.paged):
            table = rc.tables[gi]
            while len(table) > keep:
                page = table.pop()
                if page != RELEASED:
                    g.pool.free(page, request)
        rc.length = length

    def trim(self, request: Hashable) -> None:
        """Give back pages reserved beyond the committed length (a step that was reserved but did not run)."""
        rc = self.requests[request]
        keep = -(-rc.length // self.page_size)
        rc.epoch = next(self._epochs)
        for gi, g in enumerate(self.paged):
            table = rc.tables[gi]
            while len(table) > keep:
                page = table.pop()
                if page != RELEASED:
                    g.pool.free(page, request)

    def close(self, request: Hashable) -> None:
        rc = self.requests.pop(request)
        for gi, g in enumerate(self.paged):
            for page in rc.tables[gi]:
                if page != RELEASED:
                    g.pool.free(page, request)
            rc.tables[gi] = []
        self.slots.free(rc.state_slot, request)

    def table(self, request: Hashable, group: int) -> List[int]:
        return self.requests[request].tables[group]

    def table_epoch(self, request: Hashable) -> int:
        """A number that is new whenever the request's tables changed otherwise than by growing at their end
        (and for every opening of a request): who keeps a copy of a table may extend it while this stays."""
        return self.requests[request].epoch

    def state_slot(self, request: Hashable) -> int:
        return self.requests[request].state_slot

    # ---- books ---------------------------------------------------------------------------------------------
    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.paged]

    def check(self) -> None:
        """No page lost, none held twice: every held page is in exactly one table, once, under its holder."""
        self.slots.check()
        for gi, g in enumerate(self.paged):
            g.pool.check()
            seen = {}
            for rc in self.requests.values():
                for page in rc.tables[gi]:
                    if page == RELEASED:
                        continue
                    if page in seen:
                        raise PageBookkeepingError(f"group {gi}: page {page} is in the tables of {seen[page]!r} "
                                                   f"and {rc.request!r}")
                    seen[page] = rc.request
                    if g.pool.holder(page) != rc.request:
                        raise PageBookkeepingError(f"group {gi}: page {page} is in the table of {rc.request!r} "
                                                   f"but held by {g.pool.holder(page)!r}")
            if len(seen) != g.pool.num_held:
                raise PageBookkeepingError(f"group {gi}: {g.pool.num_held} pages are held, {len(seen)} are in tables")
