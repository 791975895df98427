"""The cache manager: groups of layer runs, a block table per request and group, and state slots.

Every mixer says what it needs to keep between steps (`CacheNeed`): keys and values for
all earlier positions, for a window of them, a state of fixed size, or nothing. Layer runs
with the same need form a *group*; a group of keys and values has a page pool of its own
and every request has one block table per group (position p of the request lives in page
`table[p // page_size]`, row `p % page_size`: docs/24-paged-kv-cache.md:59-72 of the
reference, which has a single group because its layers always move together, :395-397).
A windowed group gives pages back as soon as the window has passed them; the others keep
theirs until the request ends. A fixed-state group has storage [slots, ...] and each
request one slot, which is zeroed when the request is opened. A mixer may name several needs
(paged keys and values and one or more states): its run is then a member of a group of each.

Before a step, `reserve(request, start, n)` makes sure pages exist for positions
[start, start + n) in every group (the reference's `beginWrite`,
src/main/java/org/robomiri/jllm/kv/KvSequence.java:116-146); it takes all of them or none
and raises `PoolExhausted`. After the step `commit(request, length)` records the new
length and releases what a window has passed. `close` gives everything back.

The manager is host bookkeeping; the device memory of a group is made by the `allocate`
callable it is given (None in tests that need no device). The books themselves (pools, tables,
lengths, slots) are kept by the C++ host library (csrc/host/host_runtime.cpp), which also packs
a step's batch tables from them; this class chooses the groups, owns the device memory and the
names of the requests, and is the library's face towards the rest of the engine.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Dict, Hashable, Iterator, List, Optional, Sequence, Tuple

from . import native
from .pages import PageBookkeepingError, PoolExhausted, PoolView  # noqa: F401

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
    pool: Optional[PoolView] = None        # a view of the group's page pool
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
    """A snapshot of what a request holds (the live books are the library's)."""
    request: Hashable
    state_slot: int
    length: int
    tables: List[List[int]]                # one per paged group; -1 = a page that a window has passed
    epoch: int                             # changes whenever a table changed otherwise than by growing at its end


class _Requests:
    """The open requests, as a read-only mapping name -> RequestCache snapshot."""

    def __init__(self, manager: "CacheManager"):
        self._m = manager

    def __len__(self) -> int:
        return native.lib().jh_cache_num_requests(self._m._ptr)

    def __bool__(self) -> bool:
        return len(self) > 0

    def __contains__(self, request) -> bool:
        return self._m.is_open(request)

    def __iter__(self) -> Iterator:
        n = len(self)
        buf = (ctypes.c_longlong * max(1, n))()
        got = native.lib().jh_cache_request_ids(self._m._ptr, buf, n)
        return iter([self._m._names.name(buf[i]) for i in range(got)])

    def __getitem__(self, request) -> RequestCache:
        return self._m._snapshot(request)

    def get(self, request, default=None):
        return self._m._snapshot(request) if self._m.is_open(request) else default

    def keys(self):
        return list(iter(self))

    def values(self):
        return [self._m._snapshot(r) for r in self]


def needs_of(need) -> Tuple[CacheNeed, ...]:
    """What a mixer's `cache_need` returned, as a tuple: nothing, one need, or several (a mixer that keeps paged
    keys and values AND a state of fixed size says both)."""
    if need is None:
        return ()
    if isinstance(need, CacheNeed):
        return () if type(need) is CacheNeed else (need,)
    if isinstance(need, (tuple, list)):
        return tuple(n for one in need for n in needs_of(one))
    raise TypeError(f"unknown cache need {need!r}")


def group_runs(needs: Sequence) -> tuple:
    """Layer runs with the same need share a group: (paged groups, fixed-state groups, {run: paged group},
    {run: [fixed-state groups, in the order the run named them]}). A run may have at most one paged need."""
    paged: List[PagedGroup] = []
    fixed: List[StateGroup] = []
    paged_of_run: Dict[int, int] = {}
    fixed_of_run: Dict[int, List[int]] = {}
    for run, need in enumerate(needs):
        for one in needs_of(need):
            if isinstance(one, PagedKeysValues):
                if run in paged_of_run:
                    raise TypeError(f"layer run {run} names two needs of paged keys and values; one is built")
                groups, kind = paged, PagedGroup
            elif isinstance(one, FixedState):
                groups, kind = fixed, StateGroup
            else:
                raise TypeError(f"layer run {run}: unknown cache need {one!r}")
            for gi, g in enumerate(groups):
                # a run that wants two states of the same shape gets two groups: a group holds a run once
                if g.need == one and run not in g.runs:
                    g.runs.append(run)
                    break
            else:
                gi = len(groups)
                groups.append(kind(one, [run]))
            if kind is PagedGroup:
                paged_of_run[run] = gi
            else:
                fixed_of_run.setdefault(run, []).append(gi)
    return paged, fixed, paged_of_run, fixed_of_run


class CacheManager:
    def __init__(self, needs: Sequence[Optional[CacheNeed]], page_size: int, num_pages: int, max_requests: int,
                 allocate: Optional[Callable] = None):
        """`needs[i]` is the need of schedule entry i (None for a run that keeps nothing or reads another's cache)."""
        if page_size < 1:
            raise ValueError(f"page_size={page_size} must be at least 1")
        if num_pages < 1:
            raise ValueError(f"a pool needs at least one page, got {num_pages}")
        self.page_size = page_size
        self.num_pages = num_pages
        self.paged, self.fixed, self.paged_of_run, self.fixed_of_run = group_runs(needs)
        L = native.lib()
        G = len(self.paged)
        windows = (ctypes.c_int * max(1, G))(*[g.need.window for g in self.paged])
        self._names = native.Names()
        self._ptr = L.jh_cache_new(G, windows, page_size, num_pages, max_requests)
        if not self._ptr:
            native.check(1)
        for gi, g in enumerate(self.paged):
            g.pool = PoolView(L.jh_cache_pool(self._ptr, gi), self._names, num_pages, f"group{gi}")
            g.pool.num_pages = num_pages
        self.slots = PoolView(L.jh_cache_pool(self._ptr, -1), self._names, max_requests, "state slots")
        self.slots.num_slots = max_requests
        self.requests = _Requests(self)
        self._ints = (ctypes.c_int * max(8, G))()
        if allocate is not None:
            for g in self.paged:
                g.storage = allocate((len(g.runs), 2, num_pages, g.need.kv_heads, page_size, g.need.head_dim), "kv")
            for g in self.fixed:
                g.storage = allocate((len(g.runs), max_requests) + tuple(g.need.shape), g.need.dtype)

    def release_storage(self) -> None:
        """Lets go of the groups' device storage now (the books stay): for a runner that is being closed."""
        for g in list(self.paged) + list(self.fixed):
            g.storage = None

    def __del__(self):
        try:
            if getattr(self, "_ptr", None):
                native.lib().jh_cache_delete(self._ptr)
                self._ptr = None
        except Exception:        # the interpreter is shutting down and the module is gone
            pass

    def _h(self, request: Hashable) -> int:
        return self._names.handle(request)

    def _check(self, code: int) -> None:
        if code:
            native.check(code, self._names)

    # ---- what a layer run reads and writes ----------------------------------------------------------------
    def paged_group_of(self, run: int) -> int:
        if run not in self.paged_of_run:
            raise KeyError(f"layer run {run} keeps no keys and values")
        return self.paged_of_run[run]

    def keys_values(self, run: int):
        return self.paged[self.paged_group_of(run)].keys_values(run)

    def states(self, run: int) -> list:
        """The fixed-size states of a run, [slots, ...] each, in the order its mixer named them."""
        return [self.fixed[gi].state(run) for gi in self.fixed_of_run.get(run, ())]

    def state(self, run: int, which: int = 0):
        held = self.fixed_of_run.get(run, ())
        if which >= len(held):
            raise KeyError(f"layer run {run} keeps no fixed-size state" + (f" number {which}" if held else ""))
        return self.fixed[held[which]].state(run)

    @staticmethod
    def page_bytes(needs: Sequence, page_size: int, element_bytes: int) -> List[int]:
        """Bytes of one page of every paged group these needs would form (for sizing the pool before it exists)."""
        from .budget import group_page_bytes
        return [group_page_bytes(len(g.runs), g.need.kv_heads, g.need.head_dim, page_size, element_bytes)
                for g in group_runs(needs)[0]]

    # ---- requests ---------------------------------------------------------------------------------------
    def open(self, request: Hashable) -> RequestCache:
        if self.is_open(request):
            raise ValueError(f"request {request!r} is open already")
        h = self._names.handle(request, make=True)
        code = native.lib().jh_cache_open(self._ptr, h, None)
        if code:
            self._names.forget(request)
            self._check(code)
        snap = self._snapshot(request)
        for g in self.fixed:          # a slot is handed out clean: whoever held it before left its state there
            if hasattr(g.storage, "zero_"):
                g.storage[:, snap.state_slot].zero_()
        return snap

    def is_open(self, request: Hashable) -> bool:
        return request in self._names._handle      # the names that have a handle are the open requests

    def _info(self, request: Hashable):
        length, slot, epoch = ctypes.c_int(), ctypes.c_int(), ctypes.c_longlong()
        code = native.lib().jh_cache_request(self._ptr, self._h(request), ctypes.byref(length), ctypes.byref(slot),
                                             ctypes.byref(epoch), self._ints)
        if code:
            raise KeyError(request)
        return length.value, slot.value, epoch.value, [self._ints[g] for g in range(len(self.paged))]

    def _snapshot(self, request: Hashable) -> RequestCache:
        length, slot, epoch, _ = self._info(request)
        return RequestCache(request, slot, length, [self.table(request, g) for g in range(len(self.paged))], epoch)

    def length(self, request: Hashable) -> int:
        return self._info(request)[0]

    def pages_missing(self, request: Hashable, start: int, n: int) -> List[int]:
        """How many pages each paged group would have to take for positions [start, start + n)."""
        native.lib().jh_cache_pages_missing(self._ptr, self._h(request), start, n, self._ints)
        return [self._ints[g] for g in range(len(self.paged))]

    def can_reserve(self, request: Hashable, start: int, n: int) -> bool:
        return bool(native.lib().jh_cache_can_reserve(self._ptr, self._h(request), start, n))

    def reserve(self, request: Hashable, start: int, n: int) -> None:
        """Pages for positions [start, start + n) in every group, all or none; positions from `start`
        on that an earlier step wrote are dropped first (a rewind)."""
        self._check(native.lib().jh_cache_reserve(self._ptr, self._h(request), start, n))

    def commit(self, request: Hashable, length: int) -> List[Tuple[int, int]]:
        """The request now holds `length` positions. Returns the (group, page) pairs given back
        because a window has passed them."""
        cap = 2 * (self.num_pages if any(g.need.window > 0 for g in self.paged) else 0) * max(1, len(self.paged))
        buf = (ctypes.c_int * max(2, cap))()
        count = ctypes.c_int()
        self._check(native.lib().jh_cache_commit(self._ptr, self._h(request), length, buf, cap, ctypes.byref(count)))
        return [(buf[2 * i], buf[2 * i + 1]) for i in range(count.value)]

    def truncate(self, request: Hashable, length: int) -> None:
        """Forget positions >= length: pages wholly past it go back (KvSequence.java:149-157). A windowed
        group cannot go back behind pages it has given up already."""
        self._check(native.lib().jh_cache_truncate(self._ptr, self._h(request), length))

    def trim(self, request: Hashable) -> None:
        """Give back pages reserved beyond the committed length (a step that was reserved but did not run)."""
        self._check(native.lib().jh_cache_trim(self._ptr, self._h(request)))

    def close(self, request: Hashable) -> None:
        code = native.lib().jh_cache_close(self._ptr, self._h(request))
        if code == 4:
            raise KeyError(request)
        self._check(code)
        self._names.forget(request)

    def table(self, request: Hashable, group: int) -> List[int]:
        """A copy of the request's block table of one group."""
        entries = self._info(request)[3][group]
        buf = (ctypes.c_int * max(1, entries))()
        self._check(native.lib().jh_cache_table(self._ptr, self._h(request), group, buf, entries))
        return list(buf[:entries])

    def table_epoch(self, request: Hashable) -> int:
        """A number that is new whenever the request's tables changed otherwise than by growing at their end
        (and for every opening of a request): who keeps a copy of a table may extend it while this stays."""
        return self._info(request)[2]

    def state_slot(self, request: Hashable) -> int:
        return self._info(request)[1]

    # ---- a whole step at once ------------------------------------------------------------------------------------
    def handles(self, requests: Sequence[Hashable]) -> List[int]:
        return [self._names.handle(r) for r in requests]

    def reserve_all(self, requests: Sequence[Hashable], starts: Sequence[int], counts: Sequence[int]) -> None:
        """`reserve` for every request of a step in one call: all of them get their pages, or none does (what the
        earlier ones took is given back) and `PoolExhausted` is raised."""
        n = len(requests)
        ids = (ctypes.c_longlong * n)(*self.handles(requests))
        a, b = (ctypes.c_int * n)(*starts), (ctypes.c_int * n)(*counts)
        self._check(native.lib().jh_step_reserve(self._ptr, n, ids, a, b))

    # ---- books ---------------------------------------------------------------------------------------------
    def free_pages(self) -> List[int]:
        native.lib().jh_cache_free_pages(self._ptr, self._ints)
        return [self._ints[g] for g in range(len(self.paged))]

    def check(self) -> None:
        """No page lost, none held twice: every held page is in exactly one table, once, under its holder."""
        self._check(native.lib().jh_cache_check(self._ptr))
