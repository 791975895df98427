"""Page pools and state slots: who holds which page, and nothing about what a page contains.

A page ("block" in the reference: docs/24-paged-kv-cache.md:57-72,
src/main/java/org/robomiri/jllm/kv/KvPool.java:249-275) is `page_size` consecutive positions
of every layer run of one group. Ids are plain integers, stable for the pool's life. The
pool hands out the page freed last first, so a page that has just been given back is the
first to be used again: reuse happens early and shows faults early.

Without a prefix cache there is nothing to evict: a pool with no free page raises
`PoolExhausted` and the caller (the scheduler) decides what to do.

The books themselves are kept by the C++ host library (csrc/host/host_runtime.cpp); the classes
here are its faces: a pool of its own (`PagePool`, `StateSlotPool`) or a view of a pool that
belongs to a cache (`PoolView`).
"""
from __future__ import annotations

import ctypes
from typing import Hashable

from . import native
from .native import PageBookkeepingError, PoolExhausted  # noqa: F401  (the names live here for callers)


class PoolView:
    """What can be asked of a pool; `_ptr` is the library's pool, `_names` says who the holders are."""

    def __init__(self, ptr, names: native.Names, num: int, name: str):
        self._ptr, self._names, self._num, self.name = ptr, names, num, name

    @property
    def num_free(self) -> int:
        return native.lib().jh_pool_num_free(self._ptr)

    @property
    def num_held(self) -> int:
        return self._num - self.num_free

    def _stats(self):
        a, r = ctypes.c_longlong(), ctypes.c_longlong()
        native.lib().jh_pool_stats(self._ptr, ctypes.byref(a), ctypes.byref(r))
        return a.value, r.value

    @property
    def allocations(self) -> int:
        return self._stats()[0]

    @property
    def reuses(self) -> int:
        return self._stats()[1]

    def holder(self, index: int):
        h = native.lib().jh_pool_holder(self._ptr, index)
        return None if h == native.NOBODY else self._names.name(h)

    def check(self) -> None:
        native.check(native.lib().jh_pool_check(self._ptr), self._names)


class _OwnPool(PoolView):
    def __init__(self, count: int, name: str, what: str):
        if count < 1:
            raise ValueError(f"a pool needs at least one {what}, got {count}")
        ptr = native.lib().jh_pool_new(count, name.encode())
        super().__init__(ptr, native.Names(), count, name)

    def __del__(self):
        try:
            if getattr(self, "_ptr", None):
                native.lib().jh_pool_delete(self._ptr)
                self._ptr = None
        except Exception:        # the interpreter is shutting down and the module is gone
            pass

    def alloc(self, holder: Hashable) -> int:
        if holder is None:
            raise ValueError("a page needs a holder")
        out = ctypes.c_int()
        native.check(native.lib().jh_pool_alloc(self._ptr, self._names.handle(holder, make=True), ctypes.byref(out)),
                     self._names)
        return out.value

    def free(self, index: int, holder: Hashable) -> None:
        native.check(native.lib().jh_pool_free(self._ptr, index, self._names.handle(holder, make=True)), self._names)


class PagePool(_OwnPool):
    def __init__(self, num_pages: int, name: str = "pages"):
        super().__init__(num_pages, name, "page")
        self.num_pages = num_pages


class StateSlotPool(_OwnPool):
    """Slots of fixed size for per-request state (recurrent or convolution state of a mixer that keeps
    some). The reference keeps such state inside each slot's backend, outside the pool
    (docs/24-paged-kv-cache.md:349-351); here a request takes one slot id when it is admitted and
    gives it back when it ends, and every fixed-state group has storage [num_slots, ...] indexed by it."""

    def __init__(self, num_slots: int):
        super().__init__(num_slots, "state slots", "slot")
        self.num_slots = num_slots
