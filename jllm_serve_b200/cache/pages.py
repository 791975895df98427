"""Page pools and state slots: who holds which page, and nothing about what a page contains.

A page ("block" in the reference: docs/24-paged-kv-cache.md:57-72,
src/main/java/org/robomiri/jllm/kv/KvPool.java:249-275) is `page_size` consecutive positions
of every layer run of one group. Ids are plain integers, stable for the pool's life. The
pool hands out the page freed last first, so a page that has just been given back is the
first to be used again: reuse happens early and shows faults early.

Without a prefix cache there is nothing to evict: a pool with no free page raises
`PoolExhausted` and the caller (the scheduler) decides what to do.
"""
from __future__ import annotations

from typing import Hashable, List, Optional


class PoolExhausted(RuntimeError):
    """No free page (the reference's KvPoolExhausted, src/main/java/org/robomiri/jllm/kv/KvPoolExhausted.java:4)."""


class PageBookkeepingError(AssertionError):
    """A page was freed twice, freed by someone who does not hold it, or handed out twice: a bug."""


class PagePool:
    def __init__(self, num_pages: int, name: str = "pages"):
        if num_pages < 1:
            raise ValueError(f"a pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self.name = name
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # pop() takes page 0 first
        self._holder: List[Optional[Hashable]] = [None] * num_pages
        self.allocations = 0
        self.reuses = 0
        self._used_before = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, holder: Hashable) -> int:
        if holder is None:
            raise ValueError("a page needs a holder")
        if not self._free:
            raise PoolExhausted(f"{self.name}: all {self.num_pages} pages are held")
        page = self._free.pop()
        if self._holder[page] is not None:
            raise PageBookkeepingError(f"{self.name}: page {page} is free and held by {self._holder[page]!r}")
        self._holder[page] = holder
        self.allocations += 1
        if self._used_before[page]:
            self.reuses += 1
        self._used_before[page] = True
        return page

    def free(self, page: int, holder: Hashable) -> None:
        if not 0 <= page < self.num_pages:
            raise PageBookkeepingError(f"{self.name}: page {page} does not exist")
        if self._holder[page] is None:
            raise PageBookkeepingError(f"{self.name}: page {page} is freed twice")
        if self._holder[page] != holder:
            raise PageBookkeepingError(f"{self.name}: page {page} is held by {self._holder[page]!r}, "
                                       f"freed by {holder!r}")
        self._holder[page] = None
        self._free.append(page)

    def holder(self, page: int):
        return self._holder[page]

    def check(self) -> None:
        """Every page is either free once or held once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageBookkeepingError(f"{self.name}: a page is on the free list twice")
        for page in range(self.num_pages):
            if (page in free) == (self._holder[page] is not None):
                raise PageBookkeepingError(f"{self.name}: page {page} is {'free and held' if page in free else 'lost'}")


class StateSlotPool:
    """Slots of fixed size for per-request state (recurrent or convolution state of a mixer that keeps
    some). The reference keeps such state inside each slot's backend, outside the pool
    (docs/24-paged-kv-cache.md:349-351); here a request takes one slot id when it is admitted and
    gives it back when it ends, and every fixed-state group has storage [num_slots, ...] indexed by it."""

    def __init__(self, num_slots: int):
        if num_slots < 1:
            raise ValueError(f"a slot pool needs at least one slot, got {num_slots}")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._holder: List[Optional[Hashable]] = [None] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, holder: Hashable) -> int:
        if not self._free:
            raise PoolExhausted(f"all {self.num_slots} state slots are held")
        slot = self._free.pop()
        self._holder[slot] = holder
        return slot

    def free(self, slot: int, holder: Hashable) -> None:
        if not 0 <= slot < self.num_slots or self._holder[slot] is None:
            raise PageBookkeepingError(f"state slot {slot} is freed twice or does not exist")
        if self._holder[slot] != holder:
            raise PageBookkeepingError(f"state slot {slot} is held by {self._holder[slot]!r}, freed by {holder!r}")
        self._holder[slot] = None
        self._free.append(slot)

    def check(self) -> None:
        free = set(self._free)
        for s in range(self.num_slots):
            if (s in free) == (self._holder[s] is not None):
                raise PageBookkeepingError(f"state slot {s} is {'free and held' if s in free else 'lost'}")
