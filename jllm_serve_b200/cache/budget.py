"""How many pages the cache pool gets when nobody chose a number: a share of the memory that is free.

The reference sizes its caches from the memory that is left once the weights are loaded: a reserve for
activations and scratch comes off, and of the rest a share (0.6 there) goes to the caches, so that other
programs and the allocator's slack keep some room (src/main/java/org/robomiri/jllm/ContextBudget.java:30-40,
143-186; its reserve is the larger of 512 MB and 1/32 of the device's memory). There the result is a context
length per slot; here, with one pool that all requests share, it is a number of pages, and never more than the
requests could use if each of them filled its context.

`plan_pages` is a pure function, tested without a device; the model runner gathers the numbers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

DEFAULT_SHARE = 0.6
MIN_RESERVE = 512 << 20


@dataclass(frozen=True)
class PagePlan:
    pages: int
    bytes_per_page: int                    # over all paged groups: every group has a page of each number
    budget: int                            # bytes the pools may take
    limited_by: str                        # "memory" or "requests"
    basis: str                             # the arithmetic, for the log

    @property
    def pool_bytes(self) -> int:
        return self.pages * self.bytes_per_page


def group_page_bytes(runs: int, kv_heads: int, head_dim: int, page_size: int, element_bytes: int) -> int:
    """Bytes of one page of a group: keys and values of `page_size` positions for each of its layer runs."""
    return runs * 2 * kv_heads * page_size * head_dim * element_bytes


def plan_pages(free_bytes: int, total_bytes: int, page_bytes_by_group: Sequence[int], page_size: int, ctx: int,
               max_requests: int, share: float = DEFAULT_SHARE, held_bytes: int = 0) -> PagePlan:
    """`free_bytes`: free device memory now (weights and fixed buffers already taken); `held_bytes`: what is still
    to be taken before the pool (buffers that are made at the first step). The pool gets `share` of what is left
    after a reserve of max(512 MB, total / 32), but no more pages than `max_requests` full contexts need."""
    if not 0 < share <= 1:
        raise ValueError(f"the cache's share of the free memory must be in (0, 1], got {share}")
    per_page = int(sum(page_bytes_by_group))
    if per_page <= 0:
        return PagePlan(1, 0, 0, "requests", "no layer keeps keys and values: one page")
    reserve = max(MIN_RESERVE, total_bytes // 32)
    usable = max(0, free_bytes - held_bytes - reserve)
    budget = int(share * usable)
    by_memory = budget // per_page
    by_requests = max_requests * (-(-ctx // page_size))
    pages = min(by_memory, by_requests)
    basis = (f"free {free_bytes / 1e9:.1f} GB - buffers {held_bytes / 1e9:.1f} - reserve {reserve / 1e9:.1f} = "
             f"{usable / 1e9:.1f} GB, {100 * share:.0f}% for the cache = {budget / 1e9:.1f} GB at "
             f"{per_page / 1e6:.2f} MB a page")
    if pages < 1:
        raise MemoryError(f"no room for a single cache page: {basis}")
    return PagePlan(int(pages), per_page, budget, "memory" if by_memory <= by_requests else "requests", basis)
