"""The cache manager and the batch tables on a fake storage whose rows are hashes of the token prefix (no GPU).

As in the reference's pool test (src/test/java/org/robomiri/jllm/KvPoolTest.java:16-50), a "row" of the cache is
the rolling hash of the request's tokens up to its position: like a real key it depends on the whole prefix, so a
row that is read through a block table must be the row that was written for exactly that (request, position),
and every mistake in the books (a page handed to two requests, a table row that was not refreshed after a rewind,
a released page that is still read) shows as a wrong number. Rows are written where the step's `slots` say and
read back through the step's block tables, i.e. through what the kernels would use. Freed pages are overwritten
with a poison value. Two groups: one keeps everything, one a window.
"""
import random

import numpy as np
import pytest
import torch

from jllm_serve_b200.cache import RELEASED, CacheManager, PagedKeysValues, PoolExhausted
from jllm_serve_b200.engine.batch import BatchBuilder, Segment

POISON = -7
MASK = (1 << 61) - 1


def prefix_hashes(tokens):
    out, h = [], 1469598103934665603 & MASK
    for t in tokens:
        h = ((h * 1099511628211) ^ (t + 1)) & MASK
        out.append(h)
    return out


class FakeCache:
    """A pool of `pages` pages of `page` rows per group, one int64 per row."""

    def __init__(self, page, pages, max_requests, window, ctx):
        self.page, self.window = page, window
        self.manager = CacheManager([PagedKeysValues(1, 8, 0), PagedKeysValues(1, 8, window)], page, pages, max_requests)
        self.builder = BatchBuilder(torch.device("cpu"), max_rows=64, max_segments=max_requests,
                                    max_blocks=-(-ctx // page), num_paged_groups=2, page_size=page, resident_blocks=296)
        self.rows = [np.full(pages * page, POISON, np.int64) for _ in range(2)]
        self.tokens = {}            # request -> its tokens so far (what the rows must be hashes of)

    def poison(self, pages):
        for g, pg in pages:
            self.rows[g][pg * self.page:(pg + 1) * self.page] = POISON

    def held(self, request):
        return [(g, pg) for g in range(2) for pg in self.manager.table(request, g) if pg != RELEASED]

    def step(self, feeds):
        """feeds: [(request, new tokens)]; all or nothing. Writes the new rows through the step's slots, then reads
        every row each request may see through the step's block tables."""
        segs = []
        for r, new in feeds:
            if not self.manager.is_open(r):
                self.manager.open(r)
                self.tokens[r] = []
            segs.append(Segment(r, new, len(self.tokens[r]), [len(new) - 1]))
        batch = self.builder.build(segs, self.manager, vocab=1 << 20, reserve=True)
        row = 0
        for r, new in feeds:
            hashes = prefix_hashes(self.tokens[r] + list(new))
            for i in range(len(new)):
                for g in range(2):
                    slot = int(batch.slots[g][row])
                    assert self.rows[g][slot] == POISON, f"{r}: slot {slot} of group {g} is in use"
                    self.rows[g][slot] = hashes[len(self.tokens[r]) + i]
                row += 1
            self.tokens[r] = self.tokens[r] + list(new)
        for si, (r, new) in enumerate(feeds):       # what a kernel would read: the step's tables, not the manager's
            hashes = prefix_hashes(self.tokens[r])
            n = len(hashes)
            for g in range(2):
                table = batch.block_tables[g][si].tolist()
                first = 0 if g == 0 else max(0, n - len(new) + 1 - self.window)   # the oldest key any new row sees
                for p in range(first, n):
                    pg = table[p // self.page]
                    assert pg >= 0, f"{r}: position {p} of group {g} reads a released page"
                    assert self.rows[g][pg * self.page + p % self.page] == hashes[p], (r, g, p)
        self.poison(self.builder.commit(self.manager))
        self.manager.check()

    def close(self, r):
        pages = self.held(r)
        self.manager.close(r)
        self.poison(pages)
        del self.tokens[r]

    def truncate(self, r, n):
        before = set(self.held(r))
        self.manager.truncate(r, n)
        self.poison(before - set(self.held(r)))
        self.tokens[r] = self.tokens[r][:n]
        for g in range(2):      # the rows of the cut-off positions inside a kept page are free to be written again
            for p in range(n, -(-n // self.page) * self.page):
                pg = self.manager.table(r, g)[p // self.page] if p // self.page < len(self.manager.table(r, g)) else RELEASED
                if pg != RELEASED:
                    self.rows[g][pg * self.page + p % self.page] = POISON


def test_rows_read_through_block_tables_are_the_rows_written_under_random_orders():
    rng = random.Random(5)
    ctx = 96
    fake = FakeCache(page=4, pages=40, max_requests=5, window=10, ctx=ctx)
    names = [f"q{i}" for i in range(9)]
    steps = exhausted = truncated = reopened = refused = 0
    for _ in range(600):
        live = list(fake.tokens)
        roll = rng.random()
        if live and roll < 0.08:
            fake.close(rng.choice(live))
            continue
        if live and roll < 0.14:
            r = rng.choice(live)
            # the windowed group cannot go back behind what it has released: cut inside the last page only
            n = len(fake.tokens[r])
            keep = rng.randint(max(1, n - 6), n)
            # a rewind is refused when the window group has already released a page that the next query would see
            first_needed = lambda length: max(0, length + 1 - fake.window) // fake.page
            if first_needed(n) > first_needed(keep):
                with pytest.raises(ValueError, match="recompute from the start"):
                    fake.truncate(r, keep)
                assert len(fake.tokens[r]) == n and fake.manager.length(r) == n
                refused += 1
            else:
                fake.truncate(r, keep)
                truncated += 1
            continue
        if live and roll < 0.18:      # preempted: everything back, then fed again from the start in later steps
            r = rng.choice(live)
            fake.close(r)
            reopened += 1
            continue
        chosen = rng.sample(names, rng.randint(1, 4))
        room, kept = 5 - len(fake.tokens), []
        for r in chosen:
            if r in fake.tokens:
                kept.append(r)
            elif room > 0:
                kept.append(r)
                room -= 1
        chosen = kept
        feeds = []
        for r in chosen:
            have = len(fake.tokens.get(r, []))
            if have >= ctx - 1:
                continue
            n = min(ctx - have, rng.choice([1, 1, 1, 2, 3, 7, 13]))
            feeds.append((r, [rng.randrange(1000) for _ in range(n)]))
        if not feeds:
            continue
        before = {r: list(fake.tokens.get(r, [])) for r, _ in feeds}
        opened = [r for r, _ in feeds if r not in fake.tokens]
        try:
            fake.step(feeds)
            steps += 1
        except PoolExhausted:
            exhausted += 1
            for r in opened:                       # nothing of the step happened: those it opened hold nothing
                assert not fake.held(r)
                fake.manager.close(r)
                del fake.tokens[r]
            for r, toks in before.items():
                if r in fake.tokens:
                    assert fake.tokens[r] == toks
            fake.manager.check()
            if fake.tokens:
                fake.close(max(fake.tokens, key=lambda r: len(fake.tokens[r])))
    for r in list(fake.tokens):
        fake.close(r)
    assert fake.manager.free_pages() == [40, 40]
    assert all((rows == POISON).all() for rows in fake.rows), "a freed page kept rows"
    assert steps > 200 and exhausted > 0 and truncated > 5 and reopened > 3 and refused > 0, \
        (steps, exhausted, truncated, reopened, refused)
