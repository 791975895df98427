"""The cache manager without a model: no page lost, held twice or freed twice, under random orders."""
import random

import pytest

from jllm_serve_b200.cache import (RELEASED, CacheManager, FixedState, PageBookkeepingError, PagedKeysValues, PagePool,
                                   PoolExhausted, StateSlotPool)


def test_block_table_arithmetic():
    # docs/24-paged-kv-cache.md:63-68 of the reference: p = 37, B = 16, table [7, 12, 3] -> page 3, row 5
    table, page_size, p = [7, 12, 3], 16, 37
    assert (table[p // page_size], p % page_size) == (3, 5)


def test_pool_alloc_free_reuse():
    pool = PagePool(3)
    a, b, c = pool.alloc("x"), pool.alloc("x"), pool.alloc("y")
    assert sorted([a, b, c]) == [0, 1, 2] and pool.num_free == 0
    with pytest.raises(PoolExhausted):
        pool.alloc("z")
    pool.free(b, "x")
    assert pool.alloc("z") == b and pool.reuses == 1          # the page freed last is used again first
    with pytest.raises(PageBookkeepingError):
        pool.free(a, "y")                                      # not the holder
    pool.free(a, "x")
    with pytest.raises(PageBookkeepingError):
        pool.free(a, "x")                                      # freed twice
    pool.check()


def test_one_long_request_takes_ceil_pages():
    # the reference's KvPoolTest: a conversation of 4100 tokens takes ceil(4100 / 16) blocks
    m = CacheManager([PagedKeysValues(2, 16)] * 3, 16, 300, 4)
    m.open("a")
    m.reserve("a", 0, 4100)
    m.commit("a", 4100)
    assert len(m.table("a", 0)) == 257 and m.free_pages() == [300 - 257]
    m.truncate("a", 33)                                        # pages wholly past 33 go back
    assert len(m.table("a", 0)) == 3 and m.length("a") == 33
    m.close("a")
    assert m.free_pages() == [300]                             # everything is released afterwards
    m.check()


def test_groups_by_need_and_tables_per_group():
    needs = [PagedKeysValues(2, 16), PagedKeysValues(2, 16, window=8), None, PagedKeysValues(2, 16),
             FixedState((4, 3)), PagedKeysValues(2, 16, window=8)]
    made = []
    m = CacheManager(needs, 4, 10, 2, allocate=lambda shape, kind: made.append((shape, kind)) or ("mem", shape))
    assert [g.runs for g in m.paged] == [[0, 3], [1, 5]] and [g.runs for g in m.fixed] == [[4]]
    assert ((2, 2, 10, 2, 4, 16), "kv") in made and ((1, 2, 4, 3), "float32") in made
    assert m.paged_group_of(3) == 0 and m.paged_group_of(5) == 1
    with pytest.raises(KeyError):
        m.paged_group_of(2)


def test_window_group_gives_pages_back_as_the_window_passes():
    m = CacheManager([PagedKeysValues(1, 8), PagedKeysValues(1, 8, window=6)], 4, 8, 2)
    m.open("a")
    m.reserve("a", 0, 20)
    released = m.commit("a", 20)
    # the next query (position 20) sees keys >= 15: pages 0..2 (positions 0..11) are passed; page 3 holds 12..15
    assert [p for g, p in released if g == 1] == m.table("a", 0)[:3] or len(released) == 3
    assert m.table("a", 1)[:3] == [RELEASED] * 3 and m.table("a", 1)[3] != RELEASED
    assert m.free_pages() == [8 - 5, 8 - 2]
    for pos in range(20, 31):                                  # decoding: the window group stays at <= 3 pages
        m.reserve("a", pos, 1)
        m.commit("a", pos + 1)
        assert sum(p != RELEASED for p in m.table("a", 1)) <= 3
        m.check()
    m.close("a")
    assert m.free_pages() == [8, 8]


def test_reserve_takes_all_or_nothing():
    m = CacheManager([PagedKeysValues(1, 8), PagedKeysValues(1, 8, window=6)], 4, 4, 3)
    m.open("a")
    m.open("b")
    m.reserve("a", 0, 9)          # 3 pages in both groups
    with pytest.raises(PoolExhausted):
        m.reserve("b", 0, 8)      # needs 2, one is free
    assert m.table("b", 0) == [] and m.table("b", 1) == [] and m.free_pages() == [1, 1]
    assert not m.can_reserve("b", 0, 8) and m.can_reserve("b", 0, 4)
    assert m.pages_missing("a", 9, 3) == [0, 0] and m.pages_missing("a", 9, 4) == [1, 1]
    m.check()


def test_state_slots():
    s = StateSlotPool(2)
    a, b = s.alloc("x"), s.alloc("y")
    with pytest.raises(PoolExhausted):
        s.alloc("z")
    s.free(a, "x")
    with pytest.raises(PageBookkeepingError):
        s.free(a, "x")
    assert s.alloc("z") == a
    s.check()
    m = CacheManager([FixedState((3,))], 4, 1, 2)
    m.open("p")
    m.open("q")
    assert {m.state_slot("p"), m.state_slot("q")} == {0, 1}
    with pytest.raises(PoolExhausted):
        m.open("r")
    m.close("p")
    m.open("r")


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    """Requests open, grow by portions and single tokens, rewind, and end in random order; after every
    operation every page is either free once or in exactly one table once."""
    rng = random.Random(seed)
    page = rng.choice([1, 4, 16])
    m = CacheManager([PagedKeysValues(2, 16), PagedKeysValues(2, 16, window=rng.choice([5, 40])), None], page, 40, 5)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.15 and len(live) < 5:
            rid = f"r{next_id}"
            next_id += 1
            m.open(rid)
            live[rid] = 0
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 33])
            try:
                m.reserve(rid, live[rid], n)
                live[rid] += n
                m.commit(rid, live[rid])
            except PoolExhausted:
                assert not m.can_reserve(rid, live[rid], n)
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            keep = rng.randrange(live[rid] + 1)
            try:
                m.truncate(rid, keep)
                live[rid] = min(live[rid], keep)
            except ValueError:
                pass                                           # a windowed group cannot rewind behind its window
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.length(rid) == n
            assert len(m.table(rid, 0)) >= -(-n // page)
    for rid in list(live):
        m.close(rid)
    m.check()
    assert m.free_pages() == [40, 40] and m.slots.num_free == 5


def test_table_epoch_changes_with_everything_but_growth():
    m = CacheManager([PagedKeysValues(2, 16, 0), PagedKeysValues(2, 16, 8)], page_size=4, num_pages=12, max_requests=2)
    m.open("a")
    e0 = m.table_epoch("a")
    m.reserve("a", 0, 13)
    assert m.table_epoch("a") == e0                      # growth at the end keeps it
    m.commit("a", 13)
    e1 = m.table_epoch("a")
    assert e1 != e0                                      # the windowed group gave a page back
    m.reserve("a", 13, 4)
    assert m.table_epoch("a") == e1
    m.trim("a")
    e2 = m.table_epoch("a")
    assert e2 != e1
    m.close("a")
    m.open("a")
    assert m.table_epoch("a") not in (e0, e1, e2)        # a request opened again is another one
    m.reserve("a", 0, 6)
    m.commit("a", 6)
    e3 = m.table_epoch("a")
    m.truncate("a", 2)
    assert m.table_epoch("a") != e3


def test_batch_tables_follow_the_requests_tables():
    """The batch builder extends its copy of a block table while the epoch stays; after a rewind, a request that
    changed rows, or a request opened again, the row is written anew."""
    import torch

    from jllm_serve_b200.engine.batch import BatchBuilder, Segment
    m = CacheManager([PagedKeysValues(1, 8, 0)], page_size=2, num_pages=64, max_requests=4)
    b = BatchBuilder(torch.device("cpu"), max_rows=32, max_segments=4, max_blocks=16, num_paged_groups=1, page_size=2, resident_blocks=296)
    rng = random.Random(0)
    lengths = {}

    def step(reqs, n_of):
        segs = []
        for r in reqs:
            if not m.is_open(r):
                m.open(r)
                lengths[r] = 0
            segs.append(Segment(r, [1] * n_of[r], lengths[r], [n_of[r] - 1]))
        batch = b.build(segs, m, vocab=10, reserve=True)
        row = 0
        for si, r in enumerate(reqs):
            table = m.table(r, 0)
            assert batch.block_tables[0][si, :len(table)].tolist() == table
            for i in range(n_of[r]):
                p = lengths[r] + i
                assert int(batch.slots[0][row]) == table[p // 2] * 2 + p % 2
                row += 1
            lengths[r] += n_of[r]
        assert b.commit(m) == [] and all(m.length(r) == lengths[r] for r in reqs)

    step(["a", "b"], {"a": 5, "b": 3})
    for _ in range(6):
        step(["a", "b"], {"a": 1, "b": 1})
    step(["b", "a"], {"a": 1, "b": 1})                      # rows swapped
    m.truncate("a", 3)                                      # a rewind, then other pages under the same indices
    m.open("c")
    m.reserve("c", 0, 7)
    lengths["a"] = 3
    step(["b", "a"], {"a": 4, "b": 1})
    m.close("b")                                            # opened again under the same name
    step(["b", "a"], {"a": 1, "b": 2})
    for _ in range(8):
        reqs = rng.sample(["a", "b"], 2)
        step(reqs, {"a": rng.randint(1, 3), "b": 1})


def test_pool_sized_from_free_memory():
    """A share of what is free after a reserve, in whole pages over all groups, capped by what the requests can use
    (the reference's context budget: src/main/java/org/robomiri/jllm/ContextBudget.java:30-40,143-186)."""
    from jllm_serve_b200.cache import plan_pages
    from jllm_serve_b200.cache.budget import group_page_bytes
    GB = 1 << 30
    # Qwen3-32B shape: 64 layer runs, 8 kv heads of 128, pages of 16 positions, bfloat16: 4 MiB a page
    per_page = group_page_bytes(64, 8, 128, 16, 2)
    assert per_page == 64 * 2 * 8 * 16 * 128 * 2 == 4 << 20
    plan = plan_pages(free_bytes=110 * GB, total_bytes=180 * GB, page_bytes_by_group=[per_page], page_size=16, ctx=8192,
                      max_requests=64, share=0.9, held_bytes=1 * GB)
    reserve = 180 * GB // 32
    assert plan.limited_by == "memory" and plan.pages == int(0.9 * (110 * GB - GB - reserve)) // per_page
    assert plan.pool_bytes <= plan.budget < plan.pool_bytes + per_page
    few = plan_pages(110 * GB, 180 * GB, [per_page], 16, 8192, max_requests=4, share=0.9)
    assert few.limited_by == "requests" and few.pages == 4 * 512          # never more than the requests can use
    two = plan_pages(10 * GB, 180 * GB, [per_page, per_page // 2], 16, 1 << 20, 64, 0.6)
    assert two.bytes_per_page == per_page * 3 // 2 and two.pages == int(0.6 * (10 * GB - reserve)) // two.bytes_per_page
    with pytest.raises(MemoryError):
        plan_pages(5 * GB, 180 * GB, [per_page], 16, 8192, 4, 0.6)          # the reserve alone is 5.6 GB: nothing is left
    with pytest.raises(ValueError):
        plan_pages(110 * GB, 180 * GB, [per_page], 16, 8192, 4, share=1.5)
    assert plan_pages(110 * GB, 180 * GB, [], 16, 8192, 4).pages == 1     # a model that keeps no keys and values
    from jllm_serve_b200.cache import CacheManager, FixedState, PagedKeysValues
    needs = [PagedKeysValues(2, 16), (PagedKeysValues(2, 16, window=8), FixedState((3,))), None, PagedKeysValues(2, 16)]
    assert CacheManager.page_bytes(needs, 4, 2) == [2 * 2 * 2 * 4 * 16 * 2, 1 * 2 * 2 * 4 * 16 * 2]


def test_a_run_may_keep_paged_keys_and_a_state():
    from jllm_serve_b200.cache import CacheManager, FixedState, PagedKeysValues
    needs = [(PagedKeysValues(2, 16), FixedState((5,))), FixedState((5,)), (FixedState((5,)), FixedState((5,)), FixedState((2,)))]
    made = {}
    m = CacheManager(needs, 4, 10, 3, allocate=lambda shape, kind: made.setdefault((shape, kind), object()))
    assert [g.runs for g in m.paged] == [[0]] and [g.runs for g in m.fixed] == [[0, 1, 2], [2], [2]]
    assert m.paged_of_run == {0: 0} and m.fixed_of_run == {0: [0], 1: [0], 2: [0, 1, 2]}
    assert ((3, 3, 5), "float32") in made and ((1, 3, 5), "float32") in made and ((1, 3, 2), "float32") in made
    with pytest.raises(TypeError, match="two needs of paged"):
        CacheManager([(PagedKeysValues(2, 16), PagedKeysValues(2, 16, window=4))], 4, 10, 3)
    with pytest.raises(KeyError):
        m.state(0, 1)
