"""The scheduler's decisions without a model: pass forming, admission, finishing, preemption (CPU)."""
import random

import pytest

from jllm_serve_b200.cache import CacheManager, PagedKeysValues
from jllm_serve_b200.cli import Settings, SettingsError, main
from jllm_serve_b200.engine.scheduler import Item, Request, Scheduler, plan_pass
from jllm_serve_b200.sampling import SamplingParams


def names(picks):
    return [f"{p.ref}:{p.rows}" for p in picks]


def worked_example():
    # the reference's worked pass (docs/25-scheduler.md:140-159; SchedulerPolicyTest.java:60-108): decoding
    # slots D1..D6, a 5-row verification run V1, and two prompts of 256 rows each waiting to be prefilled
    return [Item("D1", "rider", 1, 0), Item("P-A", "chunk", 256, 1), Item("V1", "rider", 5, 2),
            Item("D2", "rider", 1, 3), Item("D3", "rider", 1, 4), Item("D4", "rider", 1, 5), Item("D5", "rider", 1, 6),
            Item("D6", "rider", 1, 7), Item("P-B", "chunk", 256, 8)]


def test_riders_first_then_one_chunk():
    picks = plan_pass(worked_example(), 288, 16)
    assert names(picks) == ["P-A:256", "D1:1", "V1:5", "D2:1", "D3:1", "D4:1", "D5:1", "D6:1"]
    assert sum(p.rows for p in picks) == 267


def test_chunk_is_trimmed_to_the_room_riders_never():
    picks = plan_pass(worked_example(), 100, 16)
    assert names(picks)[0] == "P-A:89" and sum(p.rows for p in picks) == 100


def test_chunk_waits_when_the_leftover_is_too_small():
    picks = plan_pass(worked_example(), 20, 16)                 # 9 rows left < min_chunk
    assert all(p.kind == "rider" for p in picks) and sum(p.rows for p in picks) == 11


def test_small_chunk_runs_whole_and_nothing_stalls():
    assert names(plan_pass([Item("P", "chunk", 7, 0), Item("D", "rider", 1, 1)], 64, 16)) == ["P:7", "D:1"]
    # a run larger than the budget still goes, alone
    assert names(plan_pass([Item("V", "rider", 9, 0)], 4, 16)) == ["V:9"]
    assert names(plan_pass([Item("P", "chunk", 500, 0)], 64, 16)) == ["P:64"]
    assert plan_pass([], 64, 16) == []


def test_a_chunk_that_is_cut_anyway_is_cut_at_a_whole_number_of_tiles():
    riders = [Item(f"D{i}", "rider", 1, i) for i in range(32)]
    # 32 riders + 512 rows would be four tiles of 128 rows and 32 rows of a fifth: the portion gives 32 rows up
    picks = plan_pass(riders + [Item("P", "chunk", 512, 99, True)], 2048, 16, row_quantum=128)
    assert names(picks)[0] == "P:480" and sum(p.rows for p in picks) == 512
    # the last portion of a prompt is not cut (that would only add a step)
    picks = plan_pass(riders + [Item("P", "chunk", 512, 99, False)], 2048, 16, row_quantum=128)
    assert names(picks)[0] == "P:512"
    # ... unless the budget cuts it already
    picks = plan_pass(riders + [Item("P", "chunk", 512, 99, False)], 300, 16, row_quantum=128)
    assert names(picks)[0] == "P:224" and sum(p.rows for p in picks) == 256
    # a pass of less than a tile stays as it is, and so does one that is whole already
    assert names(plan_pass([Item("D", "rider", 1, 0), Item("P", "chunk", 100, 1, True)], 2048, 16, 128))[0] == "P:100"
    assert names(plan_pass(riders + [Item("P", "chunk", 96, 99, True)], 2048, 16, 128))[0] == "P:96"
    # never below the smallest portion
    assert names(plan_pass(riders[:2] + [Item("P", "chunk", 140, 99, True)], 2048, 16, 128))[0] == "P:126"
    run = [Item("V", "rider", 120, 0)]
    assert names(plan_pass(run + [Item("P", "chunk", 20, 99, True)], 2048, 16, 128))[0] == "P:20"
    assert names(plan_pass(run + [Item("P", "chunk", 20, 99, True)], 2048, 8, 128))[0] == "P:8"
    # no quantum, no cutting
    assert names(plan_pass(riders + [Item("P", "chunk", 512, 99, True)], 2048, 16))[0] == "P:512"


# ---- the scheduler over a real cache manager, with a fake model -------------------------------------------

def make(pages=64, page_size=4, budget=32, chunk=16, max_running=4, ctx=256, eos=(), row_quantum=0, fill_portions=False):
    """(`fill_portions` off: the reference's one prompt portion to a pass, which most of these tests pin.)"""
    cache = CacheManager([PagedKeysValues(1, 8)], page_size, pages, max_running)
    return Scheduler(cache, ctx, budget, chunk, min_chunk=4, max_running=max_running, eos_ids=eos,
                     row_quantum=row_quantum, fill_portions=fill_portions), cache


def drive(s, cache, token_of=lambda r: 7, limit=10000):
    """Runs the loop with a fake model; returns the list of steps as [(request id, start, rows, wants)]."""
    steps = []
    while s.has_work():
        plan = s.plan()
        if not plan:
            break
        steps.append([(p.request.id, p.start, len(p.tokens), p.wants_logits) for p in plan])
        s.complete(plan, [token_of(p.request) for p in plan if p.wants_logits])
        cache.check()
        assert len(steps) < limit
    return steps


def test_portions_beside_decoding_rows_fill_whole_tiles():
    s, cache = make(pages=200, budget=64, chunk=30, row_quantum=8)
    s.add(Request("a", [1, 2], SamplingParams.greedy_params(40)))
    for _ in range(3):                                                 # "a" is decoding now
        plan = s.plan()
        s.complete(plan, [7 for p in plan if p.wants_logits])
    s.add(Request("b", list(range(100)), SamplingParams.greedy_params(2)))
    steps = drive(s, cache)
    cut = [sum(rows for _, _, rows, _ in st) for st in steps if any(rid == "b" and rows > 1 for rid, _, rows, _ in st)]
    # every step that holds a portion of b's prompt (but its last) beside a's row has a multiple of 8 rows
    assert cut and all(n % 8 == 0 for n in cut[:-1]), cut
    assert s.finished["b"].finish_reason == "length" and len(s.finished["b"].output) == 2


def test_prompt_is_cut_into_portions_and_decoding_rides_along():
    s, cache = make()
    s.add(Request("a", list(range(40)), SamplingParams.greedy_params(3)))
    s.add(Request("b", list(range(5)), SamplingParams.greedy_params(6)))
    steps = drive(s, cache)
    assert steps[0] == [("a", 0, 16, False)]
    assert steps[1] == [("b", 0, 5, True)]                       # prompts alternate: a went to the back of the line
    assert steps[2] == [("a", 16, 16, False), ("b", 5, 1, True)]  # b decodes beside a's next portion
    assert steps[3] == [("a", 32, 8, True), ("b", 6, 1, True)]
    assert all(rows <= 32 for st in steps for rows in [sum(x[2] for x in st)])
    assert s.finished["a"].output == [7, 7, 7] and s.finished["a"].finish_reason == "length"
    assert len(s.finished["b"].output) == 6
    assert cache.free_pages() == [64] and not cache.requests


def test_a_pass_with_room_takes_the_next_prompts_portions_too():
    """Beyond the reference's rule: when the head of the prefill line got all it asked for, the prompts behind it are
    taken into the same pass while the budget lasts, the last one cut to the room (never below the smallest portion,
    and with a row quantum to a whole number of tiles); portions stay in front of the single rows."""
    s, cache = make(budget=32, chunk=16, fill_portions=True)
    s.add(Request("a", list(range(40)), SamplingParams.greedy_params(3)))
    s.add(Request("b", list(range(5)), SamplingParams.greedy_params(6)))
    s.add(Request("c", list(range(30)), SamplingParams.greedy_params(2)))
    steps = drive(s, cache)
    assert steps[0] == [("a", 0, 16, False), ("b", 0, 5, True), ("c", 0, 11, False)]      # 16 + 5 + 11 = the budget
    assert steps[1] == [("a", 16, 16, False), ("c", 11, 15, False), ("b", 5, 1, True)]     # c asked for 16: cut to the room
    assert all(sum(x[2] for x in st) <= 32 for st in steps)
    for st in steps:                                             # portions first, then the single rows of decoding requests
        kinds = [rows > 1 or not wants for _, _, rows, wants in st]
        assert kinds == sorted(kinds, reverse=True), st
    assert [len(s.finished[r].output) for r in "abc"] == [3, 6, 2] and cache.free_pages() == [64]
    # thirty short prompts that arrive together: a few passes, not thirty
    s, cache = make(pages=400, budget=64, chunk=16, max_running=30, fill_portions=True)
    for i in range(30):
        s.add(Request(f"p{i}", list(range(6)), SamplingParams.greedy_params(2)))
    steps = drive(s, cache)
    assert len(steps) <= 5 and sum(rows for _, _, rows, _ in steps[0]) == 64        # ten whole prompts and four rows of the next
    one, cache1 = make(pages=400, budget=64, chunk=16, max_running=30)
    for i in range(30):
        one.add(Request(f"p{i}", list(range(6)), SamplingParams.greedy_params(2)))
    assert len(drive(one, cache1)) >= 30
    # a head that the budget cut leaves no room: nothing is added; a portion that would fall below the smallest waits
    s, cache = make(budget=20, chunk=16, fill_portions=True)
    s.add(Request("a", list(range(16)), SamplingParams.greedy_params(2)))
    s.add(Request("b", list(range(30)), SamplingParams.greedy_params(2)))
    steps = drive(s, cache)
    assert steps[0] == [("a", 0, 16, True), ("b", 0, 4, False)]          # 4 rows: the smallest portion
    s, cache = make(budget=19, chunk=16, fill_portions=True)
    s.add(Request("a", list(range(16)), SamplingParams.greedy_params(2)))
    s.add(Request("b", list(range(30)), SamplingParams.greedy_params(2)))
    assert drive(s, cache)[0] == [("a", 0, 16, True)]                    # 3 rows of room: below it
    # with a row quantum the last portion is cut so that the pass is a whole number of tiles
    s, cache = make(pages=200, budget=64, chunk=30, row_quantum=8, fill_portions=True)
    s.add(Request("a", list(range(30)), SamplingParams.greedy_params(2)))
    s.add(Request("b", list(range(100)), SamplingParams.greedy_params(2)))
    assert drive(s, cache)[0] == [("a", 0, 30, True), ("b", 0, 26, False)]        # 30 + 30 would be 60: cut to 56


def test_stop_token_ends_without_being_emitted():
    s, cache = make(eos=(9,))
    seq = iter([4, 5, 9, 1, 1])
    s.add(Request("a", [1, 2, 3], SamplingParams.greedy_params(10)))
    drive(s, cache, token_of=lambda r: next(seq))
    assert s.finished["a"].output == [4, 5] and s.finished["a"].finish_reason == "stop"
    s.add(Request("b", [1, 2, 3], SamplingParams.greedy_params(4, ignore_eos=True)))
    drive(s, cache, token_of=lambda r: 9)
    assert s.finished["b"].output == [9, 9, 9, 9] and s.finished["b"].finish_reason == "length"


def test_context_limits():
    s, cache = make(ctx=16)
    with pytest.raises(ValueError, match="does not fit the context"):
        s.add(Request("big", list(range(16)), SamplingParams.greedy_params(4)))
    with pytest.raises(ValueError, match="empty"):
        s.add(Request("none", [], SamplingParams.greedy_params(4)))
    s.add(Request("a", list(range(12)), SamplingParams.greedy_params(100)))
    drive(s, cache)
    assert len(s.finished["a"].output) == 4 and s.finished["a"].finish_reason == "length"   # clamped to ctx - prompt


def test_max_running_and_first_come_first_served():
    s, cache = make(max_running=2)
    for i in range(4):
        s.add(Request(f"r{i}", [1, 2, 3], SamplingParams.greedy_params(2)))
    steps = drive(s, cache)
    first_seen = []
    for st in steps:
        for rid, *_ in st:
            if rid not in first_seen:
                first_seen.append(rid)
        assert len({rid for rid, *_ in st}) <= 2
    assert first_seen == ["r0", "r1", "r2", "r3"]


def test_preempts_the_newest_when_pages_run_out_and_recomputes():
    # 8 pages of 4 positions: two requests of 8 tokens both start (3 pages each with the token to come, and one to
    # spare), but with up to 12 new tokens each (5 pages in the end) they cannot both stay
    s, cache = make(pages=8, page_size=4, budget=32, chunk=16, max_running=2)
    s.add(Request("old", list(range(8)), SamplingParams.greedy_params(12)))
    s.add(Request("new", list(range(8)), SamplingParams.greedy_params(12)))
    steps = drive(s, cache)
    assert s.preemptions >= 1 and s.finished["new"].preemptions >= 1 and s.finished["old"].preemptions == 0
    assert len(s.finished["old"].output) == 12 and len(s.finished["new"].output) == 12
    # after its preemption `new` is prefilled again from position 0 with what it had generated so far
    restarts = [x for st in steps for x in st if x[0] == "new" and x[1] == 0]
    assert len(restarts) >= 2 and restarts[-1][2] > 8
    assert cache.free_pages() == [8]


def test_a_waiting_request_starts_when_all_it_has_fits_not_only_its_first_portion():
    # 10 pages of 4 positions. `a` (8 tokens, 20 more to come) runs; `b` has 28 tokens: 8 pages with the token to come,
    # beside the pages `a` still lacks for its own tokens and a page to spare for it: more than there are. Its first
    # portion (16 rows) would fit at once, and started on that it would be preempted when `a` has grown. It waits for
    # `a` to end instead; nothing is preempted.
    s, cache = make(pages=10, page_size=4, budget=32, chunk=16, max_running=2)
    s.add(Request("a", list(range(8)), SamplingParams.greedy_params(20)))
    s.add(Request("b", list(range(28)), SamplingParams.greedy_params(4)))
    steps = drive(s, cache)
    assert s.preemptions == 0
    last_a = max(i for i, st in enumerate(steps) if any(x[0] == "a" for x in st))
    first_b = min(i for i, st in enumerate(steps) if any(x[0] == "b" for x in st))
    assert first_b > last_a
    assert len(s.finished["a"].output) == 20 and len(s.finished["b"].output) == 4
    # with 23 tokens (6 pages, beside the 3 that `a` still lacks and the one to spare) it starts beside `a` at once
    s, cache = make(pages=10, page_size=4, budget=32, chunk=16, max_running=2)
    s.add(Request("a", list(range(8)), SamplingParams.greedy_params(4)))
    s.add(Request("b", list(range(23)), SamplingParams.greedy_params(1)))
    steps = drive(s, cache)
    assert any(x[0] == "b" for x in steps[1]) and s.preemptions == 0
    # alone in the pool a request starts on its first portion even if all of it will never fit (it ends when the pool does)
    s, cache = make(pages=4, page_size=4, budget=32, chunk=8, max_running=2)
    s.add(Request("long", list(range(15)), SamplingParams.greedy_params(9)))
    drive(s, cache)
    assert s.finished["long"].finish_reason == "kv_exhausted" and len(s.finished["long"].output) == 2


def test_a_preempted_request_does_not_come_back_into_the_room_it_gave_up():
    """Many growing requests in a pool that holds a third of them: a request that was preempted waits until all it has
    fits again, so preemptions stay few (started on its first portion alone it came back at once, was preempted again as
    soon as it had grown, and every time its prompt was computed anew)."""
    rng = random.Random(5)
    s, cache = make(pages=60, page_size=4, budget=48, chunk=32, max_running=12, ctx=256)
    want = {}
    for i in range(30):
        n, m = rng.randrange(8, 60), rng.randrange(10, 40)
        s.add(Request(f"r{i}", [rng.randrange(50) for _ in range(n)], SamplingParams.greedy_params(m)))
        want[f"r{i}"] = (n, m)
    steps = drive(s, cache, token_of=lambda r: len(r.output))
    assert set(s.finished) == set(want)
    for rid, (n, m) in want.items():
        assert s.finished[rid].output == list(range(m))
    computed = sum(rows for st in steps for _, _, rows, _ in st)
    needed = sum(n + m - 1 for n, m in want.values())
    print(f"preemptions {s.preemptions}, rows computed {computed} for {needed} needed")
    assert s.preemptions <= len(want) and computed <= 1.5 * needed
    assert cache.free_pages() == [60]


def test_request_that_can_never_fit_ends_with_kv_exhausted():
    s, cache = make(pages=2, page_size=4)
    s.add(Request("huge", list(range(20)), SamplingParams.greedy_params(4)))
    s.add(Request("ok", [1, 2], SamplingParams.greedy_params(2)))
    drive(s, cache)
    assert s.finished["huge"].finish_reason == "kv_exhausted" and s.finished["huge"].output == []
    assert s.finished["ok"].finish_reason == "length"
    s2, cache2 = make(pages=3, page_size=4)
    s2.add(Request("grows", list(range(10)), SamplingParams.greedy_params(50)))
    drive(s2, cache2)
    assert s2.finished["grows"].finish_reason == "kv_exhausted" and len(s2.finished["grows"].output) == 3
    assert cache2.free_pages() == [3]


@pytest.mark.parametrize("row_quantum", [0, 8])
@pytest.mark.parametrize("seed", range(4))
def test_random_load_always_finishes(seed, row_quantum):
    rng = random.Random(seed)
    s, cache = make(pages=24, page_size=4, budget=24, chunk=12, max_running=4, ctx=128, row_quantum=row_quantum)
    want = {}
    for i in range(12):
        n, m = rng.randrange(1, 40), rng.randrange(1, 20)
        s.add(Request(f"r{i}", [rng.randrange(50) for _ in range(n)], SamplingParams.greedy_params(m)))
        want[f"r{i}"] = m
    drive(s, cache, token_of=lambda r: len(r.output))
    assert set(s.finished) == set(want)
    for rid, m in want.items():
        assert s.finished[rid].output == list(range(m))              # preemption loses no token and repeats none
    assert cache.free_pages() == [24]


@pytest.mark.parametrize("ahead", [False, True])
@pytest.mark.parametrize("seed", range(6))
def test_random_arrivals_and_cancels_keep_the_books(seed, ahead):
    """Requests arrive while others run, some are cancelled where they stand (waiting, in the middle of their prompt,
    decoding, with a row in a step that is in flight), the pool is tight; with and without planning a step ahead. After
    every step the cache's books are in order; at the end every request has ended once, the cancelled ones with a
    beginning of what they would have produced, the others with all of it, and every page is back."""
    rng = random.Random(100 + seed)
    s, cache = make(pages=20, page_size=4, budget=24, chunk=12, max_running=4, ctx=128, fill_portions=seed % 2 == 0)
    plans = [(rng.randrange(1, 40), rng.randrange(1, 20)) for _ in range(30)]
    pending, cancelled, inflight, steps = list(range(30)), set(), None, 0

    def complete(plan):
        # the fake model's token is the request's output length at the time its row is read
        s.complete(plan, [len(p.request.output) for p in plan if p.wants_logits])

    while pending or s.has_work() or inflight is not None:
        for _ in range(min(len(pending), rng.randrange(0, 3))):
            i = pending.pop(0)
            s.add(Request(f"r{i}", [rng.randrange(50) for _ in range(plans[i][0])], SamplingParams.greedy_params(plans[i][1])))
        live = [r.id for r in s.running + s.waiting]
        if live and rng.random() < 0.15:
            rid = rng.choice(live)
            assert s.cancel(rid).finish_reason == "cancelled"
            cancelled.add(rid)
        plan = None
        if inflight is not None and ahead:
            plan = s.plan(inflight=inflight)
        if plan is None:
            if inflight is not None:
                complete(inflight)
                inflight = None
            plan = s.plan()
        s.take_ended()
        if inflight is not None:
            complete(inflight)
        inflight = plan or None
        if not ahead and inflight is not None:
            complete(inflight)
            inflight = None
        cache.check()
        steps += 1
        assert steps < 5000
    assert set(s.finished) == {f"r{i}" for i in range(30)} and cancelled
    for i, (_, m) in enumerate(plans):
        r = s.finished[f"r{i}"]
        if r.id in cancelled:
            assert r.finish_reason == "cancelled" and r.output == list(range(len(r.output))) and len(r.output) <= m
        else:
            assert r.finish_reason == "length" and r.output == list(range(m))
    assert cache.free_pages() == [20] and not cache.requests


# ---- settings and command line ------------------------------------------------------------------------------

def test_settings_layers_aliases_and_errors(tmp_path):
    f = tmp_path / "my.properties"
    f.write_text("# comment\nsampling.top-k = 5\nbackend.ctx=300\n")
    s = Settings.load(["--config", str(f), "--temp", "0", "--sampling.top-p=0.5", "--ignore-eos"]).validate()
    assert s.get("sampling.top-k") == "5" and s.sources["sampling.top-k"] == str(f)
    assert s.sampling().temperature == 0 and s.sampling().top_p == 0.5 and s.sampling().ignore_eos
    assert s.sources["sampling.temperature"] == "flag" and s.sources["backend.batch"] == "default"
    assert "backend.ctx = 300" in s.describe()
    with pytest.raises(SettingsError, match="unknown option --nope"):
        Settings.load(["--nope", "1"])
    with pytest.raises(SettingsError, match="top_p"):
        Settings.load(["--top-p", "0"]).validate()
    f.write_text("sampling.topk=5\n")
    with pytest.raises(SettingsError, match="unknown setting"):
        Settings.load(["--config", str(f)])
    assert main(["run", "--nope"]) == 2 and main(["frobnicate"]) == 2 and main(["config"]) == 0


def test_sampling_params_validation():
    for bad in (dict(temperature=-0.1), dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5), dict(min_p=2.0),
                dict(temperature=float("nan")), dict(max_tokens=0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    d = SamplingParams()
    assert (d.temperature, d.top_k, d.top_p, d.min_p, d.seed, d.max_tokens) == (0.6, 20, 0.95, 0.0, -1, 1024)
    assert SamplingParams(temperature=0).greedy and SamplingParams(top_k=1).greedy and not d.greedy


def test_requests_the_planner_ends_itself_are_handed_to_the_caller():
    """A request that can never fit the pool ends inside `plan` with `kv_exhausted`; `take_ended` hands it over once,
    so whoever drives the steps by hand learns of it although it never reaches `complete`."""
    from jllm_serve_b200.cache import CacheManager, PagedKeysValues
    from jllm_serve_b200.engine.scheduler import Request, Scheduler
    from jllm_serve_b200.sampling.params import SamplingParams
    cache = CacheManager([PagedKeysValues(1, 8)], page_size=4, num_pages=3, max_requests=2)      # room for 12 tokens
    s = Scheduler(cache, ctx=64, max_batch_tokens=32, chunk=32, min_chunk=1, max_running=2)
    s.add(Request("big", list(range(1, 31)), SamplingParams.greedy_params(4)))
    s.add(Request("small", [1, 2, 3], SamplingParams.greedy_params(2)))
    plan = s.plan()
    ended = s.take_ended()
    assert [r.id for r in ended] == ["big"] and ended[0].finish_reason == "kv_exhausted"
    assert s.take_ended() == []                                    # handed over once
    assert [p.request.id for p in plan] == ["small"]               # the next request in line runs in the same step


def drive_ahead(scheduler, token_of, ahead: bool, max_steps=500):
    """Runs the scheduler against a fake model (`token_of(request, position)` is what a step samples for the token
    that follows `position`), either completing every step before the next is planned or planning one step ahead.
    Returns {request id: (output, finish reason)} and the steps as lists of (id, start, tokens, wants)."""
    steps, inflight = [], None

    def result_of(plan):
        return [token_of(p.request, p.start + len(p.tokens) - 1) for p in plan if p.wants_logits]

    for _ in range(max_steps):
        if not scheduler.has_work() and inflight is None:
            break
        plan = None
        if inflight is not None and ahead:
            plan = scheduler.plan(inflight=inflight)
        if plan is None:
            if inflight is not None:
                scheduler.complete(inflight, result_of(inflight))
                inflight = None
            plan = scheduler.plan()
        scheduler.take_ended()
        if plan:
            steps.append([(p.request.id, p.start, list(p.tokens), p.wants_logits) for p in plan])
        if inflight is not None:
            scheduler.complete(inflight, result_of(inflight))
        inflight = plan or None
        if not ahead and inflight is not None:
            scheduler.complete(inflight, result_of(inflight))
            inflight = None
    return {rid: (r.output, r.finish_reason) for rid, r in scheduler.finished.items()}, steps


def test_planning_one_step_ahead_gives_the_same_outputs():
    """With a step planned while the one before is unread: the next token of a decoding request is a marker for "row j
    of the step before's samples", a request that ends by length is not planned again, one that ends by a stop token
    has had one row too many (wasted), and all outputs and reasons are those of the step-by-step order; a pool that
    is short makes the planner wait for the step in flight (None) instead of preempting blindly."""
    def token_of(r, position):       # a fake model: the token after `position` of request r
        return (7 * position + 3 * len(r.prompt)) % 50

    def make(pages):
        cache = CacheManager([PagedKeysValues(1, 8)], page_size=4, num_pages=pages, max_requests=4)
        s = Scheduler(cache, ctx=64, max_batch_tokens=24, chunk=16, min_chunk=2, max_running=3, eos_ids=[11, 17])
        for i, (n, new) in enumerate([(5, 12), (30, 6), (9, 40), (3, 1), (14, 9)]):
            s.add(Request(f"q{i}", [(i + t) % 50 for t in range(n)], SamplingParams.greedy_params(new)))
        return s, cache

    for pages in (64, 11):           # roomy, and so tight that a request is preempted and recomputed
        a, _ = make(pages)
        want, sync_steps = drive_ahead(a, token_of, ahead=False)
        b, cache = make(pages)
        got, ahead_steps = drive_ahead(b, token_of, ahead=True)
        assert got == want and set(want) == {f"q{i}" for i in range(5)}
        assert any(reason == "stop" for _, reason in want.values()) and any(reason == "length" for _, reason in want.values())
        markers = [t for st in ahead_steps for _, _, toks, _ in st for t in toks if t < 0]
        assert markers and not [t for st in sync_steps for _, _, toks, _ in st for t in toks if t < 0]
        # a marker names a row of the step before: the j-th of its segments that wanted logits
        for before, st in zip(ahead_steps, ahead_steps[1:]):
            wanting = [rid for rid, _, _, wants in before if wants]
            for rid, start, toks, _ in st:
                if toks[0] < 0:
                    assert len(toks) == 1 and wanting[-toks[0] - 1] == rid
        assert not cache.requests and cache.free_pages() == [pages]
        cache.check()
        if pages == 11:
            assert a.preemptions > 0 and b.preemptions > 0


def test_cancel_ends_a_waiting_or_running_request_and_frees_its_pages():
    """`cancel` ends a request where it stands: one that waits never starts; one that runs gives its pages back at
    once and keeps what it had generated; a row of it in a step that is still in flight is passed over when the step
    completes, and the others in that step are untouched. A second cancel, or one of an unknown request, is None."""
    s, cache = make(pages=16, max_running=2)
    for name, n in (("a", 6), ("b", 5), ("c", 7)):
        s.add(Request(name, list(range(1, n + 1)), SamplingParams.greedy_params(8)))
    for _ in range(4):                                                  # a and b decode; c waits (two may run)
        plan = s.plan()
        s.complete(plan, [7 for p in plan if p.wants_logits])
    assert {r.id for r in s.running} == {"a", "b"} and [r.id for r in s.waiting] == ["c"]
    assert s.cancel("c").finish_reason == "cancelled" and not s.waiting and s.finished["c"].output == []
    held = cache.free_pages()[0]
    inflight = s.plan()                                                 # a step with a row of a and a row of b ...
    assert sorted(p.request.id for p in inflight) == ["a", "b"]
    had = list(next(r for r in s.running if r.id == "a").output)
    gone = s.cancel("a")                                                # ... and a is cancelled before it is read
    assert gone.finish_reason == "cancelled" and gone.output == had and len(had) >= 1
    assert cache.free_pages()[0] > held and not cache.is_open("a")
    cache.check()
    after = s.plan(inflight=inflight)                                   # planned ahead: b alone, a's row is gone
    assert [p.request.id for p in after] == ["b"]
    b_before = len(next(r for r in s.running if r.id == "b").output)
    done = s.complete(inflight, [9, 9])
    assert done == [] and gone.output == had                            # a's token of that step is dropped
    assert len(next(r for r in s.running if r.id == "b").output) == b_before + 1
    assert s.cancel("a") is None and s.cancel("nobody") is None
    s.complete(after, [7])
    drive(s, cache)
    assert s.finished["b"].finish_reason == "length" and len(s.finished["b"].output) == 8
    assert cache.free_pages() == [16] and not cache.requests


def test_a_request_name_is_taken_until_its_result_is():
    s, cache = make()
    s.add(Request("a", [1, 2, 3], SamplingParams.greedy_params(2)))
    with pytest.raises(ValueError, match="already"):
        s.add(Request("a", [4, 5], SamplingParams.greedy_params(2)))
    drive(s, cache)
    with pytest.raises(ValueError, match="result not taken"):
        s.add(Request("a", [4, 5], SamplingParams.greedy_params(2)))
    s.finished.pop("a")
    s.add(Request("a", [4, 5], SamplingParams.greedy_params(2)))
    drive(s, cache)
    assert len(s.finished["a"].output) == 2
