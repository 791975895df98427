"""Steps of the scheduler's own form at the sizes of the product kernels' tiles, against the plain logits (GPU).

The scheduler puts the one prompt portion of a step first and the decoding requests' single rows behind it;
the attention then runs the portion through the flash kernel and the single rows through the decode kernel, and
the products see more rows than one 128-row tile. The reference checks the same thing with its scripts of
mixed passes (src/test/java/org/robomiri/jllm/MixedPassChecks.java:166-252, MixedSchedulerTest.java:49-60).
Here: traces of that form (portions of 129 to 512 rows beside 1 to 19 single rows, a pool so small that pages
are used again, freed pages filled with NaN), and the very steps `Scheduler.plan` forms inside
`Engine.generate`, recorded and replayed with the logits of every row asked for.
"""
import pytest
import torch

from tests import traces
from tests.helpers import RowChecker, model_folder, replay_checked
from tests.tiny import CONFIGS, random_tokens

pytestmark = pytest.mark.gpu


def runner_for(name, dtype, steps, max_requests, ctx=1024, rows=576):
    from jllm_serve_b200.engine import ModelRunner
    page = 16
    return ModelRunner(model_folder(name), dtype=dtype, page_size=page, num_pages=traces.peak_tokens(steps, 64) // page,
                       max_batch_tokens=rows, max_requests=max_requests, ctx=ctx, poison_freed_pages=True)


def count_scheduler_shaped(runner_steps):
    """Steps whose batch had a leading portion of more than 128 rows and single rows behind it."""
    return sum(1 for ms, mr, rows in runner_steps if ms > 0 and mr > 128 and rows > mr)


def run_trace(name, dtype, requests, steps, max_requests):
    runner = runner_for(name, dtype, steps, max_requests)
    seen = []
    step = runner.step

    def watched(segments, logits_out=None):
        out = step(segments, logits_out)
        b = runner.last_batch
        seen.append((b.multi_segments, b.multi_rows, b.rows))
        return out

    runner.step = watched
    checker = RowChecker(model_folder(name), requests, dtype, what=f"{name} scheduled")
    replay_checked(runner, steps, checker)
    checker.finish()
    assert all(g.pool.reuses > 0 for g in runner.cache.paged), "the pool was so large that no page was used again"
    assert all(g.pool.num_free == g.pool.num_pages for g in runner.cache.paged), "pages were not all given back"
    return seen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_portion_first_then_decoding_rows_four_live(name, dtype):
    lengths = (330, 520, 700, 450, 640, 380, 560, 410, 300)
    vocab = CONFIGS[name]["vocab_size"]
    requests = {f"r{i}": random_tokens(n, vocab, 40 + i) for i, n in enumerate(lengths)}
    prompts = {f"r{i}": n - (40 + 15 * (i % 4)) for i, n in enumerate(lengths)}
    steps = traces.scheduled(requests, prompts, max_live=4, portions=(300, 129, 260, 200, 385, 140))
    assert all(s is not None for s in traces.shape_of(steps))
    seen = run_trace(name, dtype, requests, steps, max_requests=4)
    assert count_scheduler_shaped(seen) >= 10, seen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_portion_first_then_many_decoding_rows(name, dtype):
    """Sixteen short requests decode while four long prompts come in portions of up to 512 rows."""
    lengths = (100,) * 16 + (640, 520, 900, 450)
    vocab = CONFIGS[name]["vocab_size"]
    requests = {f"r{i}": random_tokens(n + i % 5, vocab, 70 + i) for i, n in enumerate(lengths)}
    prompts = {f"r{i}": (40 + i if n == 100 else n - 20) for i, n in enumerate(lengths)}
    steps = traces.scheduled(requests, prompts, max_live=20, portions=(257, 140, 512, 129, 363, 200))
    seen = run_trace(name, dtype, requests, steps, max_requests=20)
    assert count_scheduler_shaped(seen) >= 10, seen
    assert max(rows - mr for ms, mr, rows in seen if mr > 128) >= 16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "E"])
def test_the_steps_generate_forms_replayed_with_every_row_wanted(name, dtype):
    """`Engine.generate` under a budget of 300 rows and portions of 260, with a pool that forces preemption: the
    steps the scheduler formed are recorded (segments and the requests it closed), then replayed through a fresh
    runner asking for the logits of every row, which are compared with the plain logits of prompt + output."""
    from jllm_serve_b200.engine import Engine, ModelRunner, Segment
    from jllm_serve_b200.sampling import SamplingParams
    vocab = CONFIGS[name]["vocab_size"]
    lengths = (300, 150, 420, 280, 510, 200, 345, 180, 390, 260, 470, 330)
    prompts = [random_tokens(n, vocab, 90 + i) for i, n in enumerate(lengths)]
    engine = Engine(model_folder(name), dtype=dtype, page_size=16, max_tokens_cached=1280, max_batch_tokens=300,
                    chunk=260, min_chunk=16, max_running=6, ctx=1024)
    log = []
    step, close = engine.runner.step, engine.runner.cache.close

    def watched_step(segments, logits_out=None, **kw):
        log.append(("step", [[s.request, list(s.tokens), s.start] for s in segments]))
        return step(segments, logits_out, **kw)

    def watched_close(request):
        log.append(("end", request))
        return close(request)

    engine.runner.step, engine.runner.cache.close = watched_step, watched_close
    ids = [engine.add_request(p, SamplingParams.greedy_params(40 + 8 * (i % 3), ignore_eos=True))
           for i, p in enumerate(prompts)]
    engine.run_until_done()
    results = [engine.result_of(i) for i in ids]
    assert engine.scheduler.preemptions > 0, "the pool was large enough: no request was preempted"
    sequences = {rid: p + r.tokens for rid, p, r in zip(ids, prompts, results)}
    del engine

    runner = ModelRunner(model_folder(name), dtype=dtype, page_size=16, num_pages=96, max_batch_tokens=300,
                         max_requests=6, ctx=1024, poison_freed_pages=True)
    checker = RowChecker(model_folder(name), sequences, dtype, what=f"{name} generate's steps")
    shaped = several = 0
    for kind, what in log:
        if kind == "end":
            runner.finish(what)
            continue
        # a token that went from one step into the next on the device (a marker in the plan) is known by now; a row
        # that was planned ahead for a request whose token before it turned out to be its last is left out
        what = [[rid, [sequences[rid][start + k] if t < 0 else t for k, t in enumerate(toks)], start]
                for rid, toks, start in what if start + len(toks) <= len(sequences[rid])]
        if not what:
            continue
        segs = [Segment(rid, toks, start, list(range(len(toks)))) for rid, toks, start in what]
        rows = runner.step(segs).float().cpu()
        b = runner.last_batch
        shaped += b.multi_segments > 0 and b.multi_rows > 128 and b.rows > b.multi_rows
        several += b.multi_segments > 1          # a step with room took a second prompt's portion too
        r = 0
        for rid, toks, start in what:
            for k in range(len(toks)):
                checker.row(rid, start + k, rows[r])
                r += 1
    runner.cache.check()
    # the last token of an output is never fed, so its position has no row
    for rid, toks in sequences.items():
        checker.seen.add((rid, len(toks) - 1))
    checker.finish()
    assert shaped >= 10, f"only {shaped} steps had a portion of more than 128 rows before single rows"
    assert several >= 3, f"only {several} steps held portions of more than one prompt"
