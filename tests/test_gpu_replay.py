"""The engine against the plain implementation under every way of cutting the work (GPU)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import traces
from tests.helpers import compare_with_plain, model_folder, replay, requests_for
from tests.tiny import CONFIGS

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"A": (5, 17, 33, 70), "B": (1, 7, 64, 129), "C": (3, 50, 97, 130), "D": (2, 65, 150, 260),
           "E": (4, 129, 300, 470)}         # E: portions of more than 128 and of more than 256 rows in one step
PAGE = {"A": 4, "B": 8, "C": 16, "D": 16, "E": 16}


def make_runner(name, dtype, steps=None, **kw):
    from jllm_serve_b200.engine import ModelRunner
    page = kw.pop("page_size", PAGE[name])
    tokens = traces.peak_tokens(steps, 64) if steps is not None else 1024
    return ModelRunner(model_folder(name), dtype=dtype, page_size=page, num_pages=-(-tokens // page),
                       max_batch_tokens=kw.pop("max_batch_tokens", 512), max_requests=8, ctx=512,
                       poison_freed_pages=True, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_requests(name, dtype):
    reqs = requests_for(name, LENGTHS[name])
    steps = traces.whole(reqs)
    got = replay(make_runner(name, dtype, steps), steps)
    compare_with_plain(got, model_folder(name), reqs, dtype, what=f"{name} whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_last_32_tokens_one_by_one(name, dtype):
    reqs = requests_for(name, LENGTHS[name])
    steps = traces.prompt_then_decode(reqs, 32)
    got = replay(make_runner(name, dtype, steps), steps)
    compare_with_plain(got, model_folder(name), reqs, dtype, what=f"{name} decode tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_portions_of_changing_size(name, dtype):
    reqs = requests_for(name, LENGTHS[name])
    steps = traces.changing_portions(reqs)
    got = replay(make_runner(name, dtype, steps), steps)
    compare_with_plain(got, model_folder(name), reqs, dtype, what=f"{name} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_mixed_batches_with_pages_used_again(name, dtype):
    reqs = requests_for(name, LENGTHS[name] + (41, 90, 12), seed=23)
    steps = traces.mixed(reqs, max_live=4)
    runner = make_runner(name, dtype, steps)
    got = replay(runner, steps)
    compare_with_plain(got, model_folder(name), reqs, dtype, what=f"{name} mixed")
    assert all(g.pool.reuses > 0 for g in runner.cache.paged), "the pool was so large that no page was used again"
    assert all(g.pool.num_free == g.pool.num_pages for g in runner.cache.paged), "pages were not all given back"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_hundred_requests_decode_side_by_side(dtype):
    """More (row, kv head) pairs in a decode step than the SMs have places for blocks: in bfloat16 the attention
    deals the key tiles of all pairs out evenly over the blocks."""
    from jllm_serve_b200.engine import ModelRunner
    lengths = tuple(6 + (7 * i) % 23 for i in range(104))
    reqs = requests_for("D", lengths, seed=5)
    steps = traces.all_together(reqs, tail=4)
    runner = ModelRunner(model_folder("D"), dtype=dtype, page_size=16, num_pages=260, max_batch_tokens=2048,
                         max_requests=104, ctx=64, poison_freed_pages=True)
    got = replay(runner, steps)
    compare_with_plain(got, model_folder("D"), reqs, dtype, what="D a hundred side by side")
    from jllm_serve_b200.csrc import ops
    scratch = torch.empty(2 << 20, device="cuda:0")
    assert ops.decode_plan(104, 3, 1, 6, 64, scratch)[0] == "flat"      # 312 pairs for 296 places


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_cuts_agree_bit_for_bit(name):
    """In float32 every row's arithmetic is independent of the batch it rides in, so all ways of cutting
    give the same bits on one device."""
    reqs = requests_for(name, LENGTHS[name])
    base = replay(make_runner(name, "float32"), traces.whole(reqs))
    for cut in (traces.prompt_then_decode(reqs), traces.changing_portions(reqs), traces.mixed(reqs)):
        got = replay(make_runner(name, "float32"), cut)
        for key, row in base.items():
            assert torch.equal(row, got[key]), f"{name}: row {key} differs between cuts"


def test_captured_decode_steps_are_evicted_and_captured_again():
    """More decode shapes than the runner keeps graphs for: the oldest capture makes room, and a shape that comes back
    is captured anew; every step's logits are right whether it ran launch by launch, was captured, or replayed."""
    reqs = requests_for("B", (40, 40, 40), seed=9)
    ids = list(reqs)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": reqs[r][:10], "want": list(range(10))} for r in ids], "end": []}]
    at = {r: 10 for r in ids}
    for group in ([ids[0]], ids[:2], ids, [ids[0]], ids[1:], ids[:2], ids):
        for _ in range(4):
            steps.append({"step": len(steps), "entries": [{"id": r, "tokens": reqs[r][at[r]:at[r] + 1], "want": [0]}
                                                           for r in group], "end": []})
            for r in group:
                at[r] += 1
    steps.append({"step": len(steps), "entries": [{"id": r, "tokens": reqs[r][at[r]:], "want": list(range(40 - at[r]))}
                                                   for r in ids], "end": ids})
    runner = make_runner("B", "bfloat16", steps)
    runner.max_graphs = 2
    got = replay(runner, steps)
    compare_with_plain(got, model_folder("B"), reqs, "bfloat16", what="B graphs evicted")
    assert len(runner._graphs) == 2 and len(runner._graph_seen) == 3     # three shapes were met, two are kept


def test_long_decoding():
    """300 tokens one by one after a short prompt: every page edge and the window's edge are crossed."""
    for name, dtype in (("B", "float32"), ("C", "float32"), ("C", "bfloat16")):
        reqs = requests_for(name, (330,), seed=5)
        steps = traces.prompt_then_decode(reqs, 300)
        got = replay(make_runner(name, dtype, steps), steps)
        compare_with_plain(got, model_folder(name), reqs, dtype, what=f"{name} long decode")


def test_first_tokens_of_a_sequence():
    for name in ("A", "B", "C"):
        for dtype in ("float32", "bfloat16"):
            reqs = requests_for(name, (1, 2, 3), seed=31)
            steps = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}
                                             for r, t in reqs.items()], "end": list(reqs)}]
            got = replay(make_runner(name, dtype, steps), steps)
            compare_with_plain(got, model_folder(name), reqs, dtype, what=f"{name} first tokens")


@pytest.mark.parametrize("name, dtype, lengths, rows", [("B", "float32", (129, 64), 50), ("E", "bfloat16", (300, 170), 130),
                                                        ("C", "bfloat16", (130, 97), 48)])
def test_step_larger_than_a_batch_is_split(name, dtype, lengths, rows):
    """A step of more rows than a batch holds runs as several batches (also over a windowed group, which gives pages
    back between the parts); the logits come back in the order that was asked for."""
    from jllm_serve_b200.engine import Segment
    from tests.helpers import RowChecker
    reqs = requests_for(name, lengths, seed=3)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))[::-1]}
                                     for r, t in reqs.items()], "end": list(reqs)}]
    runner = make_runner(name, dtype, steps, max_batch_tokens=rows)
    got = runner.step([Segment(e["id"], e["tokens"], 0, e["want"]) for e in steps[0]["entries"]]).float().cpu()
    checker = RowChecker(model_folder(name), reqs, dtype, what=f"{name} step in parts")
    r = 0
    for rid, toks in reqs.items():
        for p in reversed(range(len(toks))):
            checker.row(rid, p, got[r])
            r += 1
    checker.finish()
    assert runner.steps >= 3
    for rid in reqs:
        runner.finish(rid)
    runner.cache.check()


def test_step_in_parts_takes_all_its_pages_or_none():
    """The pages of every part are reserved before the first part runs: a pool that cannot hold the step refuses it
    with nothing run, nothing committed and nothing held."""
    from jllm_serve_b200.cache import PoolExhausted
    from jllm_serve_b200.engine import ModelRunner, Segment
    reqs = requests_for("B", (129, 64), seed=3)
    runner = ModelRunner(model_folder("B"), dtype="float32", page_size=8, num_pages=20, max_batch_tokens=50, max_requests=4,
                         ctx=512)                               # 20 pages hold 160 tokens; the step brings 193
    with pytest.raises(PoolExhausted):
        runner.step([Segment(r, t, 0, [len(t) - 1]) for r, t in reqs.items()])
    assert runner.steps == 0 and not runner.cache.requests and runner.cache.free_pages() == [20]
    runner.cache.check()
    small = {"r0": reqs["r0"]}                                 # what fits still runs afterwards
    got = replay(runner, traces.whole(small))
    compare_with_plain(got, model_folder("B"), small, "float32", what="after a refused step")


def test_a_step_that_fails_while_running_gives_its_pages_back(monkeypatch):
    """If the forward pass raises, the pages reserved for the step go back and requests opened for it are closed, so
    the cache's books still say what the caller believes."""
    from jllm_serve_b200.engine import ModelRunner, Segment
    reqs = requests_for("A", (20, 9), seed=3)
    runner = ModelRunner(model_folder("A"), dtype="float32", page_size=4, num_pages=30, max_batch_tokens=64, max_requests=4,
                         ctx=128)
    runner.step([Segment("r0", reqs["r0"][:8], 0, [])])
    free = runner.cache.free_pages()

    def broken(batch, cache, logits_out=None):
        raise RuntimeError("a kernel failed")

    monkeypatch.setattr(runner.model, "forward", broken)
    with pytest.raises(RuntimeError, match="a kernel failed"):
        runner.step([Segment("r0", reqs["r0"][8:], 8, [11]), Segment("r1", reqs["r1"], 0, [8])])
    assert runner.cache.length("r0") == 8 and not runner.cache.is_open("r1") and runner.cache.free_pages() == free
    runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tmp_path):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files and `done` lines out."""
    name = "B"
    reqs = requests_for(name, (40, 70, 9, 33, 64), seed=17)
    steps = traces.mixed(reqs, max_live=4, portion=20)
    out = tmp_path / "logits"
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_folder(name)),
                           "--dtype", dtype, "--out", str(out), "--max-tokens", str(traces.peak_tokens(steps, 64)),
                           "--poison"], input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = CONFIGS[name]["vocab_size"]

    def rows(st):
        n = sum(len(e["want"]) for e in st["entries"])
        if n == 0:
            assert not (out / f"{st['step']}.f32").exists()
            return None
        a = np.fromfile(out / f"{st['step']}.f32", dtype="<f4")
        assert a.size == n * vocab
        return torch.from_numpy(a.reshape(n, vocab).copy())

    got = traces.collect(steps, rows)
    compare_with_plain(got, model_folder(name), reqs, dtype, what="trace_run")
