"""Generation through the public entry point and the command line (GPU)."""
import json
import random
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests.helpers import TOL, model_folder, plain_logits
from tests.plain import qwen3_plain as P
from tests.tiny import CONFIGS, make_model_folder, random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def engine_for(name, dtype, **kw):
    from jllm_serve_b200.engine import Engine
    args = dict(dtype=dtype, page_size=8, max_tokens_cached=2048, max_batch_tokens=64, chunk=32, min_chunk=4,
                max_running=4, ctx=512)
    args.update(kw)
    return Engine(model_folder(name), **args)


def prompts_for(name, lengths, seed=3):
    return [random_tokens(n, CONFIGS[name]["vocab_size"], seed + i) for i, n in enumerate(lengths)]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_float32_equals_plain(name):
    from jllm_serve_b200.sampling import SamplingParams
    cfg, w = P.load_plain(model_folder(name))
    prompts = prompts_for(name, (5, 17, 33))
    got = engine_for(name, "float32").generate(prompts, SamplingParams.greedy_params(16, ignore_eos=True))
    for p, r in zip(prompts, got):
        assert r.tokens == P.greedy_generate(cfg, w, p, 16) and r.finish_reason == "length"
        assert r.stats.prompt_tokens == len(p) and r.stats.generated == 16


@pytest.mark.parametrize("name", ["B", "D"])
def test_greedy_generation_bfloat16_follows_plain(name):
    """Every token the bfloat16 engine picks is (within bfloat16's tolerance) a best token of the plain float32
    logits for the same prefix; the prefix is the engine's own, so one near-tie cannot derail the comparison."""
    from jllm_serve_b200.sampling import SamplingParams
    prompts = prompts_for(name, (9, 40, 70))
    got = engine_for(name, "bfloat16").generate(prompts, SamplingParams.greedy_params(12, ignore_eos=True))
    for p, r in zip(prompts, got):
        assert len(r.tokens) == 12
        logits = plain_logits(model_folder(name), tuple(p + r.tokens[:-1]))
        for i, t in enumerate(r.tokens):
            row = logits[len(p) - 1 + i]
            assert float(row.max() - row[t]) <= TOL["bfloat16"] * float(logits.abs().max()), (i, t)


def test_scheduled_together_equals_alone_with_preemption():
    """Six requests through portions of 32 under a budget of 48 rows and a pool so small that the scheduler must
    preempt and recompute: the tokens are those of each request generated alone."""
    from jllm_serve_b200.sampling import SamplingParams
    name = "B"
    prompts = prompts_for(name, (70, 1, 33, 64, 129, 20), seed=9)
    params = SamplingParams.greedy_params(24, ignore_eos=True)
    alone = [engine_for(name, "float32").generate([p], params)[0].tokens for p in prompts[:3]]
    tight = engine_for(name, "float32", max_tokens_cached=224, max_batch_tokens=48)
    got = tight.generate(prompts, params)
    cfg, w = P.load_plain(model_folder(name))
    for i, (p, r) in enumerate(zip(prompts, got)):
        want = alone[i] if i < 3 else P.greedy_generate(cfg, w, p, 24)
        assert r.tokens == want, f"request {i}"
    assert tight.scheduler.preemptions > 0, "the pool was large enough: the test did not exercise preemption"
    assert tight.runner.cache.free_pages() == [28] and not tight.runner.cache.requests


def test_temperature_sampling_is_seeded_and_matches_the_plain_walk():
    from jllm_serve_b200.sampling import SamplingParams
    name = "B"
    prompts = prompts_for(name, (1, 7, 64, 129), seed=21)
    params = [SamplingParams(temperature=0.8, top_k=0, top_p=1.0, seed=100 + i, max_tokens=24, ignore_eos=True)
              for i in range(4)]
    together = engine_for(name, "float32").generate(prompts, params)
    again = engine_for(name, "float32", chunk=16, max_batch_tokens=40).generate(prompts[::-1], params[::-1])[::-1]
    for a, b in zip(together, again):
        assert a.tokens == b.tokens                      # the seed decides, not the batch or the cut
    # the plain walk with the same uniform numbers
    for p, sp, r in zip(prompts, params, together):
        rng, toks = random.Random(sp.seed), list(p)
        for t in r.tokens:
            logits = plain_logits(model_folder(name), tuple(toks))[-1]
            idx, w = P.sampling_weights(logits, sp.temperature, sp.top_k, sp.top_p, sp.min_p)
            assert t == P.draw(idx, w, rng.random())
            toks.append(t)
    other = engine_for(name, "float32").generate(prompts[2:3], SamplingParams(temperature=0.8, top_k=20, top_p=0.9,
                                                                              seed=5, max_tokens=24, ignore_eos=True))
    assert other[0].tokens != together[2].tokens


def test_stop_token_and_context_limit(tmp_path):
    from jllm_serve_b200.engine import Engine
    from jllm_serve_b200.sampling import SamplingParams
    base = CONFIGS["A"]
    prompt = random_tokens(11, base["vocab_size"], 77)
    free = Engine(make_model_folder(base, 7, tmp_path / "free"), dtype="float32", ctx=64, max_batch_tokens=32, chunk=16,
                  max_running=2, page_size=4, max_tokens_cached=256)
    tokens = free.generate([prompt], SamplingParams.greedy_params(10))[0].tokens
    stop_at = tokens[4]
    first = tokens.index(stop_at)
    stopping = Engine(make_model_folder(dict(base, eos_token_id=[stop_at, 255]), 7, tmp_path / "stop"), dtype="float32",
                      ctx=64, max_batch_tokens=32, chunk=16, max_running=2, page_size=4, max_tokens_cached=256)
    r = stopping.generate([prompt], SamplingParams.greedy_params(10))[0]
    assert r.finish_reason == "stop" and r.tokens == tokens[:first]          # the stop token is not emitted
    r = stopping.generate([prompt], SamplingParams.greedy_params(10, ignore_eos=True))[0]
    assert r.finish_reason == "length" and r.tokens == tokens
    r = free.generate([prompt], SamplingParams.greedy_params(1000))[0]
    assert r.finish_reason == "length" and len(r.tokens) == 64 - 11            # clamped to the context
    with pytest.raises(ValueError, match="does not fit the context"):
        free.generate([list(range(64))], SamplingParams.greedy_params(4))
    with pytest.raises(ValueError, match="token id outside"):
        free.generate([[1, 2, 256]], SamplingParams.greedy_params(4))


def test_command_line_run_and_bench(tmp_path):
    folder = model_folder("A")
    prompt = random_tokens(9, 256, 5)
    cmd = [sys.executable, str(ROOT / "bin" / "jllm"), "run", "--model", str(folder), "--dtype", "fp32", "--temp", "0",
           "--max-tokens", "6", "--ctx", "64", "--ignore-eos", "--tokens", ",".join(map(str, prompt))]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    cfg, w = P.load_plain(folder)
    assert [int(t) for t in proc.stdout.strip().split(",")] == P.greedy_generate(cfg, w, prompt, 6)
    assert "9 prompt tok (0 cached)" in proc.stderr and "6 generated" in proc.stderr
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CONFIGS["B"]))
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "jllm"), "bench", "--random-weights", "3", "--model-config",
                           str(cfg_file), "--ctx", "256", "--bench.prompt-tokens", "50", "--bench.max-tokens", "8",
                           "--bench.rounds", "2"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.startswith("prefill 50 tok in") and "decode 8 tok in" in proc.stdout


@pytest.mark.parametrize("overlap", [False, True])
def test_stop_tokens_with_and_without_planning_ahead(tmp_path, overlap):
    """Planned one step ahead, a request whose token turns out to be a stop token has a row in the step after: the row
    is wasted, its token ignored, and every request's output is what it is without planning ahead."""
    from jllm_serve_b200.engine import Engine
    from jllm_serve_b200.sampling import SamplingParams
    base = CONFIGS["A"]
    prompts = [random_tokens(n, base["vocab_size"], 300 + n) for n in (11, 5, 23, 8)]
    kw = dict(dtype="float32", ctx=96, max_batch_tokens=32, chunk=16, max_running=3, page_size=4, max_tokens_cached=384)
    free = Engine(make_model_folder(base, 7, tmp_path / "free"), overlap=False, **kw)
    outs = [r.tokens for r in free.generate(prompts, SamplingParams.greedy_params(20, ignore_eos=True))]
    stops = sorted({outs[0][6], outs[1][3], outs[2][12]})
    want = []
    for o in outs:
        cut = min([o.index(t) for t in stops if t in o] + [len(o)])
        want.append((o[:cut], "stop" if cut < len(o) else "length"))
    eng = Engine(make_model_folder(dict(base, eos_token_id=stops), 7, tmp_path / "stop"), overlap=overlap, **kw)
    got = eng.generate(prompts, SamplingParams.greedy_params(20))
    assert [(r.tokens, r.finish_reason) for r in got] == want
    assert not eng.runner.cache.requests and eng._inflight is None
    eng.runner.cache.check()


def test_seeded_sampling_is_the_same_with_and_without_planning_ahead():
    from jllm_serve_b200.sampling import SamplingParams
    prompts = prompts_for("B", (9, 40, 70, 3), seed=41)
    params = [SamplingParams(temperature=0.9, top_k=30, top_p=0.9, seed=7 + i, max_tokens=20, ignore_eos=True) for i in range(4)]
    a = engine_for("B", "float32", overlap=False).generate(prompts, params)
    b = engine_for("B", "float32", overlap=True).generate(prompts, params)
    assert [r.tokens for r in a] == [r.tokens for r in b]


def test_a_closed_engine_gives_its_device_memory_back_at_once(tmp_path):
    """`with Engine(...)`: at the end of the block the weights, the cache and the captured steps are let go without
    waiting for the garbage collector, so the next engine finds the memory (and no graph dies in mid-capture later)."""
    import gc

    import torch
    from jllm_serve_b200.engine import Engine
    from jllm_serve_b200.sampling import SamplingParams
    folder = model_folder("B")
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    before = torch.cuda.memory_allocated()
    gc.disable()
    try:
        with Engine(folder, dtype="bfloat16", page_size=8, max_tokens_cached=4096, max_batch_tokens=64, chunk=32,
                    max_running=4, ctx=256) as engine:
            out = engine.generate([[1, 2, 3], [4, 5, 6, 7]], SamplingParams.greedy_params(12, ignore_eos=True))
            assert len(out[0].tokens) == 12 and engine.runner._graphs          # decode steps were captured
            held = torch.cuda.memory_allocated() - before
            assert held > 1 << 20
        left = torch.cuda.memory_allocated() - before
    finally:
        gc.enable()
    assert left <= held // 20, f"{left} of {held} bytes are still held after close()"
    with pytest.raises(Exception):
        engine.generate([[1, 2]], SamplingParams.greedy_params(2))


@pytest.mark.parametrize("overlap", [False, True])
def test_cancel_in_the_middle_leaves_the_others_as_they_are_alone(overlap):
    """Three requests step by step through the entry point's own loop; one is cancelled while it decodes (with planning
    ahead: while a step that carries its row is in flight), one while it still waits. The cancelled ones end with
    "cancelled" and the tokens they had; the third's tokens are those it generates alone; a request added afterwards
    takes the pages that came back and is right too; nothing is left in the cache."""
    from jllm_serve_b200.sampling import SamplingParams
    name = "B"
    cfg, w = P.load_plain(model_folder(name))
    prompts = prompts_for(name, (21, 40, 9, 30), seed=77)
    params = SamplingParams.greedy_params(20, ignore_eos=True)
    with engine_for(name, "float32", overlap=overlap, max_running=2, max_tokens_cached=160) as eng:
        a, b, c = (eng.add_request(p, params) for p in prompts[:3])      # two may run: c waits
        for _ in range(9):
            eng.step_once()
        running = {r.id for r in eng.scheduler.running}
        assert running == {a, b} and [r.id for r in eng.scheduler.waiting] == [c]
        assert eng.cancel(c) and eng.cancel(a) and not eng.cancel(a)
        ra = eng.take_result(a)                     # at once, while a step that carries a's row may still be in flight
        d = eng.add_request(prompts[3], params)
        eng.run_until_done()
        rb, rc, rd = (eng.take_result(i) for i in (b, c, d))
        assert not eng.scheduler.finished and not eng._times and not eng._rngs       # taken: nothing is kept
        with pytest.raises(KeyError):
            eng.take_result(a)
        assert rc.finish_reason == "cancelled" and rc.tokens == []
        want_a = P.greedy_generate(cfg, w, prompts[0], 20)
        assert ra.finish_reason == "cancelled" and 1 <= len(ra.tokens) < 20 and ra.tokens == want_a[:len(ra.tokens)]
        assert rb.finish_reason == "length" and rb.tokens == P.greedy_generate(cfg, w, prompts[1], 20)
        assert rd.finish_reason == "length" and rd.tokens == P.greedy_generate(cfg, w, prompts[3], 20)
        assert not eng.runner.cache.requests and eng._inflight is None
        eng.runner.cache.check()
        assert eng.runner.cache.free_pages() == [20]


@pytest.mark.parametrize("name,seed", [("B", 0), ("E", 1), ("C", 2), ("B", 3)])
def test_random_arrivals_cancels_and_a_tight_pool(name, seed):
    """Sixty requests (greedy and seeded sampling) arrive a few at a time, some are cancelled where they stand, the pool
    holds three or four of them, so that requests are preempted and recomputed; with and without planning ahead and
    further prompts' portions in a step. In float32 every request that ran to its end has the very tokens it generates
    alone, every cancelled one a beginning of them, and the cache ends empty with its books in order."""
    from jllm_serve_b200.csrc import ops
    from jllm_serve_b200.sampling import SamplingParams
    rng = random.Random(seed)
    vocab = CONFIGS[name]["vocab_size"]
    specs = []
    for i in range(60):
        n, out = rng.randint(1, 150), rng.randint(1, 40)
        params = (SamplingParams.greedy_params(out, ignore_eos=True) if rng.random() < 0.6 else
                  SamplingParams(temperature=0.9, top_k=30, top_p=0.9, seed=1000 * seed + i, max_tokens=out, ignore_eos=True))
        specs.append((random_tokens(n, vocab, 7919 * seed + i), params))
    kw = dict(max_batch_tokens=96, chunk=64, max_running=5, ctx=256)
    with engine_for(name, "float32", max_tokens_cached=640, **kw) as roomy:
        alone = [roomy.generate([p], sp)[0].tokens for p, sp in specs]
    with engine_for(name, "float32", max_tokens_cached=384, overlap=seed % 2 == 0, fill_portions=seed % 3 != 0, **kw) as eng:
        pending, ids, cancelled, steps = list(range(60)), {}, set(), 0
        while pending or eng.scheduler.has_work() or eng._inflight is not None:
            for _ in range(min(len(pending), rng.randint(0, 3))):
                i = pending.pop(0)
                ids[eng.add_request(*specs[i])] = i
            live = [r.id for r in eng.scheduler.running + eng.scheduler.waiting]
            if live and rng.random() < 0.08:
                rid = rng.choice(live)
                assert eng.cancel(rid)
                cancelled.add(rid)
            eng.step_once()
            steps += 1
            assert steps < 20000
        ops.check_kernel_errors()
        eng.runner.cache.check()
        assert not eng.runner.cache.requests and set(eng.runner.cache.free_pages()) == {48}
        assert cancelled, "the load cancelled nothing"
        # (C's layers but the first look back 40 tokens only and give their pages back as they go: its pool is never short)
        assert name == "C" or eng.scheduler.preemptions > 0, "the pool was large enough: nothing was preempted"
        for rid, i in ids.items():
            r = eng.result_of(rid)
            if rid in cancelled:
                assert r.finish_reason == "cancelled" and r.tokens == alone[i][:len(r.tokens)], f"cancelled request {i}"
            else:
                assert r.finish_reason == "length" and r.tokens == alone[i], f"request {i}"
