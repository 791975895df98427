"""Decode and prefill throughput of the Qwen3-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 requests whose contexts end at 4,096 tokens. `value` is
decoded tokens per second timed on the device with CUDA events around exactly K steps (each step:
the batch tables copied to the device, the captured decode graph replayed, argmax on the device);
`e2e` is the same through the public entry point (`Engine.add_request` / `Engine.step_once`): host
token lists in, sampled tokens read back on the host every step (the engine plans and launches a step
while the one before runs, so the tokens it reads are those of the step before), prompts prefilled by
the engine itself. `prefill` times one 2,048-token prompt; `roofline` compares the bytes a decode step has to
read (every weight once plus the cache of the live requests) with the measured copy bandwidth;
`points` holds decode at batch 1 and 64; `check` compares the bfloat16 logits with the 32-bit path's at these
layer sizes (two layers, untimed). Peaks come from MEASURED_PEAKS.json when it exists.

The engine runs on one GPU; for --gpus above 1 the program says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                attention_bias=False, use_sliding_window=False, max_position_embeddings=40960, hidden_act="silu")
# the layer shapes of BASELINE.json's other configurations (same architecture; random weights): --shape
SHAPES = {"8b": QWEN3_8B,
          "14b": dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, intermediate_size=17408),
          "32b": dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, intermediate_size=25600)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in raw:
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            return out
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--id=0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower() == "active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_numbers(cfg: dict, layers: int) -> dict:
    D, H, Hkv, hd, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                           cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = D * (H + 2 * Hkv) * hd + H * hd * D + 3 * D * F
    return {"layer_params": per_layer, "head_params": V * D, "weight_bytes": 2 * (per_layer * layers + V * D),
            "kv_bytes_per_token": 2 * layers * Hkv * hd * 2,
            "attn_flops_per_layer": lambda T: 4 * (T * (T + 1) // 2) * H * hd}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--rounds", type=int, default=5,
                    help="the K steps are timed this many times, one after the other; the median round is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the configuration has (named in the record)")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: Qwen3-8B (default), 14B or 32B")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length at which the decode steps are timed")
    ap.add_argument("--mixed-chunk", type=int, default=0,
                    help="rows of a prompt portion that rides in every timed step beside the decoding requests")
    ap.add_argument("--kv-share", type=float, default=0.0,
                    help="size the cache pool as this share of the device memory left after the weights (else: the "
                         "pages the run needs)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--prefill-only", action="store_true", help="profiling aid: time the prefill alone and print it")
    ap.add_argument("--skip-check", action="store_true",
                    help="leave out the comparison of the bfloat16 path with the 32-bit path at these layer sizes")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "beniaminp/jllm-serve is a Java 26 program with an Apple "
                          "Metal GPU path (no Python package, no CUDA code): pip cannot install it and no JDK is present"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    args.warmup = max(3, args.warmup)

    import torch

    from jllm_serve_b200.csrc import ops
    from jllm_serve_b200.engine import Engine, Segment
    from jllm_serve_b200.sampling import SamplingParams

    shape = SHAPES[args.shape]
    args.layers = args.layers or shape["num_hidden_layers"]
    ctx = args.context
    default_run = args.shape == "8b" and ctx == CONTEXT and not args.mixed_chunk
    if not default_run:
        args.skip_points = args.skip_e2e = True
    cfg = dict(shape, num_hidden_layers=args.layers)
    nums = model_numbers(cfg, args.layers)
    pk = peaks()
    dev = torch.device("cuda:0")
    biggest = 64 if not args.skip_points else args.batch
    pool_tokens = biggest * ctx + 2 * PREFILL_TOKENS + args.mixed_chunk
    check = None
    if not (args.skip_check or args.prefill_only):
        # the 32-bit path against the bfloat16 path at these layer sizes, on two layers (untimed, before the model)
        from jllm_serve_b200.precision_check import compare_precisions
        # (a prompt of 1,280 rows in portions of 1,024, so that the products of many rows are the ones the prefill takes)
        got = compare_precisions(dict(shape, num_hidden_layers=2), seed=0, prompt=1280, tail=16, portion=1024)["mixed"]
        check = {"what": "bfloat16 logits against the 32-bit path, a 1024+256-row prompt beside 2 decoding requests, "
                         "then 16 tokens one by one", "layers": 2, "layers_of_config": shape["num_hidden_layers"],
                 "rows": got["rows"], "max_rel": round(got["max_rel"], 5), "rms_rel": round(got["rms_rel"], 5),
                 "argmax_agree": round(got["argmax_agree"], 4), "choice_gap_rel": round(got["worst_choice_gap_rel"], 5)}
    t0 = time.time()
    engine = Engine(config=cfg, seed=0, dtype="bfloat16", ctx=ctx, page_size=PAGE,
                    num_pages="auto" if args.kv_share > 0 else pool_tokens // PAGE, kv_share=args.kv_share or 0.6,
                    max_batch_tokens=PREFILL_TOKENS + 64, chunk=PREFILL_TOKENS, max_running=biggest + 1)
    runner = engine.runner
    print(f"bench: {runner.describe()} (built in {time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    for note in runner.notes:
        print(f"bench: {note}", file=sys.stderr, flush=True)
    for g in runner.cache.paged:      # any cached values do for timing; zeros would be kinder to the memory system
        g.storage.normal_()
    out_tok = torch.empty(64, dtype=torch.int32, device=dev)

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def decode_device_timed(batch: int, steps: int, warmup: int, rounds: int = 1):
        """`batch` requests whose contexts END at the context length after warmup + rounds x steps decoded tokens;
        the cache content is synthetic. With --mixed-chunk a portion of a prompt (rows 1,024 onwards of a request
        that is given back after the step) runs in every step before them. Each round times exactly `steps` steps
        between two events with a synchronize on both sides; the median round is reported.
        Returns (ms per step of the median round, mean context during that round, kernels launched in it, ms per
        step of every round)."""
        ids = [f"d{batch}-{i}" for i in range(batch)]
        start = ctx - warmup - rounds * steps
        portions = [0]
        for i in ids:
            runner.cache.open(i)
            runner.cache.reserve(i, 0, start)
            runner.cache.commit(i, start)

        def one_step():
            segs = [Segment(i, [1 + k], runner.cache.length(i), [0]) for k, i in enumerate(ids)]
            if args.mixed_chunk:
                portions[0] += 1
                rid = f"portion{portions[0]}"
                runner.cache.open(rid)
                runner.cache.reserve(rid, 0, 1024)
                runner.cache.commit(rid, 1024)
                segs.insert(0, Segment(rid, list(range(1, args.mixed_chunk + 1)), 1024, []))
            logits = runner.step(segs)
            ops.argmax(logits, out_tok[:batch])
            if args.mixed_chunk:
                runner.finish(segs[0].request)

        for _ in range(warmup):
            one_step()
        times, launched = [], 0
        for _ in range(rounds):
            torch.cuda.synchronize()
            before = ops.launch_count
            s, e = events()
            s.record()
            for _ in range(steps):
                one_step()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e) / steps)
            launched = ops.launch_count - before
        for i in ids:
            runner.finish(i)
        order = sorted(range(rounds), key=lambda r: times[r])
        mid = order[rounds // 2]
        # the median round ran steps [mid * steps, (mid + 1) * steps) of the timed ones: its mean context
        mean_ctx = ctx - (rounds - mid) * steps + steps / 2.0
        return times[mid], mean_ctx, launched, times

    def decode_bytes(batch: int, context: float) -> float:
        return nums["weight_bytes"] + batch * context * nums["kv_bytes_per_token"]

    if args.prefill_only:
        g = torch.Generator().manual_seed(1)
        prompt = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
        for i in range(max(1, args.steps)):
            s, e = events()
            s.record()
            runner.step([Segment(f"p{i}", prompt, 0, [PREFILL_TOKENS - 1])])
            e.record()
            torch.cuda.synchronize()
            runner.finish(f"p{i}")
            print(json.dumps({"prefill_ms": round(s.elapsed_time(e), 3)}))
        return 0

    # ---- the headline: decode at the default batch, clocks sampled meanwhile -------------------------------
    clocks = ClockSampler()
    clocks.start()
    ms_step, mean_ctx, launches, round_ms = decode_device_timed(args.batch, args.steps, args.warmup, max(1, args.rounds))
    clock_record = clocks.stop()
    clock_record["rounds_ms_per_step"] = [round(t, 4) for t in round_ms]
    value = args.batch * 1000.0 / ms_step
    achieved = decode_bytes(args.batch, mean_ctx) / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                "bytes": int(decode_bytes(args.batch, mean_ctx))}

    # ---- prefill of one 2,048-token prompt ---------------------------------------------------------------------
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()

    def prefill_once(tag):
        s, e = events()
        s.record()
        runner.step([Segment(tag, prompt, 0, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        runner.finish(tag)
        return s.elapsed_time(e)

    # 4 warm-up prefills, then the median of 9: a single 30 ms prefill follows the clock of the moment
    times = [prefill_once(f"p{i}") for i in range(13)] if not args.skip_prefill else [float("nan")] * 13
    pre_ms = statistics.median(times[4:])
    flops = 2.0 * nums["layer_params"] * args.layers * PREFILL_TOKENS + nums["attn_flops_per_layer"](PREFILL_TOKENS) \
        * args.layers + 2.0 * nums["head_params"]
    prefill = {"value": round(PREFILL_TOKENS / pre_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "tflops": round(flops / pre_ms / 1e9, 1),
               "peak_tflops": pk["bf16_tflops"], "peak_source": pk["source"]}
    if "bf16_tflops_sustained" in pk:       # the same against what the GEMM library sustains under the power cap
        prefill["frac_of_sustained"] = round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
    if args.skip_prefill:
        prefill = None

    # ---- decode at batch 1 and 64 --------------------------------------------------------------------------------
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            ms_b, ctx_b, _, _ = decode_device_timed(b, max(8, args.steps // 2), 3, 3)
            gbs = decode_bytes(b, ctx_b) / (ms_b * 1e-3) / 1e9
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
            points[f"decode_b{b}_ms"] = round(ms_b, 4)
            points[f"decode_b{b}_hbm_frac"] = round(gbs / pk["hbm_gbs"], 4)

    # ---- end to end through the public entry point --------------------------------------------------------------
    e2e = None
    if not args.skip_e2e:
        e2e = end_to_end(engine, args.batch, args.steps, args.warmup, cfg["vocab_size"])
        if not args.skip_points:
            for b in (1, 64):
                other = end_to_end(engine, b, args.steps, args.warmup, cfg["vocab_size"])
                points[f"e2e_b{b}"] = other["value"]

    record = {
        "metric": (f"decode tok/s @ batch {args.batch}, context {ctx} (Qwen3-{args.shape.upper()} shape, bf16, random weights"
                   + (f", a {args.mixed_chunk}-row prompt portion in every step)" if args.mixed_chunk else ")")),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights N(0, 0.02); device-timed cache content synthetic",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": args.layers,
                   "layers_of_config": shape["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "seq_len": ctx, "page_size": PAGE, "mixed_chunk": args.mixed_chunk, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 (weights {nums['weight_bytes'] / 1e9:.0f} GB per step)",
                   "cuda_graphs": runner.use_graphs},
        "clocks": clock_record, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline,
        "points": points, "check": check,
    }
    print(json.dumps(record))
    return 0


def end_to_end(engine, batch: int, steps: int, warmup: int, vocab: int):
    """Decode tokens per second through Engine.add_request / Engine.step_once: every step copies its batch
    tables from pinned host memory to the device and reads the sampled tokens back to the host."""
    import torch

    from jllm_serve_b200.sampling import SamplingParams
    # the prompts are prefilled one after the other (two portions each): a request that is ready early decodes while the
    # others' prompts still run, so every request may generate that many tokens more than the timed steps need and none
    # ends inside the timed region
    slack = 2 * batch + 2
    new_tokens = warmup + steps + 1 + slack
    prompt_len = CONTEXT - new_tokens
    g = torch.Generator().manual_seed(2)
    params = SamplingParams.greedy_params(max_tokens=new_tokens, ignore_eos=True)
    ids = [engine.add_request(torch.randint(0, vocab, (prompt_len,), generator=g).tolist(), params)
           for _ in range(batch)]
    sched = engine.scheduler
    while any(r.remaining > 1 or not r.output for r in sched.running + sched.waiting):
        engine.step_once()                       # prefill (untimed): until every request is decoding
    for _ in range(warmup - 1):
        engine.step_once()
    torch.cuda.synchronize()
    h2d = engine.runner.builder.bytes_per_step(batch)
    mine = [r for r in sched.running + sched.waiting]

    def generated():
        return sum(len(r.output) for r in mine)

    before = generated()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step_once()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    done = generated() - before          # tokens that were really sampled (a preempted request decodes nothing)
    if done != steps * batch:
        print(f"bench: end to end at batch {batch}: {done} tokens in {steps} steps, expected {steps * batch}",
              file=sys.stderr, flush=True)
    engine.run_until_done()
    for i in ids:
        engine.take_result(i)
    return {"value": round(done / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * engine.sampler.max_rows,
            "ms_per_step": round(dt / steps * 1e3, 4), "tokens_per_step": round(done / steps, 2),
            "preemptions": sched.preemptions}


if __name__ == "__main__":
    sys.exit(main())
