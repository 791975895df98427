"""Shared pieces of the GPU tests: plain-implementation logits, replay through the runner, comparisons."""
from __future__ import annotations

import functools

import torch

from tests.plain import qwen3_plain as P
from tests.tiny import CONFIGS, make_model_folder, random_tokens

# Tolerances, as a share of the largest |logit| of the compared set. float32: the engine and the plain
# implementation differ in summation order only. bfloat16: activations are rounded to 8 bits of mantissa
# several times per layer (2^-9 relative each), while the weights are the same bfloat16 values on both sides.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


@functools.lru_cache(maxsize=None)
def model_folder(name: str, seed: int = 7):
    return make_model_folder(CONFIGS[name], seed)


@functools.lru_cache(maxsize=None)
def _plain_model(folder):
    return P.load_plain(folder)


def plain_logits(folder, tokens, schedule=None) -> torch.Tensor:
    cfg, w = _plain_model(folder)
    return P.forward(cfg, w, list(tokens), schedule)


def requests_for(name: str, lengths, seed: int = 11) -> dict:
    vocab = CONFIGS[name]["vocab_size"]
    return {f"r{i}": random_tokens(n, vocab, seed + i) for i, n in enumerate(lengths)}


def replay(runner, steps) -> dict:
    """Runs a trace through the step function; {(request, position): logits row on the CPU}."""
    from jllm_serve_b200.engine import Segment
    from tests.traces import collect
    fed = {}

    def run(st):
        segs = []
        for e in st["entries"]:
            segs.append(Segment(e["id"], e["tokens"], fed.get(e["id"], 0), e["want"]))
        rows = runner.step(segs).float().cpu() if segs else None
        for e in st["entries"]:
            fed[e["id"]] = fed.get(e["id"], 0) + len(e["tokens"])
        for rid in st["end"]:
            runner.finish(rid)
            fed.pop(rid, None)
        return rows

    out = collect(steps, run)
    runner.cache.check()
    return out


def compare_with_plain(got: dict, folder, requests: dict, dtype: str, schedule=None, what: str = ""):
    """Every (request, position) row against the plain whole-sequence logits; reports the first wrong place."""
    worst, worst_at, scale = 0.0, None, 0.0
    flips = 0
    for rid, toks in requests.items():
        want = plain_logits(folder, tuple(toks), schedule)
        scale = max(scale, float(want.abs().max()))
        for p in range(len(toks)):
            assert (rid, p) in got, f"{what}: no logits for {rid} position {p}"
            row = got[(rid, p)]
            assert torch.isfinite(row).all(), f"{what}: non-finite logits for {rid} position {p}"
            d = float((row - want[p]).abs().max())
            if d > worst:
                worst, worst_at = d, (rid, p)
            flips += int(row.argmax()) != int(want[p].argmax())
    tol = TOL[dtype] * scale
    assert worst <= tol, (f"{what}: largest difference {worst:.3e} at {worst_at} exceeds {tol:.3e} "
                          f"({dtype}, largest |logit| {scale:.3f})")
    if dtype == "float32":
        assert flips == 0, f"{what}: {flips} positions choose another token than the plain implementation"
    return worst, flips
