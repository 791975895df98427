"""Shared pieces of the GPU tests: plain-implementation logits, replay through the runner, comparisons."""
from __future__ import annotations

import functools

import torch

from tests.plain import qwen3_plain as P
from tests.tiny import CONFIGS, make_model_folder, random_tokens

# Tolerances, as a share of the largest |logit| of the compared set. float32: the engine and the plain
# implementation differ in summation order only. bfloat16: activations are rounded to 8 bits of mantissa
# several times per layer (2^-9 relative each), while the weights are the same bfloat16 values on both sides.
TOL = {"float32": 5e-6, "bfloat16": 1.2e-2}
# Over all compared rows together, bfloat16 only: the root mean square of the error as a share of the root mean
# square of the logits, and the share of rows that choose the plain implementation's token. The largest
# difference alone lets a damaged row through when another row's logits are large.
RMS_TOL = {"float32": 3e-6, "bfloat16": 8e-3}
ARGMAX_SHARE = {"float32": 1.0, "bfloat16": 0.97}


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
    from jllm_serve_b200.csrc import ops
    ops.check_kernel_errors()        # bounded waits that ran out; in the checked build also accesses out of bounds
    return out


def compare_with_plain(got: dict, folder, requests: dict, dtype: str, schedule=None, what: str = ""):
    """Every (request, position) row against the plain whole-sequence logits: the largest difference (the first
    wrong place is reported), and over all rows the rms error and the share of equal choices."""
    checker = RowChecker(folder, requests, dtype, schedule, what)
    for rid, toks in requests.items():
        for p in range(len(toks)):
            assert (rid, p) in got, f"{what}: no logits for {rid} position {p}"
            checker.row(rid, p, got[(rid, p)])
    worst, _, _ = checker.finish()
    return worst, checker.flips


class RowChecker:
    """Compares logits rows with the plain implementation's as they come and keeps the sums for the bounds that
    hold over all rows together. `sequences[rid]` is the request's whole token list."""

    def __init__(self, folder, sequences: dict, dtype: str, schedule=None, what: str = ""):
        self.folder, self.sequences, self.dtype, self.schedule, self.what = folder, sequences, dtype, schedule, what
        self.rows = self.flips = 0
        self.err2 = self.ref2 = self.worst = self.scale = 0.0
        self.worst_at = None
        self.seen = set()
        self._plain = {}

    def row(self, rid, position: int, got: torch.Tensor) -> None:
        if rid not in self._plain:
            self._plain[rid] = plain_logits(self.folder, tuple(self.sequences[rid]), self.schedule)
        want = self._plain[rid][position]
        assert torch.isfinite(got).all(), f"{self.what}: non-finite logits for {rid} position {position}"
        d = (got - want).double()
        self.err2 += float((d * d).sum())
        self.ref2 += float((want.double() ** 2).sum())
        self.scale = max(self.scale, float(want.abs().max()))
        m = float(d.abs().max())
        if m > self.worst:
            self.worst, self.worst_at = m, (rid, position)
        self.flips += int(got.argmax()) != int(want.argmax())
        self.rows += 1
        self.seen.add((rid, position))

    def finish(self, every_position: bool = True):
        """Asserts the bounds; returns (largest difference, rms share, share of equal choices)."""
        if every_position:
            for rid, toks in self.sequences.items():
                missing = [p for p in range(len(toks)) if (rid, p) not in self.seen]
                assert not missing, f"{self.what}: no logits for {rid} positions {missing[:5]}"
        assert self.rows > 0
        tol = TOL[self.dtype] * self.scale
        rms = (self.err2 / max(self.ref2, 1e-300)) ** 0.5
        agree = 1.0 - self.flips / self.rows
        print(f"{self.what} [{self.dtype}] rows {self.rows}: largest difference {self.worst:.3e} "
              f"({self.worst / max(self.scale, 1e-30):.2e} of the largest |logit|), rms error {rms:.2e} of the rms "
              f"logit, same choice in {100 * agree:.2f} %")
        assert self.worst <= tol, (f"{self.what}: largest difference {self.worst:.3e} at {self.worst_at} exceeds "
                                   f"{tol:.3e} ({self.dtype}, largest |logit| {self.scale:.3f})")
        assert rms <= RMS_TOL[self.dtype], f"{self.what}: rms error {rms:.3e} of the rms logit ({self.dtype})"
        assert agree >= ARGMAX_SHARE[self.dtype], \
            f"{self.what}: only {100 * agree:.2f} % of {self.rows} rows choose the plain implementation's token"
        return self.worst, rms, agree


def replay_checked(runner, steps, checker: RowChecker) -> None:
    """Runs a trace through the step function and checks every wanted row as it comes (a request that is fed
    again from position 0 after it ended, as after a preemption, is checked both times)."""
    from jllm_serve_b200.engine import Segment
    fed = {}
    for st in steps:
        segs = [Segment(e["id"], e["tokens"], fed.get(e["id"], 0), e["want"]) for e in st["entries"]]
        if segs:
            rows = runner.step(segs).float().cpu()
            r = 0
            for e in st["entries"]:
                base = fed.get(e["id"], 0)
                for w in e["want"]:
                    checker.row(e["id"], base + w, rows[r])
                    r += 1
                fed[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            runner.finish(rid)
            fed.pop(rid, None)
    runner.cache.check()
    from jllm_serve_b200.csrc import ops
    ops.check_kernel_errors()
