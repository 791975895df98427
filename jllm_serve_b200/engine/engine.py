"""The Python entry point: load a model, generate for a list of prompts.

The reference's programmatic surface is `ModelLoader.load(...)` + `Engine.generate(prompt,
SamplingParams, sink, cancelled) -> Result(text, tokens, finishReason, Stats)`
(src/main/java/org/robomiri/jllm/ModelLoader.java:159-210, engine/Engine.java:43-78,368-376).
Here prompts are token ids (the engine carries no tokenizer) and many prompts are generated
together by the scheduler: `Engine(model_dir, ...).generate(prompts, params) -> [Result]`.
`add_request` / `run_until_done` drive the same loop by hand; `step` is the raw step
function.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence, Union

import torch

from ..csrc import ops
from ..sampling import RequestRng, Sampler, SamplingParams
from .batch import Segment
from .runner import ModelRunner
from .scheduler import FINISHED, Request, Scheduler


@dataclass
class Stats:
    """As the reference's Engine.Stats (engine/Engine.java:43-57): counts and the two phases' times."""
    prompt_tokens: int = 0
    cached_tokens: int = 0
    generated: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    preemptions: int = 0

    @property
    def tok_per_sec(self) -> float:
        return self.generated / (self.decode_ms / 1000.0) if self.decode_ms > 0 else 0.0

    def line(self) -> str:
        """The reference's stats line (Main.java:384-389)."""
        return (f"{self.prompt_tokens} prompt tok ({self.cached_tokens} cached), prefill {self.prefill_ms:.0f} ms, "
                f"{self.generated} generated in {self.decode_ms:.0f} ms = {self.tok_per_sec:.1f} tok/s")


@dataclass
class Result:
    tokens: List[int]
    finish_reason: str
    stats: Stats = field(default_factory=Stats)


class Engine:
    def __init__(self, model_dir=None, *, config: Optional[dict] = None, seed: Optional[int] = None,
                 dtype="bfloat16", device="cuda:0", ctx: Optional[int] = None, page_size: int = 16,
                 num_pages=None, max_tokens_cached: Optional[int] = None,
                 max_batch_tokens: int = 2048, chunk: int = 512, min_chunk: int = 16, max_running: int = 64,
                 sample_vocab: Optional[int] = None, cuda_graphs: bool = True, kv_share: float = 0.6,
                 overlap: bool = True, fill_portions: bool = True):
        """`num_pages`: pages of the cache pool, or "auto" for the share `kv_share` of the device memory that is
        free once the weights are loaded; without it the pool holds `max_tokens_cached` tokens (default: four
        full contexts). `overlap`: a step is planned and launched while the step before it still runs, its sampled
        tokens going from one step into the next on the device; the host reads them one step later (what `step_once`
        returns lags by a step; `run_until_done` and `generate` do not care). `fill_portions`: a step whose first prompt
        portion left room in `max_batch_tokens` takes the portions of the next waiting prompts too (False: one portion
        to a step, as the reference plans its passes)."""
        self.runner = ModelRunner(model_dir, config=config, seed=seed, dtype=dtype, device=device,
                                  page_size=page_size, num_pages=num_pages, max_tokens=max_tokens_cached,
                                  max_batch_tokens=max_batch_tokens, max_requests=max_running, ctx=ctx,
                                  cuda_graphs=cuda_graphs, kv_share=kv_share)
        core = self.runner.spec.core
        self.scheduler = Scheduler(self.runner.cache, self.runner.ctx, max_batch_tokens, chunk, min_chunk, max_running,
                                   eos_ids=core.eos, commits=False,       # the runner commits every step it ran
                                   row_quantum=ops.TILE_ROWS if self.runner.dtype == torch.bfloat16 else 0,
                                   fill_portions=fill_portions)
        self.sampler = Sampler(self.runner.device, max_running, core.vocab, sample_vocab)
        self._rngs = {}
        self._times = {}
        self._ids = 0
        self.overlap = bool(overlap)
        self._inflight = None              # (the planned segments, the ticket of their sampling) of a launched step

    # ---- requests ------------------------------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        params = params or SamplingParams()
        rid = request_id if request_id is not None else f"req-{self._ids}"
        self._ids += 1
        prompt = [int(t) for t in prompt]
        vocab = self.runner.vocab
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"request {rid!r}: token id outside [0, {vocab})")
        self.scheduler.add(Request(rid, prompt, params))
        self._rngs[rid] = RequestRng(params.seed)
        self._times[rid] = {"start": time.perf_counter(), "first": None, "end": None}
        return rid

    def cancel(self, request_id: Hashable) -> bool:
        """Ends the request now (finish reason "cancelled"; `result_of` gives what it had generated). Its pages go back
        at once; a step in flight that still carries a row of it runs on, and the row is ignored. False if there is no
        such request or it has ended already."""
        r = self.scheduler.cancel(request_id)
        if r is None:
            return False
        self._times[request_id]["end"] = time.perf_counter()
        self._rngs.pop(request_id, None)
        return True

    def step_once(self) -> List[Request]:
        """One scheduler step: plan, launch, and read the tokens of the step before (without `overlap`: of this
        step). Returns the requests that finished, those included that the scheduler ended while planning because
        the pool can never hold them (`kv_exhausted`)."""
        finished: List[Request] = []
        plan = None
        if self._inflight is not None:
            plan = self.scheduler.plan(inflight=self._inflight[0])
            if plan is None:               # the pool is short: no planning ahead of the tokens that are on their way
                finished += self._read_inflight()
        if plan is None:
            plan = self.scheduler.plan()
        ended = self.scheduler.take_ended()
        now = time.perf_counter()
        for r in ended:
            self._times[r.id]["end"] = now
            self._rngs.pop(r.id, None)
        finished += ended
        launched = self._launch(plan) if plan else None
        finished += self._read_inflight()          # the step before this one (it ran while this one was prepared)
        self._inflight = launched
        if launched is not None and not self.overlap:
            finished += self._read_inflight()
        return finished

    def _launch(self, plan):
        """Hands the planned segments to the step function and starts the choice of their tokens; waits for nothing."""
        segments = [Segment(p.request.id, p.tokens, p.start, [len(p.tokens) - 1] if p.wants_logits else [])
                    for p in plan]
        fed = any(len(p.tokens) == 1 and p.tokens[0] < 0 for p in plan)
        logits = self.runner.step(segments, fed_from=self._inflight[1].device_tokens if fed else None)
        wanting = [p.request for p in plan if p.wants_logits]
        ticket = self.sampler.launch(logits, [r.params for r in wanting],
                                     [0.0 if r.params.greedy else self._rngs[r.id].next() for r in wanting])
        return plan, ticket

    def _read_inflight(self) -> List[Request]:
        """Waits for the tokens of the step in flight, hands them to the scheduler; the requests they finished."""
        if self._inflight is None:
            return []
        plan, ticket = self._inflight
        self._inflight = None
        sampled = self.sampler.fetch(ticket)
        now = time.perf_counter()
        for p in plan:
            if p.request.state == FINISHED:             # cancelled while the step ran (its result may be taken already)
                continue
            times = self._times.get(p.request.id)
            if p.wants_logits and times is not None and times["first"] is None:
                times["first"] = now
        done = self.scheduler.complete(plan, sampled)
        for r in done:
            self._times[r.id]["end"] = now
            self._rngs.pop(r.id, None)
        return done

    def run_until_done(self) -> List[Request]:
        finished = []
        steps = 0
        while self.scheduler.has_work() or self._inflight is not None:
            finished.extend(self.step_once())
            steps += 1
            if steps % 256 == 0:
                ops.check_kernel_errors()
        ops.check_kernel_errors()          # a kernel that gave up on a bounded wait must not pass for a result
        return finished

    def close(self) -> None:
        """The engine's device memory (weights, cache, captured steps) is let go now; the engine cannot step afterwards.
        Also at the end of a `with Engine(...) as engine:` block."""
        self._inflight = None
        self.runner.close()
        self.sampler = None
        self.scheduler = None

    def __enter__(self) -> "Engine":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def result_of(self, rid: Hashable) -> Result:
        r = self.scheduler.finished[rid]
        t = self._times[rid]
        end = t["end"] or time.perf_counter()
        first = t["first"] or end
        return Result(list(r.output), r.finish_reason,
                      Stats(len(r.prompt), 0, len(r.output), (first - t["start"]) * 1e3, (end - first) * 1e3,
                            r.preemptions))

    def take_result(self, rid: Hashable) -> Result:
        """`result_of` for a request that has ended, after which the engine forgets the request: whoever drives
        `add_request` and `step_once` for a long time takes every result this way, or the finished requests pile up."""
        if rid not in self.scheduler.finished:
            raise KeyError(f"request {rid!r} has not ended (or its result was taken already)")
        out = self.result_of(rid)
        self.scheduler.finished.pop(rid)
        self._rngs.pop(rid, None)
        self._times.pop(rid, None)
        return out

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[Result]:
        """Generates for every prompt (token ids); one SamplingParams for all, or one per prompt."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError(f"{len(prompts)} prompts but {len(params)} sampling parameters")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        self.run_until_done()
        return [self.take_result(i) for i in ids]

    def step(self, segments: Sequence[Segment]) -> torch.Tensor:
        """The raw step function: logits [wanted places, vocab] for a batch of (request, its next tokens)."""
        return self.runner.step(segments)

    def finish(self, request: Hashable) -> None:
        self.runner.finish(request)

    def describe(self) -> str:
        return self.runner.describe()
