"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

`ModelRunner` ties the model, the cache manager and the batch tables together. One call of
`step` runs exactly the tokens it is given, as one batch, on top of what earlier steps left
in the cache; prompt portions and single decoded tokens ride together (the reference's
`forwardMixed`, src/main/java/org/robomiri/jllm/cpu/CpuBackend.java:821-930). Generation,
trace replay, the benchmark and the tests all go through this one function.
"""
from __future__ import annotations

import gc
import json
from pathlib import Path
from typing import Hashable, List, Optional, Sequence

import torch

from ..cache import CacheManager, PoolExhausted
from ..cache.budget import DEFAULT_SHARE, plan_pages
from ..config.registry import architecture_entry, load_config, parse_config
from ..csrc import ops
from ..parts import Runtime
from ..weights import TensorSource, convert_checked, load_checked, random_tensors
from .batch import BatchBuilder, Segment, StepBatch
from .model import build_model, model_wants

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def _as_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not built (bfloat16 or float32)")
        return dtype
    if dtype not in DTYPES:
        raise ValueError(f"dtype {dtype!r} is not built (bfloat16 or float32)")
    return DTYPES[dtype]


class ModelRunner:
    def __init__(self, model_dir=None, *, config: Optional[dict] = None, seed: Optional[int] = None,
                 dtype="bfloat16", device="cuda:0", page_size: int = 16, num_pages=None,
                 max_tokens: Optional[int] = None, max_batch_tokens: int = 2048, max_requests: int = 64,
                 ctx: Optional[int] = None, schedule=None, poison_freed_pages: bool = False,
                 cuda_graphs: bool = True, kv_share: float = DEFAULT_SHARE):
        """Either `model_dir` (config.json + model.safetensors) or `config` + `seed` (random weights made on
        the device). The pool holds `num_pages` pages per group, or enough for `max_tokens` cached tokens, or,
        with `num_pages="auto"`, the share `kv_share` of the device memory that is free once the weights are
        loaded (never more than `max_requests` full contexts need)."""
        ops.require_device()
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = _as_dtype(dtype)
        if model_dir is not None:
            spec, raw = load_config(model_dir)
        elif config is not None:
            spec, raw = parse_config(config), config
        else:
            raise ValueError("a model folder, or a config and a seed, is needed")
        if schedule is not None:
            spec = spec.with_schedule(schedule)
        self.spec, self.config = spec, raw
        entry = architecture_entry(raw["model_type"])
        self.ctx = int(ctx or spec.core.max_positions)
        self.page_size = int(page_size)
        self.max_rows = int(max_batch_tokens)
        self.max_requests = int(max_requests)
        rt = Runtime(self.device, self.dtype, self.ctx, self.max_rows, self.page_size)
        wants = model_wants(entry, spec)
        self.notes: List[str] = []
        if model_dir is not None:
            tensors = load_checked(TensorSource(model_dir), wants, self.dtype, self.device, self.notes)
        else:
            made = random_tensors(wants, 0 if seed is None else seed, self.device, torch.bfloat16)
            tensors = convert_checked(made, wants, self.dtype, self.device)
            del made
        self.model = build_model(entry, spec, tensors, rt)
        self.notes.extend(rt.notes)
        del tensors
        self.runtime = rt
        self.vocab = spec.core.vocab
        needs = self.model.cache_needs()
        self.page_plan = None
        if num_pages == "auto":
            free, total = torch.cuda.mem_get_info(self.device)
            element = torch.empty((), dtype=self.dtype).element_size()
            # the parts' scratch buffers and the logits are made at the first steps: some tens of bytes per element
            # of a step's residual stream, taken off before the share
            held = self.max_rows * int(getattr(spec.core, "dim", 0)) * 64 + 2 * self.max_requests * self.vocab * 4
            self.page_plan = plan_pages(free, total, CacheManager.page_bytes(needs, self.page_size, element),
                                        self.page_size, self.ctx, self.max_requests, kv_share, held)
            num_pages = self.page_plan.pages
            self.notes.append(f"cache pool: {num_pages} pages ({self.page_plan.pool_bytes / 1e9:.1f} GB), limited by "
                              f"{self.page_plan.limited_by}: {self.page_plan.basis}")
        elif num_pages is None:
            tokens = max_tokens if max_tokens is not None else self.ctx * min(self.max_requests, 4)
            num_pages = max(1, -(-int(tokens) // self.page_size))
        self.poison = poison_freed_pages
        self.cache = CacheManager(needs, self.page_size, int(num_pages), self.max_requests, allocate=self._allocate)
        max_blocks = -(-self.ctx // self.page_size)
        self.builder = BatchBuilder(self.device, self.max_rows, self.max_requests, max_blocks, len(self.cache.paged),
                                    self.page_size, ops.resident_blocks())
        self.steps = 0
        self._checked = ops.checks_bounds()
        self.use_graphs = bool(cuda_graphs)
        self.graph_safe = bool(getattr(self.model, "graph_safe", False))    # a model that does not say is not replayed
        self._graphs, self._graph_seen, self._static_logits, self._graph_kernels = {}, set(), None, {}
        self._bucket_caps = {}         # rows of a decode step -> the bucket from which on its launches stay the same
        self.max_graphs = 256          # captured decode shapes kept (rows x wanted rows x key-range bucket)

    def _allocate(self, shape, kind):
        if kind == "kv":
            t = torch.empty(shape, dtype=self.dtype, device=self.device)
            t.fill_(float("nan")) if self.poison else t.zero_()
            return t
        return torch.zeros(shape, dtype=getattr(torch, kind), device=self.device)

    # ---- the step -----------------------------------------------------------------------------------------
    def step(self, segments: Sequence[Segment], logits_out: Optional[torch.Tensor] = None,
             fed_from: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the segments as one batch; returns float32 logits [wanted places, vocab] on the device, in
        the order of the segments and of each segment's `want`. A single-token segment may give the token -(j + 1)
        instead of an id: row j of `fed_from`, an int32 tensor of tokens on the device that the step before sampled
        and the host has not read yet."""
        segments = list(segments)
        if sum(len(s.tokens) for s in segments) > self.max_rows:
            if fed_from is not None:
                raise ValueError("a step that is split over several batches takes its tokens from the host")
            return self._step_in_parts(segments, logits_out)
        return self._step_once(segments, logits_out, fed_from=fed_from)

    def _step_in_parts(self, segments, logits_out):
        """More rows than one batch holds: the same tokens as several batches, one after the other. The
        logits come back in the order that was asked for. The pages of ALL the parts are reserved before the first
        part runs, so a pool that is too small refuses the step before anything of it ran (a windowed group then
        needs pages for the whole span at once, more than running part by part would)."""
        opened = self._open(segments)
        try:
            self.cache.reserve_all([s.request for s in segments], [s.start for s in segments],
                                   [len(s.tokens) for s in segments])
        except Exception:
            for r in opened:
                self.cache.close(r)
            raise
        wanted = sum(len(s.want) for s in segments)
        out = logits_out[:wanted] if logits_out is not None else \
            torch.empty((wanted, self.vocab), dtype=torch.float32, device=self.device)
        parts, room, order = [[]], self.max_rows, [[]]
        k = 0
        for seg in segments:
            places = {}
            for w in seg.want:
                places.setdefault(w, []).append(k)
                k += 1
            lo = 0
            while lo < len(seg.tokens):
                if room == 0:
                    parts.append([])
                    order.append([])
                    room = self.max_rows
                n = min(room, len(seg.tokens) - lo)
                want = [w - lo for w in sorted(places) if lo <= w < lo + n for _ in places[w]]
                order[-1].extend(i for w in sorted(places) if lo <= w < lo + n for i in places[w])
                parts[-1].append(Segment(seg.request, seg.tokens[lo:lo + n], seg.start + lo, want))
                lo += n
                room -= n
        try:
            for part, idx in zip(parts, order):
                logits = self._step_once(part, None, reserve=False)
                if idx:
                    out[torch.tensor(idx, device=self.device)] = logits
        except Exception:
            # a part failed while running: the parts before it stay committed (their rows are in the cache); what
            # was reserved beyond that goes back, and requests that this call opened are closed
            self._give_back(segments, opened)
            raise
        return out

    def _open(self, segments) -> list:
        """Opens the requests of a step that are not open yet; returns those it opened. Nothing stays open if a
        segment does not fit the context."""
        opened = []
        try:
            for seg in segments:
                if seg.start + len(seg.tokens) > self.ctx:
                    raise ValueError(f"request {seg.request!r}: position {seg.start + len(seg.tokens)} is beyond "
                                     f"the context of {self.ctx}")
                if not self.cache.is_open(seg.request):
                    self.cache.open(seg.request)
                    opened.append(seg.request)
        except Exception:
            for r in opened:
                self.cache.close(r)
            raise
        return opened

    def _give_back(self, segments, opened) -> None:
        for seg in segments:
            if seg.request in opened:
                if self.cache.is_open(seg.request):
                    self.cache.close(seg.request)
            elif self.cache.is_open(seg.request):
                self.cache.trim(seg.request)

    def _step_once(self, segments, logits_out, reserve: bool = True, fed_from=None):
        opened = self._open(segments)
        try:
            batch = self.builder.build(segments, self.cache, self.vocab, reserve=reserve)   # all pages or none
        except Exception:
            for r in opened:
                self.cache.close(r)
            raise
        if self._checked:
            ops.set_pool_pages(self.cache.num_pages)     # the library with bounds checks compares page ids with it
        try:
            if fed_from is not None:
                ops.feed_tokens(batch.token_ids, fed_from)
            logits = self._run_model(batch, logits_out)
        except Exception:
            # the step did not run to its end: its pages go back and the books say what they said before it, so
            # the cache and whoever drives the steps still agree
            self._give_back(segments, opened)
            raise
        released = self.builder.commit(self.cache)
        if self.poison:
            self._poison(released)
        self.steps += 1
        self.last_batch = batch
        return logits

    def _run_model(self, batch: StepBatch, logits_out):
        """Decode-only batches are replayed from a captured CUDA graph: a step is some hundreds of short
        kernels, and launching them one by one from the host costs more than running them (the reference
        met the same wall and answered with decode replay, docs/08-metal-backend.md:1354 there). A graph is
        captured the second time a shape is seen (the first run warms every buffer up) and is keyed by what
        the launches bake in: rows, wanted rows and the split of the attention's key range. All device
        addresses a step uses are fixed (batch tables, scratch buffers, the cache), so replaying is exact.
        The returned logits live in a buffer that the next replay overwrites."""
        if batch.decode_only:
            # the bucket that the parts plan their launches by: clamped to where it stops mattering, and below that rounded
            # down to one of a few levels, so that a growing context seldom asks for a new plan (and a new capture)
            cap = self._bucket_caps.get(batch.rows)
            if cap is None:
                cap = self._bucket_caps[batch.rows] = getattr(self.model, "decode_bucket_cap", lambda _: 32)(batch.rows)
            batch.kv_bucket = cap if batch.kv_bucket >= cap else ops.bucket_level(batch.kv_bucket)
        if not (self.use_graphs and self.graph_safe and batch.decode_only):
            return self.model.forward(batch, self.cache, logits_out)
        key = (batch.rows, batch.num_wanted, batch.kv_bucket)
        graph = self._graphs.get(key)
        if graph is None:
            if key not in self._graph_seen:
                self._graph_seen.add(key)
                return self.model.forward(batch, self.cache, logits_out)
            if self._static_logits is None:
                self._static_logits = torch.empty((self.max_requests, self.vocab), dtype=torch.float32,
                                                  device=self.device)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            # Nothing may destroy another CUDA graph while this one is captured (the driver forbids it and the capture
            # is lost): the garbage collector could, if it found an abandoned runner's graphs just now. It is held off
            # during the capture. (A full collection beforehand costs 30 ms and more with a model's objects alive, as
            # much as eight decode steps; `close()` is how a runner's graphs go at a chosen time.)
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    self.model.forward(batch, self.cache, self._static_logits)
            finally:
                if collecting:
                    gc.enable()
            if len(self._graphs) >= self.max_graphs:       # the shape that was captured first makes room
                oldest = next(iter(self._graphs))
                del self._graphs[oldest], self._graph_kernels[oldest]
            self._graphs[key] = graph
            self._graph_kernels[key] = ops.launch_count - before
            ops.launch_count = before
        graph.replay()
        ops.launch_count += self._graph_kernels[key]
        out = self._static_logits[:batch.num_wanted]
        if logits_out is not None:
            logits_out[:batch.num_wanted].copy_(out)
            return logits_out[:batch.num_wanted]
        return out

    def close(self) -> None:
        """Lets go of what the runner holds on the device (captured graphs, the model, the cache), now and not when the
        garbage collector gets to it: a program that builds one runner after another need not hold two at a time. The
        runner cannot step afterwards."""
        torch.cuda.synchronize(self.device)
        self._graphs.clear()
        self._graph_kernels.clear()
        self._graph_seen.clear()
        self._static_logits = None
        self.model = None
        if self.cache is not None:
            self.cache.release_storage()       # (the manager and its books are a cycle: the collector's, later)
        self.cache = None
        self.builder = None
        self.last_batch = None
        self.runtime._buffers.clear()

    def finish(self, request: Hashable) -> None:
        """The request is over: everything it holds is given back."""
        if not self.cache.is_open(request):
            return
        if self.poison:
            rc = self.cache.requests[request]
            held = [(g, p) for g in range(len(self.cache.paged)) for p in rc.tables[g] if p >= 0]
            self.cache.close(request)
            self._poison(held)
        else:
            self.cache.close(request)

    def _poison(self, pages) -> None:
        """Testing aid: a page that was given back is filled with NaN, so a kernel that reads a page its
        request does not hold (or a row that was never written) shows in the logits."""
        for g, page in pages:
            self.cache.paged[g].storage[:, :, page].fill_(float("nan"))

    def describe(self) -> str:
        core = self.spec.core
        return (f"{core.description} | dtype={str(self.dtype).replace('torch.', '')} ctx={self.ctx} "
                f"page={self.page_size} pages={self.cache.num_pages} groups={len(self.cache.paged)} "
                f"max_batch_tokens={self.max_rows}")
