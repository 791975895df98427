"""The scheduler: admits requests, forms each step's batch under a token budget, finishes and frees.

`plan_pass` is a port of the reference's pass-forming rule, function for function (docs/25-scheduler.md;
src/main/java/org/robomiri/jllm/engine/PassPlanner.java:74-112, without its classes, aging and background cap, and
with the row quantum added): the rule is the contract, and the reference's own test vectors are this module's
tests. Every decoding request
rides along with its one token, in order of arrival, while it fits the budget; then ONE
prompt portion, the head of the prefill line, takes what is left, trimmed to the room, but
only if that is at least `min_chunk` rows (or all the portion needs); if nothing fits, the
oldest item goes alone, so a pass is never empty. A prompt that has run a portion goes to
the back of the prefill line, so prompts alternate (docs/25:133-134). Beyond that rule, a pass whose head portion
left room takes the portions of the next prompts in the line too (`_more_portions`; `fill_portions=False` is the
reference's one portion to a pass).

Admission is first come, first served (the reference's classes, aging and sessions,
engine/Admission.java:217-285, are not built): a waiting request starts when fewer than
`max_running` run and there are free pages for all the tokens it has (prompt and, after a preemption, what it had
generated) and one more, and a page to spare for every request that runs already; with nothing else running it
starts if its first portion fits.

When pages run out. A step's pages are reserved before it runs. If the pool cannot cover
a step, the most recently admitted running request is preempted: its pages go back, it
returns to the FRONT of the waiting line with everything it has generated so far as part
of its prompt, and is recomputed later (the reference pauses the newest background request
and recomputes what could not be kept: engine/Admission.java:288-301, engine/Engine.java:
657-666). The oldest request is never preempted, so it always finishes; a request that
cannot fit in the empty pool ends with the reason "kv_exhausted".

One step ahead. `plan` may be called while the step before is still running on the device and its
sampled tokens have not been read (`plan(inflight=that step's segments)`): a request whose next token is
among them is planned with a marker in place of the token (the runner takes the token from the device),
on the guess that the token is no stop token; a request that those tokens complete by length is left out.
`complete` of the earlier step comes afterwards; if it ends a request by a stop token, the rows that were
planned for it on the guess are wasted and their token ignored. Planning ahead never preempts: if the pool
is short it returns None and the caller completes the step in flight first.

The scheduler is host logic only: it asks the cache manager for pages and tells the caller
which segments to run; it never touches a tensor.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence

from ..cache import PoolExhausted
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    state: str = WAITING
    computed: int = 0                      # tokens whose keys and values are in the cache (steps that were completed)
    launched: int = 0                      # tokens whose rows were handed to a step; ahead of `computed` by a step in flight
    unknown: int = 0                       # tokens that steps in flight will sample: part of the sequence, not yet read
    finish_reason: Optional[str] = None
    arrival: int = 0
    admitted: int = -1                     # order of (re)admission, for choosing whom to preempt
    preemptions: int = 0
    max_new: int = 0                       # max_tokens clamped to the context

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def tokens_between(self, lo: int, hi: int) -> List[int]:
        """tokens[lo:hi] without joining the prompt and the output."""
        n = len(self.prompt)
        if lo >= n:
            return self.output[lo - n:hi - n]
        if hi <= n:
            return self.prompt[lo:hi]
        return self.prompt[lo:] + self.output[:hi - n]

    @property
    def remaining(self) -> int:
        """Tokens of the sequence (those still to be read from a step in flight included) not yet handed to a step."""
        return len(self.prompt) + len(self.output) + self.unknown - self.launched

    @property
    def ends_by_length(self) -> bool:
        """The tokens it has, with those on their way, are all it may have: it is not scheduled again."""
        n_out = len(self.output) + self.unknown
        return n_out >= self.max_new

    def feed_marker(self, index: int) -> int:
        """What stands for a token that is still on the device: row `index` of the step before's samples."""
        return -(index + 1)


@dataclass(frozen=True)
class Item:
    """One piece of pending work for the pass planner."""
    ref: object
    kind: str                              # "rider" (a decoding request's rows, all wanted) or "chunk"
    rows: int
    enqueued: int
    more: bool = False                     # a chunk whose prompt goes on after these rows


@dataclass(frozen=True)
class Pick:
    ref: object
    kind: str
    rows: int


def plan_pass(pending: Sequence[Item], budget: int, min_chunk: int, row_quantum: int = 0) -> List[Pick]:
    """The picks of the next pass: the chunk (if any) first, then the riders by arrival.

    Riders that do not fit are left for the next pass, never trimmed; the chunk is the head of the
    `pending` chunks in the order given, trimmed to the room left, and waits if the room is smaller
    than min(min_chunk, its rows). With `row_quantum` (the rows of a matrix-product tile) a chunk that is cut
    anyway, because its prompt goes on after it, is cut so that the pass has a whole number of tiles: the rows
    beyond the last full tile would cost a tile of their own."""
    if budget < 1:
        raise ValueError("a pass needs a budget of at least one row")
    riders = sorted((i for i in pending if i.kind != "chunk"), key=lambda i: i.enqueued)
    chunks = [i for i in pending if i.kind == "chunk"]
    used, rider_picks = 0, []
    for r in riders:
        if used + r.rows <= budget:
            rider_picks.append(Pick(r.ref, r.kind, r.rows))
            used += r.rows
    out: List[Pick] = []
    if chunks:
        c = chunks[0]
        rows = min(c.rows, budget - used)
        over = (used + rows) % row_quantum if row_quantum > 1 else 0
        if over and used + rows > row_quantum and (c.more or rows < c.rows) and rows - over >= max(min_chunk, 1):
            rows -= over
        if rows >= min(min_chunk, c.rows) and rows > 0:
            out.append(Pick(c.ref, "chunk", rows))
    out.extend(rider_picks)
    if not out and pending:
        first = min(pending, key=lambda i: i.enqueued)
        out.append(Pick(first.ref, first.kind, min(first.rows, budget) if first.kind == "chunk" else first.rows))
    return out


@dataclass
class PlannedSegment:
    request: Request
    start: int
    tokens: List[int]
    wants_logits: bool


class Scheduler:
    def __init__(self, cache, ctx: int, max_batch_tokens: int, chunk: int = 512, min_chunk: int = 16,
                 max_running: int = 64, eos_ids: Sequence[int] = (), commits: bool = True, row_quantum: int = 0,
                 fill_portions: bool = True):
        """`commits`: whether `plan` records the new lengths in the cache when it hands a step out (False when whoever
        runs the steps does that itself, as the model runner does at launch). `row_quantum`: see `plan_pass`.
        `fill_portions`: see `_more_portions`."""
        self.cache, self.ctx, self.commits, self.row_quantum = cache, ctx, commits, row_quantum
        self.fill_portions = fill_portions
        self.budget, self.chunk, self.min_chunk, self.max_running = max_batch_tokens, chunk, min_chunk, max_running
        self.eos = set(eos_ids)
        self.waiting: List[Request] = []
        self.running: List[Request] = []
        self.prefill_line: List[Request] = []
        self.finished: Dict[Hashable, Request] = {}
        self._clock = itertools.count()
        self._admissions = itertools.count()
        self.preemptions = 0
        self.on_finish: Optional[Callable[[Request], None]] = None
        self._ended_planning: List[Request] = []

    # ---- requests in -------------------------------------------------------------------------------------
    def add(self, request: Request) -> None:
        n = len(request.prompt)
        if n < 1:
            raise ValueError(f"request {request.id!r}: the prompt is empty")
        if n >= self.ctx:
            raise ValueError(f"request {request.id!r}: a prompt of {n} tokens does not fit the context of {self.ctx}")
        if request.id in self.finished or any(r.id == request.id for r in self.waiting + self.running):
            raise ValueError(f"request {request.id!r}: there is a request of this name already "
                             f"({'ended, its result not taken' if request.id in self.finished else 'not ended'})")
        request.arrival = next(self._clock)
        request.max_new = min(request.params.max_tokens, self.ctx - n)
        request.state = WAITING
        self.waiting.append(request)

    def cancel(self, request_id: Hashable) -> Optional[Request]:
        """Ends a waiting or running request now, with the reason "cancelled" (the reference: engine/Engine.java:668-671):
        what it holds is given back, what it has generated so far stays its output. Rows of it that a step in flight
        still carries are passed over when that step is completed, as those of a request that a stop token ended. None if
        there is no such request, or it has ended already."""
        for r in self.waiting + self.running:
            if r.id == request_id:
                if r in self.waiting:
                    self.waiting.remove(r)
                self._release(r)
                self._finish(r, "cancelled")
                return r
        return None

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def take_ended(self) -> List[Request]:
        """The requests that `plan` ended itself since the last call (they can never fit the pool: `kv_exhausted`).
        They never reach `complete`, so whoever drives the steps learns of them here."""
        out, self._ended_planning = self._ended_planning, []
        return out

    # ---- one step ------------------------------------------------------------------------------------------
    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.max_running:
            r = self.waiting[0]
            first = min(r.remaining, self.chunk, self.budget)
            # Room for everything it has so far (its prompt, and what it had generated when it was preempted) and one
            # token more, not only for its first portion: a request that starts on less is preempted as soon as it has
            # grown, and one that was preempted would come back into the room it has just given up, again and again.
            # ... beside what the running requests still lack for the tokens THEY have (one that was admitted a moment
            # ago holds nothing yet), and a page of growth for each of them.
            if self.running:
                page = self.cache.page_size
                owed = sum(max(0, -(-(len(q.prompt) + len(q.output) + 1) // page) - -(-q.launched // page))
                           for q in self.running)
                if not self._fits_now(r, r.remaining + 1, spare_pages=owed + len(self.running)):
                    break
            if not self._fits_now(r, first + 1):
                # alone in an empty pool and still no room for its first portion: it can never run
                self.waiting.pop(0)
                self._finish(r, "kv_exhausted")
                continue
            self.waiting.pop(0)
            r.state, r.admitted = RUNNING, next(self._admissions)
            self.running.append(r)
            self.cache.open(r.id)
            if r.remaining > 1:
                self.prefill_line.append(r)

    def _fits_now(self, r: Request, rows: int, spare_pages: int = 0) -> bool:
        rows = min(rows, self.ctx - r.launched)
        if self.cache.is_open(r.id):
            return self.cache.can_reserve(r.id, r.launched, rows)
        missing = -(-(r.launched + rows) // self.cache.page_size)
        return all(missing + spare_pages <= free for free in self.cache.free_pages())

    def plan(self, inflight: Optional[Sequence["PlannedSegment"]] = None) -> Optional[List[PlannedSegment]]:
        """Admits, picks the step's segments and reserves their pages (preempting if the pool is short). With
        `inflight` (the segments of a step whose tokens have not been read yet) it plans one step ahead and never
        preempts: None means that the step in flight has to be completed first."""
        ahead = inflight is not None
        fed = {}
        if ahead:
            wanting = [seg.request for seg in inflight if seg.wants_logits]
            fed = {r.id: j for j, r in enumerate(wanting)}
        self._admit()
        while True:
            items = []
            for r in sorted(self.running, key=lambda q: q.arrival):
                if r.remaining == 1 and r not in self.prefill_line and not self._full(r):
                    items.append(Item(r, "rider", 1, r.arrival))
            for r in self.prefill_line:
                items.append(Item(r, "chunk", min(r.remaining, self.chunk), r.arrival, r.remaining > self.chunk + 1))
            if not items:
                return []
            picks = plan_pass(items, self.budget, self.min_chunk, self.row_quantum)
            if self.fill_portions:
                picks = self._more_portions(picks, items)
            try:      # pages for every pick, or for none
                self.cache.reserve_all([p.ref.id for p in picks], [p.ref.launched for p in picks],
                                       [p.rows for p in picks])
            except PoolExhausted:
                if ahead:
                    return None
                if not self._preempt_one():
                    # a single running request that cannot grow: it ends here
                    r = self.running[0]
                    self._release(r)
                    self._finish(r, "kv_exhausted")
                    if not self.has_work():
                        return []
                    self._admit()
                continue
            segments = []
            for p in picks:
                r = p.ref
                known = len(r.prompt) + len(r.output)
                if r.launched + p.rows > known:
                    # its next token is among those the step in flight samples: the runner takes it from the device
                    toks = [r.feed_marker(fed[r.id])]
                else:
                    toks = r.tokens_between(r.launched, r.launched + p.rows)
                wants = r.launched + p.rows == known + r.unknown
                segments.append(PlannedSegment(r, r.launched, toks, wants))
                if p.kind == "chunk":
                    self.prefill_line.remove(r)
                    if r.remaining - p.rows > 1:
                        self.prefill_line.append(r)   # to the back: prompts alternate
            for seg in segments:
                seg.request.launched += len(seg.tokens)
                seg.request.unknown += 1 if seg.wants_logits else 0
                if self.commits:       # as the model runner does when it launches a step: the rows count as written
                    self.cache.commit(seg.request.id, seg.request.launched)
            return segments

    def _more_portions(self, picks: List[Pick], items: Sequence[Item]) -> List[Pick]:
        """Beyond the reference's rule (one prompt portion to a pass): if the head of the prefill line got all the rows it
        asked for and the budget has room left, the portions of the prompts behind it are taken too, in the line's order,
        each whole or cut to the room as the head would be. The reference's passes are sized for a GPU that a portion of
        512 rows fills; here a step streams every weight once whatever its rows, and thirty prompts of fifty tokens that
        arrive together should cost two steps, not thirty. The portions stay in front of the single rows."""
        chunks = [i for i in items if i.kind == "chunk"]
        if not picks or picks[0].kind != "chunk" or len(chunks) < 2 or picks[0].rows < chunks[0].rows:
            return picks
        used, more, q = sum(p.rows for p in picks), [], self.row_quantum
        for it in chunks[1:]:
            rows = min(it.rows, self.budget - used)
            over = (used + rows) % q if q > 1 else 0
            if over and used + rows > q and (it.more or rows < it.rows) and rows - over >= max(self.min_chunk, 1):
                rows -= over
            if rows < 1 or rows < min(self.min_chunk, it.rows):
                break
            more.append(Pick(it.ref, "chunk", rows))
            used += rows
            if rows < it.rows:
                break
        return picks[:1] + more + picks[1:]

    def _full(self, r: Request) -> bool:
        """With the tokens it has and those on their way the request has all it may have."""
        return r.ends_by_length or len(r.prompt) + len(r.output) + r.unknown >= self.ctx

    def _preempt_one(self) -> bool:
        """The most recently admitted running request gives everything back and waits again, in front."""
        if len(self.running) <= 1:
            return False
        victim = max(self.running, key=lambda q: q.admitted)
        self._release(victim)
        victim.state, victim.computed, victim.launched = WAITING, 0, 0
        victim.preemptions += 1
        self.preemptions += 1
        self.waiting.insert(0, victim)
        return True

    def _release(self, r: Request) -> None:
        if r in self.running:
            self.running.remove(r)
        if r in self.prefill_line:
            self.prefill_line.remove(r)
        if self.cache.is_open(r.id):
            self.cache.close(r.id)

    def _finish(self, r: Request, reason: str) -> None:
        r.state, r.finish_reason = FINISHED, reason
        self.finished[r.id] = r
        if reason == "kv_exhausted":
            self._ended_planning.append(r)
        if self.on_finish:
            self.on_finish(r)

    def complete(self, segments: Sequence[PlannedSegment], sampled: Sequence[int]) -> List[Request]:
        """After the step ran: lengths are committed, the sampled tokens (one per segment that wanted
        logits, in order) are appended, and requests that are done are finished and freed. Rows of a request that an
        earlier step's token has ended meanwhile (they were planned ahead, on the guess that it goes on) are passed
        over."""
        done = []
        it = iter(sampled)
        for seg in segments:
            r = seg.request
            tok = next(it) if seg.wants_logits else None
            if r.state == FINISHED:
                continue
            r.computed = seg.start + len(seg.tokens)
            if not seg.wants_logits:
                continue
            r.unknown -= 1
            if not r.params.ignore_eos and (tok in self.eos or tok in r.params.stop_token_ids):
                reason = "stop"            # the stop token is not part of the output
            else:
                r.output.append(tok)
                reason = "length" if len(r.output) >= r.max_new or len(r.prompt) + len(r.output) >= self.ctx else None
            if reason:
                self._release(r)
                self._finish(r, reason)
                done.append(r)
        return done
