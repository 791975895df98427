"""One step's batch: which tokens of which requests run, and the device tables the kernels read.

A step is a list of segments. A segment is a request's next tokens: a portion of its prompt
or one decoded token; the reference calls it `Segment(owner, tokens, off, n, pos, logits,
stride)` (src/main/java/org/robomiri/jllm/model/Backend.java:138-153). All rows of all
segments are laid side by side, segment after segment; row-wise kernels see one batch of
`rows` rows, the attention kernels see per-row (segment, position) and per-segment tables.

`BatchBuilder` owns one pinned host buffer and one device buffer of fixed size, so the
device addresses never change (a captured decode step can be replayed) and a step costs
two host-to-device copies. The tables are packed by the C++ host library straight from the
cache's books into the pinned buffers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Sequence

import numpy as np
import torch

from ..cache import native


@dataclass
class Segment:
    request: Hashable
    tokens: Sequence[int]
    start: int                             # position of tokens[0] in the request
    want: Sequence[int] = ()               # places among `tokens` whose logits are asked for


@dataclass
class StepBatch:
    rows: int
    segments: List[Segment]
    token_ids: torch.Tensor                # int32 [rows]
    positions: torch.Tensor                # int32 [rows]
    row_seg: torch.Tensor                  # int32 [rows]
    seg_start: torch.Tensor                # int32 [segments]: first row of the segment
    seg_len: torch.Tensor                  # int32 [segments]: its rows in this step
    seg_kv_len: torch.Tensor               # int32 [segments]: positions the request holds after this step
    state_slots: torch.Tensor              # int32 [segments]
    logit_rows: torch.Tensor               # int32 [wanted]: rows whose logits are computed, in order
    slots: List[torch.Tensor]              # per paged group: int32 [rows], cache row = page * page_size + offset
    block_tables: List[torch.Tensor]       # per paged group: int32 [segments, max_blocks]
    num_wanted: int
    max_q_len: int
    max_kv_len: int
    kv_bucket: int = 1                     # max_kv_len in units of 256 keys, capped: picks the decode split
    multi_segments: int = -1               # segments [0, multi_segments) bring several rows, the rest one row each;
    multi_rows: int = 0                    # they cover rows [0, multi_rows); -1 = the batch is not of that form
    host_seg_start: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)

    @property
    def decode_only(self) -> bool:
        return self.max_q_len == 1


class BatchBuilder:
    def __init__(self, device, max_rows: int, max_segments: int, max_blocks: int, num_paged_groups: int,
                 page_size: int, resident_blocks: int):
        """`resident_blocks`: places for blocks of the decode attention on the device (the runner asks the device);
        a step's key-range bucket, which is part of a captured step's key, is capped by it."""
        self.device, self.resident_blocks = device, max(1, int(resident_blocks))
        self.max_rows, self.max_segments, self.max_blocks = max_rows, max_segments, max_blocks
        self.groups, self.page_size = num_paged_groups, page_size
        R, S, G = max_rows, max_segments, num_paged_groups
        # row region: token_ids, positions, row_seg, logit_rows, slots per group; then the segment region
        self._row_fields = 4 + G
        self._seg_fields = 4
        n_small = self._row_fields * R + self._seg_fields * S
        self._host_small = torch.empty(n_small, dtype=torch.int32).pin_memory() if torch.cuda.is_available() \
            else torch.empty(n_small, dtype=torch.int32)
        self._host_tables = torch.empty(max(1, G) * S * max_blocks, dtype=torch.int32)
        if torch.cuda.is_available():
            self._host_tables = self._host_tables.pin_memory()
        self._dev_small = torch.zeros(n_small, dtype=torch.int32, device=device)
        self._dev_tables = torch.zeros(max(1, G) * S * max_blocks, dtype=torch.int32, device=device)
        self._copied = torch.cuda.Event() if torch.cuda.is_available() else None
        self._np_small = self._host_small.numpy()
        self._np_tables = self._host_tables.numpy().reshape(max(1, G), S, max_blocks)
        self._p_small, self._p_tables = self._host_small.data_ptr(), self._host_tables.data_ptr()
        # the arguments of the library's calls, kept between steps
        arrays = {"ids": np.zeros(S, np.int64), "starts": np.zeros(S, np.int32), "counts": np.zeros(S, np.int32),
                  "want_at": np.zeros(S + 1, np.int32), "tokens": np.zeros(R, np.int32), "wants": np.zeros(R, np.int32),
                  "info": np.zeros(8, np.int32), "lengths": np.zeros(S, np.int32),
                  "released": np.zeros(2 * max(64, S * max_blocks * max(1, G)), np.int32)}
        self._args = dict(arrays)
        self._args.update({"p_" + k: v.ctypes.data for k, v in arrays.items()})
        self._builder = native.lib().jh_builder_new(R, S, max_blocks, G, page_size)
        self._built = 0
        self._views = {}

    def commit(self, cache) -> list:
        """After the step that was built last has been launched: every segment's request now holds its new
        positions. Returns the (group, page) pairs that windows have passed."""
        a, S = self._args, self._built
        np.add(a["starts"][:S], a["counts"][:S], out=a["lengths"][:S])
        cap = a["released"].shape[0]
        code = native.lib().jh_step_commit(cache._ptr, S, a["p_ids"], a["p_lengths"], a["p_released"], cap, a["p_info"])
        if code:
            native.check(code, cache._names)
        n = int(a["info"][0])
        if 2 * n > cap:
            raise RuntimeError(f"{n} pages released in one step, room for {cap // 2}")
        rel = a["released"]
        return [(int(rel[2 * i]), int(rel[2 * i + 1])) for i in range(n)]

    def __del__(self):
        try:
            if getattr(self, "_builder", None):
                native.lib().jh_builder_delete(self._builder)
                self._builder = None
        except Exception:        # the interpreter is shutting down and the module is gone
            pass

    def bytes_per_step(self, segments: int) -> int:
        """Bytes a step with `segments` segments copies from pinned host memory to the device."""
        return 4 * (self._dev_small.numel() + self.groups * segments * self.max_blocks)

    def _row_view(self, buf, i):
        R = self.max_rows
        return buf[i * R:(i + 1) * R]

    def _seg_view(self, buf, i):
        base = self._row_fields * self.max_rows
        S = self.max_segments
        return buf[base + i * S: base + (i + 1) * S]

    def build(self, segments: List[Segment], cache, vocab: int, reserve: bool = False) -> StepBatch:
        """Fills the tables from the segments and the cache manager's block tables. With `reserve` the pages of
        every segment are taken first, all or none (else they must have been reserved). Reserving and packing are
        the host library's (`jh_step_reserve`, `jh_builder_build`): two calls per step."""
        if self._copied is not None:
            self._copied.synchronize()     # the last step's copies have left the pinned buffers
        S = len(segments)
        if S == 0:
            raise ValueError("a step needs at least one segment")
        if S > self.max_segments:
            raise ValueError(f"{S} segments in one step, the engine was made for {self.max_segments}")
        a = self._args
        ids, starts, counts, want_at = a["ids"], a["starts"], a["counts"], a["want_at"]
        handles = cache.handles([seg.request for seg in segments])
        n_tok = n_want = 0
        single = True
        for si, seg in enumerate(segments):
            n = len(seg.tokens)
            ids[si], starts[si], counts[si], want_at[si] = handles[si], seg.start, n, n_want
            n_tok += n
            n_want += len(seg.want)
            single = single and n == 1
        want_at[S] = n_want
        if n_tok > self.max_rows:
            raise ValueError(f"{n_tok} rows in one step, the engine was made for {self.max_rows}")
        tokens, wants = a["tokens"], a["wants"]
        if n_want > wants.shape[0]:
            raise ValueError(f"{n_want} wanted places in one step, the engine was made for {wants.shape[0]}")
        try:
            if single:
                for si, seg in enumerate(segments):
                    tokens[si] = seg.tokens[0]
            else:
                at = 0
                for seg in segments:
                    n = len(seg.tokens)
                    tokens[at:at + n] = seg.tokens
                    at += n
        except OverflowError:
            raise ValueError(f"a token id outside [0, {vocab})") from None
        at = 0
        for seg in segments:
            for w in seg.want:
                wants[at] = w
                at += 1
        info = a["info"]
        if reserve:
            code = native.lib().jh_step_reserve(cache._ptr, S, a["p_ids"], a["p_starts"], a["p_counts"])
            if code:
                native.check(code, cache._names)
        code = native.lib().jh_builder_build(self._builder, cache._ptr, S, a["p_ids"], a["p_starts"], a["p_counts"],
                                             a["p_tokens"], a["p_want_at"], a["p_wants"], vocab, self._p_small,
                                             self._p_tables, a["p_info"])
        if code:
            if reserve:
                for seg in segments:
                    if cache.is_open(seg.request):
                        cache.trim(seg.request)
            native.check(code, cache._names)
        rows, n_want, max_q, max_kv, multi_segments, multi_rows = (int(v) for v in info[:6])
        self._built = S
        h = self._np_small
        sstart, sslot = self._seg_view(h, 0), self._seg_view(h, 3)
        self._dev_small.copy_(self._host_small, non_blocking=True)
        MB = self.max_blocks
        for g in range(self.groups):
            lo = g * self.max_segments * MB
            self._dev_tables[lo:lo + S * MB].copy_(self._host_tables[lo:lo + S * MB], non_blocking=True)
        if self._copied is not None:
            self._copied.record()
        views = self._views.get((rows, S, n_want))
        if views is None:       # the device views of a shape are made once: slicing tensors is the dearest thing left here
            d = self._dev_small
            dt = self._dev_tables.view(max(1, self.groups), self.max_segments, MB)
            views = dict(
                token_ids=self._row_view(d, 0)[:rows], positions=self._row_view(d, 1)[:rows],
                row_seg=self._row_view(d, 2)[:rows], logit_rows=self._row_view(d, 3)[:n_want],
                slots=[self._row_view(d, 4 + g)[:rows] for g in range(self.groups)],
                seg_start=self._seg_view(d, 0)[:S], seg_len=self._seg_view(d, 1)[:S],
                seg_kv_len=self._seg_view(d, 2)[:S], state_slots=self._seg_view(d, 3)[:S],
                block_tables=[dt[g, :S] for g in range(self.groups)])
            if len(self._views) < 4096:
                self._views[(rows, S, n_want)] = views
        return StepBatch(
            rows=rows, segments=list(segments), num_wanted=n_want, max_q_len=max_q, max_kv_len=max_kv,
            kv_bucket=max(1, min(32, max_kv // 256, -(-self.resident_blocks // rows))),
            multi_segments=multi_segments, multi_rows=multi_rows,
            host_seg_start=sstart[:S].tolist(), host_state_slots=sslot[:S].tolist(), **views)
