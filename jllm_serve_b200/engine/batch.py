"""One step's batch: which tokens of which requests run, and the device tables the kernels read.

A step is a list of segments. A segment is a request's next tokens: a portion of its prompt
or one decoded token; the reference calls it `Segment(owner, tokens, off, n, pos, logits,
stride)` (src/main/java/org/robomiri/jllm/model/Backend.java:138-153). All rows of all
segments are laid side by side, segment after segment; row-wise kernels see one batch of
`rows` rows, the attention kernels see per-row (segment, position) and per-segment tables.

`BatchBuilder` owns one pinned host buffer and one device buffer of fixed size, so the
device addresses never change (a captured decode step can be replayed) and a step costs
two host-to-device copies.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Sequence

import numpy as np
import torch


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
                 page_size: int):
        self.device = device
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
        # what each row of the host tables holds: (request, its table epoch, entries written)
        self._table_rows = [[None] * S for _ in range(max(1, G))]

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

    def build(self, segments: List[Segment], cache, vocab: int) -> StepBatch:
        """Fills the tables from the segments and the cache manager's block tables (pages must be reserved)."""
        if self._copied is not None:
            self._copied.synchronize()     # the last step's copies have left the pinned buffers
        S = len(segments)
        if S == 0:
            raise ValueError("a step needs at least one segment")
        if S > self.max_segments:
            raise ValueError(f"{S} segments in one step, the engine was made for {self.max_segments}")
        rows = sum(len(s.tokens) for s in segments)
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows in one step, the engine was made for {self.max_rows}")
        seen = set()
        h = self._np_small
        tok, pos, rseg, lrows = (self._row_view(h, i) for i in range(4))
        slot_views = [self._row_view(h, 4 + g) for g in range(self.groups)]
        sstart, slen, skv, sslot = (self._seg_view(h, i) for i in range(4))
        r = 0
        n_want = 0
        max_q = max_kv = 0
        multi_segments, multi_rows, ordered = 0, 0, True
        ps = self.page_size
        for si, seg in enumerate(segments):
            n = len(seg.tokens)
            if n < 1:
                raise ValueError(f"request {seg.request!r}: a segment needs at least one token")
            if seg.request in seen:
                raise ValueError(f"request {seg.request!r} appears twice in one step")
            seen.add(seg.request)
            if n == 1:
                t0 = int(seg.tokens[0])
                if not 0 <= t0 < vocab:
                    raise ValueError(f"request {seg.request!r}: token id outside [0, {vocab})")
                tok[r], pos[r], rseg[r] = t0, seg.start, si
            else:
                t = np.asarray(seg.tokens, dtype=np.int64)
                if t.min() < 0 or t.max() >= vocab:
                    raise ValueError(f"request {seg.request!r}: token id outside [0, {vocab})")
                tok[r:r + n] = t
                p = np.arange(seg.start, seg.start + n, dtype=np.int32)
                pos[r:r + n] = p
                rseg[r:r + n] = si
            sstart[si], slen[si], skv[si] = r, n, seg.start + n
            sslot[si] = cache.state_slot(seg.request)
            for w in seg.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {seg.request!r}: wanted place {w} is outside its {n} tokens")
                lrows[n_want] = r + w
                n_want += 1
            epoch = cache.table_epoch(seg.request) if self.groups else 0
            for g in range(self.groups):
                table = cache.table(seg.request, g)
                nb = len(table)
                if nb > self.max_blocks:
                    raise ValueError(f"request {seg.request!r} holds {nb} pages, tables have {self.max_blocks} columns")
                # the row of the host table: only what the request's table grew by since this row was last
                # written for it, if nothing else about the table changed (its epoch)
                held = self._table_rows[g][si]
                lo = held[2] if held is not None and held[0] == seg.request and held[1] == epoch and held[2] <= nb else 0
                if lo < nb:
                    self._np_tables[g, si, lo:nb] = table[lo:nb]
                self._table_rows[g][si] = (seg.request, epoch, nb)
                if n == 1:
                    slot_views[g][r] = table[seg.start // ps] * ps + seg.start % ps
                else:
                    slot_views[g][r:r + n] = self._np_tables[g, si, :nb][p // ps] * ps + p % ps
            if n > 1:
                ordered = ordered and multi_segments == si       # no single-row segment came before it
                multi_segments, multi_rows = si + 1, r + n
            r += n
            max_q = max(max_q, n)
            max_kv = max(max_kv, seg.start + n)
        self._dev_small.copy_(self._host_small, non_blocking=True)
        MB = self.max_blocks
        for g in range(self.groups):
            lo = g * self.max_segments * MB
            self._dev_tables[lo:lo + S * MB].copy_(self._host_tables[lo:lo + S * MB], non_blocking=True)
        if self._copied is not None:
            self._copied.record()
        d = self._dev_small
        dt = self._dev_tables.view(max(1, self.groups), self.max_segments, MB)
        return StepBatch(
            rows=rows, segments=list(segments),
            token_ids=self._row_view(d, 0)[:rows], positions=self._row_view(d, 1)[:rows],
            row_seg=self._row_view(d, 2)[:rows], logit_rows=self._row_view(d, 3)[:n_want],
            slots=[self._row_view(d, 4 + g)[:rows] for g in range(self.groups)],
            seg_start=self._seg_view(d, 0)[:S], seg_len=self._seg_view(d, 1)[:S], seg_kv_len=self._seg_view(d, 2)[:S],
            state_slots=self._seg_view(d, 3)[:S],
            block_tables=[dt[g, :S] for g in range(self.groups)],
            num_wanted=n_want, max_q_len=max_q, max_kv_len=max_kv,
            kv_bucket=max(1, min(32, max_kv // 256, -(-296 // rows))),
            multi_segments=multi_segments if ordered else -1, multi_rows=multi_rows,
            host_seg_start=[int(v) for v in sstart[:S]], host_state_slots=[int(v) for v in sslot[:S]])
