"""The generic decoder: embedding, the scheduled layer runs, final norm and head, built from parts.

The model is what a registry entry builds from a `Decoder` spec. It knows the order of
layer runs (data: `spec.schedule`), hands every run the cache it reads or writes, and
computes logits only for the rows that were asked for, as the reference does
(src/main/java/org/robomiri/jllm/cpu/CpuBackend.java:895-928,980-985). The head is the
embedding when `tie_word_embeddings` is set (a `lm_head.weight` that the file still has is
left unread, as the reference's converter drops it: model/ModelConverter.java:663-665), else
`lm_head.weight`, and the embedding again if the file has none (model/ModelWeights.java:37).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.specs import Decoder
from ..csrc import ops
from ..parts import Linear, RunCache, Runtime, part_class
from ..weights.loader import TensorWant


class DecoderModel:
    def __init__(self, spec: Decoder, tensors: Dict[str, torch.Tensor], runtime: Runtime):
        self.spec, self.rt = spec, runtime
        core, names = spec.core, spec.names
        tensors = dict(tensors)
        self.embedding = tensors.pop(names.embedding)
        head = None if core.tied else tensors.pop(names.head, None)
        if head is None and not core.tied:
            runtime.notes.append(f"{names.head} is not in the checkpoint: the embedding serves as the head")
        self.head = Linear(self.embedding, keep_plain=True) if head is None else Linear(head)
        self.position_encodings = []
        for t in spec.rope_tables:
            cls = part_class("position", t.kind)
            extra = {"tensors": tensors, "dim": core.dim} if cls.wants(t, core.dim, "") else {}
            self.position_encodings.append(cls(t, runtime.max_positions, runtime.device, **extra))
        self.blocks = []
        for l, layer in enumerate(spec.layers):
            cls = part_class("block", layer.arrangement)
            self.blocks.append(cls(layer, core.dim, tensors, names.layer.format(l), runtime, self.position_encodings))
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm, core.dim, tensors,
                                                                   names.final_norm, runtime)
        self.vocab, self.dim = core.vocab, core.dim

    @classmethod
    def wants(cls, spec: Decoder) -> Dict[str, TensorWant]:
        core, names = spec.core, spec.names
        out = {names.embedding: TensorWant((core.vocab, core.dim))}
        if not core.tied:
            out[names.head] = TensorWant((core.vocab, core.dim), optional=True)
        for t in spec.rope_tables:
            out.update(part_class("position", t.kind).wants(t, core.dim, ""))
        for l, layer in enumerate(spec.layers):
            out.update(part_class("block", layer.arrangement).wants(layer, core.dim, names.layer.format(l)))
        out.update(part_class("norm", spec.final_norm.kind).wants(spec.final_norm, core.dim, names.final_norm))
        return out

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model may be captured once and replayed: every part says so of itself."""
        return all(b.graph_safe for b in self.blocks) and all(pe.graph_safe for pe in self.position_encodings)

    def decode_bucket_cap(self, rows: int) -> int:
        """The bucket from which on a decode step of `rows` rows no longer changes its launches: the largest the parts name."""
        return max([getattr(b, "decode_bucket_cap", lambda _: 32)(rows) for b in self.blocks] or [1])

    def cache_needs(self) -> List[Optional[object]]:
        """One entry per scheduled run: what it keeps between steps (None if it reads another run's cache; a
        tuple if the mixer keeps several things, say paged keys and values and a state of fixed size)."""
        needs = []
        for run in self.spec.schedule:
            mixer = self.spec.layers[run.layer].mixer
            needs.append(None if run.cache_of is not None else part_class("mixer", mixer.kind).cache_need(mixer))
        return needs

    def _run_cache(self, cache, i: int) -> RunCache:
        run = self.spec.schedule[i]
        owner = i if run.cache_of is None else run.cache_of
        out = RunCache(owner, run.cache_of is None)
        if owner in cache.paged_of_run:
            out.group = cache.paged_of_run[owner]
            out.keys, out.values = cache.keys_values(owner)
        states = cache.states(owner)
        if states:
            out.states, out.state = tuple(states), states[0]
        return out

    def forward(self, batch, cache, logits_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the batch's rows through every scheduled layer; returns float32 logits [wanted rows, vocab]."""
        rows = batch.rows
        x = self.rt.buffer("residual", self.dim, torch.float32)[:rows]
        ops.embed_rows(batch.token_ids, self.embedding, x)
        for pe in self.position_encodings:
            pe.on_embedding(x, batch)
        for i, run in enumerate(self.spec.schedule):
            self.blocks[run.layer].forward(x, batch, self._run_cache(cache, i))
        n = batch.num_wanted
        if logits_out is None:
            logits_out = torch.empty((n, self.vocab), dtype=torch.float32, device=self.rt.device)
        if n == 0:
            return logits_out[:0]
        hb = self.rt.buffer("head_in", self.dim)[:n]
        self.final_norm.forward(x, hb, row_index=batch.logit_rows, rows=n)
        self.head.forward(hb, logits_out[:n])
        return logits_out[:n]


def build_model(entry, spec, tensors, runtime):
    """What the registry's entry builds: its own builder, else the generic decoder."""
    return (entry.build or DecoderModel)(spec, tensors, runtime)


def model_wants(entry, spec) -> Dict[str, TensorWant]:
    builder = entry.build or DecoderModel
    return builder.wants(spec)
