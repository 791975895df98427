"""The arrangement of one layer: which norm feeds which part, and where results are added.

`pre_norm` is the reference's layer loop (src/main/java/org/robomiri/jllm/cpu/CpuBackend.java:
959-969): x += mixer(norm(x)); x += feed_forward(norm(x)), no norms after the parts. The
residual stream x is float32 in both precisions; the parts add into it themselves (the add
is the epilogue of their last matrix product).
"""
from __future__ import annotations

from .base import Block, part_class, register_block


class PreNormBlock(Block):
    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime, position_encodings):
        names = spec.names
        norm_cls = part_class("norm", spec.norm.kind)
        self.rt, self.dim = runtime, dim
        self.mixer_norm = norm_cls(spec.norm, dim, tensors, prefix + names.mixer_norm, runtime)
        self.ffn_norm = norm_cls(spec.norm, dim, tensors, prefix + names.feed_forward_norm, runtime)
        mixer_cls = part_class("mixer", spec.mixer.kind)
        table = getattr(spec.mixer, "rope_table", -1)
        extra = {"rope": position_encodings[table]} if table is not None and table >= 0 and position_encodings else {}
        self.mixer = mixer_cls(spec.mixer, dim, tensors, prefix + names.mixer, runtime, **extra)
        self.feed_forward = part_class("feed_forward", spec.feed_forward.kind)(
            spec.feed_forward, dim, tensors, prefix + names.feed_forward, runtime)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in (self.mixer_norm, self.ffn_norm, self.mixer, self.feed_forward))

    def decode_bucket_cap(self, rows: int) -> int:
        # (norms and feed-forwards do not look at the bucket; a mixer that does not say gets the safe answer)
        return getattr(self.mixer, "decode_bucket_cap", lambda _: 32)(rows)

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        names = spec.names
        norm_cls = part_class("norm", spec.norm.kind)
        out = {}
        out.update(norm_cls.wants(spec.norm, dim, prefix + names.mixer_norm))
        out.update(norm_cls.wants(spec.norm, dim, prefix + names.feed_forward_norm))
        out.update(part_class("mixer", spec.mixer.kind).wants(spec.mixer, dim, prefix + names.mixer))
        out.update(part_class("feed_forward", spec.feed_forward.kind).wants(spec.feed_forward, dim,
                                                                            prefix + names.feed_forward))
        return out

    def forward(self, x, batch, cache) -> None:
        xb = self.rt.buffer("normed", self.dim)[:x.shape[0]]
        self.mixer_norm.forward(x, xb)
        self.mixer.forward(xb, x, batch, cache)
        self.ffn_norm.forward(x, xb)
        self.feed_forward.forward(xb, x, batch)


register_block("pre_norm", PreNormBlock, replace=True)
