"""Grouped-query causal attention over the paged cache, with optional per-head q/k RMSNorm and RoPE.

Order of operations from the reference (src/main/java/org/robomiri/jllm/cpu/CpuBackend.java:
422-458,595-615): q, k, v projections (biases if configured); RMSNorm of every query and key
head with the shared gains `q_norm` / `k_norm`; rotation; keys and values into the cache;
attention of every row over its request's keys [first, position]; `x += att @ Wo^T`.
Query head h reads kv head h // (heads / kv_heads) (cpu/KvCache.java:82,527). q, k and v
are one stacked [Q + 2 KV, dim] matrix, as the reference's fused `matmul3`.

A run that reads another run's cache (`cache.writes == False`) projects queries only.
"""
from __future__ import annotations

import torch

from ..cache.manager import PagedKeysValues
from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Mixer, register_mixer
from .linear import Linear


class GqaAttention(Mixer):
    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime, rope=None):
        self.spec, self.dim, self.rt, self.rope = spec, dim, runtime, rope
        H, Hkv, hd = spec.heads, spec.kv_heads, spec.head_dim
        self.q_width, self.kv_width = H * hd, Hkv * hd
        names = ("q_proj", "k_proj", "v_proj")
        w = [tensors.pop(prefix + n + ".weight") for n in names]
        b = [tensors.pop(prefix + n + ".bias") for n in names] if spec.bias else None
        self.qkv = Linear(torch.cat(w, dim=0).contiguous(), torch.cat(b).contiguous() if b else None)
        self._q_only = None          # the query rows alone, made when a run first reads another run's cache
        del w, b
        self.out = Linear(tensors.pop(prefix + "o_proj.weight"),
                          tensors.pop(prefix + "o_proj.bias") if spec.out_bias else None)
        self.q_gain = tensors.pop(prefix + "q_norm.weight") if spec.qk_norm else None
        self.k_gain = tensors.pop(prefix + "k_norm.weight") if spec.qk_norm else None
        if rope is not None and rope.rotary_dim > hd:
            raise ValueError(f"rotary_dim={rope.rotary_dim} exceeds head_dim={hd}")

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        H, Hkv, hd = spec.heads, spec.kv_heads, spec.head_dim
        out = {prefix + "q_proj.weight": TensorWant((H * hd, dim)),
               prefix + "k_proj.weight": TensorWant((Hkv * hd, dim)),
               prefix + "v_proj.weight": TensorWant((Hkv * hd, dim)),
               prefix + "o_proj.weight": TensorWant((dim, H * hd))}
        if spec.bias:
            out.update({prefix + "q_proj.bias": TensorWant((H * hd,), "vector"),
                        prefix + "k_proj.bias": TensorWant((Hkv * hd,), "vector"),
                        prefix + "v_proj.bias": TensorWant((Hkv * hd,), "vector")})
        if spec.out_bias:
            out[prefix + "o_proj.bias"] = TensorWant((dim,), "vector")
        if spec.qk_norm:
            out[prefix + "q_norm.weight"] = TensorWant((hd,), "vector", init="gain")
            out[prefix + "k_norm.weight"] = TensorWant((hd,), "vector", init="gain")
        return out

    @classmethod
    def cache_need(cls, spec):
        return PagedKeysValues(spec.kv_heads, spec.head_dim, spec.window)

    def decode_bucket_cap(self, rows: int) -> int:
        s = self.spec
        if not ops.attention_decode_fits(self.rt.dtype, s.heads, s.kv_heads, s.head_dim):
            return 1                   # the plain attention's launches do not depend on the context
        scratch = self.rt.buffer("attention_scratch", 2 << 20, torch.float32, rows=1)[0]
        return ops.decode_bucket_cap(rows, s.kv_heads, s.heads, s.head_dim, s.window, scratch)

    def forward(self, xb, x, batch, cache) -> None:
        s, rows = self.spec, xb.shape[0]
        if cache.writes:
            qkv = self.rt.buffer("qkv", self.q_width + 2 * self.kv_width)[:rows]
            self.qkv.forward(xb, qkv)
        else:
            qkv = self.rt.buffer("q_only", self.q_width)[:rows]
            if self._q_only is None:
                self._q_only = self.qkv.rows(0, self.q_width)
            self._q_only.forward(xb, qkv)
        rope = self.rope
        att = self.rt.buffer("attention_out", self.q_width)[:rows]
        scratch = self.rt.buffer("attention_scratch", 2 << 20, torch.float32, rows=1)[0]
        if (cache.writes and batch.decode_only and rope is not None and ops.attention_decode_fits(qkv.dtype, s.heads, s.kv_heads, s.head_dim)
                and ops.attention_decode_fresh_fits(qkv.dtype, s.heads, s.kv_heads, s.head_dim, rope.rotary_dim)):
            # a step of single rows: the attention kernel norms and rotates its own rows and writes their keys and values
            # (where that pays: it says whether it ran)
            if ops.attention_decode_fresh(qkv, self.q_gain, self.k_gain, s.qk_norm_eps, rope.cos, rope.sin, cache.keys,
                                          cache.values, att, batch.row_seg, batch.positions,
                                          batch.block_tables[cache.group], rows, s.heads, s.kv_heads, s.head_dim,
                                          self.rt.page_size, s.window, s.scale, batch.kv_bucket, scratch):
                return self.out.forward(att, x, accumulate=True)
        ops.qk_norm_rope_store(qkv, self.q_gain, self.k_gain, s.qk_norm_eps,
                               rope.cos if rope else None, rope.sin if rope else None,
                               rope.rotary_dim if rope else 0, batch.positions,
                               batch.slots[cache.group] if cache.writes else None, cache.keys, cache.values,
                               s.heads, s.kv_heads, s.head_dim, self.rt.page_size, write_kv=cache.writes)
        ops.attention(qkv, cache.keys, cache.values, att, batch, cache.group, s.heads, s.kv_heads, s.head_dim,
                      self.rt.page_size, s.window, s.scale, scratch)
        self.out.forward(att, x, accumulate=True)


register_mixer("gqa_attention", GqaAttention, replace=True)
