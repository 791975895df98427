"""Choosing next tokens for a batch of logits rows on the device.

Greedy rows take the argmax (lowest index among equal maxima, as
src/main/java/org/robomiri/jllm/sampling/Sampler.java:458-466); the others are drawn by the
sampling kernel from one uniform number per row and step. The uniform numbers come from a
host generator per request, seeded by the request's seed, so a fixed seed gives the same
tokens whatever else is in the batch.
"""
from __future__ import annotations

import os
import random
from typing import List, Sequence

import torch

from ..csrc import ops
from .params import SamplingParams


class RequestRng:
    """The stream of uniform numbers of one request."""

    def __init__(self, seed: int):
        self.seed = seed if seed >= 0 else int.from_bytes(os.urandom(8), "little") >> 1
        self._rng = random.Random(self.seed)

    def next(self) -> float:
        return self._rng.random()


class Sampler:
    def __init__(self, device, max_rows: int, vocab: int, sample_vocab: int | None = None):
        self.device, self.max_rows, self.vocab = device, max_rows, vocab
        self.sample_vocab = min(vocab, sample_vocab or vocab)  # ids at or above it are never drawn (padding rows)
        pin = torch.cuda.is_available()
        self._host_f = torch.empty((3, max_rows), dtype=torch.float32, pin_memory=pin)   # temperature, top_p, min_p
        self._host_k = torch.empty(max_rows, dtype=torch.int32, pin_memory=pin)
        self._host_u = torch.empty(max_rows, dtype=torch.float64, pin_memory=pin)
        self._f = torch.empty((3, max_rows), dtype=torch.float32, device=device)
        self._k = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._u = torch.empty(max_rows, dtype=torch.float64, device=device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.empty(max_rows, dtype=torch.int32).pin_memory()
        self._out_host_np = self._out_host.numpy()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], uniforms: Sequence[float]) -> List[int]:
        """logits float32 [n, vocab] on the device -> n token ids on the host."""
        n = logits.shape[0]
        if n == 0:
            return []
        assert n <= self.max_rows and len(params) == n
        out = self._out[:n]
        if all(p.greedy for p in params):
            ops.argmax(logits, out, self.sample_vocab)
        else:
            for i, p in enumerate(params):
                self._host_f[0, i], self._host_f[1, i], self._host_f[2, i] = p.temperature, p.top_p, p.min_p
                self._host_k[i] = p.top_k
                self._host_u[i] = uniforms[i]
            self._f.copy_(self._host_f, non_blocking=True)
            self._k.copy_(self._host_k, non_blocking=True)
            self._u.copy_(self._host_u, non_blocking=True)
            ops.sample(logits, self._f[0, :n], self._k[:n], self._f[1, :n], self._f[2, :n], self._u[:n], out,
                       self.sample_vocab)
        self._out_host.copy_(self._out, non_blocking=True)     # all of the small buffer: no views to make
        torch.cuda.current_stream().synchronize()
        return self._out_host_np[:n].tolist()
