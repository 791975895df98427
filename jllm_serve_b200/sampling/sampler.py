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


class Ticket:
    """A launched sampling whose tokens the host has not read yet."""

    def __init__(self, slot: int, rows: int, device_tokens: torch.Tensor, done):
        self.slot, self.rows, self.device_tokens, self.done = slot, rows, device_tokens, done


class Sampler:
    """`launch` starts the choice of a step's tokens on the device and their copy to pinned host memory and returns at
    once; `fetch` waits for that copy and gives the tokens. Two sets of buffers take turns, so the tokens of one step
    can be on their way (and be fed into the next step on the device, `Ticket.device_tokens`) while the next step's
    sampling is launched. `sample` is the two in one."""

    def __init__(self, device, max_rows: int, vocab: int, sample_vocab: int | None = None):
        self.device, self.max_rows, self.vocab = device, max_rows, vocab
        self.sample_vocab = min(vocab, sample_vocab or vocab)  # ids at or above it are never drawn (padding rows)
        pin = torch.cuda.is_available()
        self._sets = []
        for _ in range(2):
            host_out = torch.empty(max_rows, dtype=torch.int32, pin_memory=pin)
            self._sets.append(dict(
                host_f=torch.empty((3, max_rows), dtype=torch.float32, pin_memory=pin),   # temperature, top_p, min_p
                host_k=torch.empty(max_rows, dtype=torch.int32, pin_memory=pin),
                host_u=torch.empty(max_rows, dtype=torch.float64, pin_memory=pin),
                f=torch.empty((3, max_rows), dtype=torch.float32, device=device),
                k=torch.empty(max_rows, dtype=torch.int32, device=device),
                u=torch.empty(max_rows, dtype=torch.float64, device=device),
                out=torch.zeros(max_rows, dtype=torch.int32, device=device),
                host_out=host_out, host_out_np=host_out.numpy(),
                done=torch.cuda.Event() if pin else None))
        self._next = 0

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], uniforms: Sequence[float]) -> Ticket:
        """logits float32 [n, vocab] on the device; nothing is waited for."""
        n = logits.shape[0]
        assert n <= self.max_rows and len(params) == n
        b = self._sets[self._next]
        slot, self._next = self._next, self._next ^ 1
        if n > 0:
            out = b["out"][:n]
            if all(p.greedy for p in params):
                ops.argmax(logits, out, self.sample_vocab)
            else:
                hf, hk, hu = b["host_f"], b["host_k"], b["host_u"]
                for i, p in enumerate(params):
                    hf[0, i], hf[1, i], hf[2, i] = p.temperature, p.top_p, p.min_p
                    hk[i] = p.top_k
                    hu[i] = uniforms[i]
                b["f"].copy_(hf, non_blocking=True)
                b["k"].copy_(hk, non_blocking=True)
                b["u"].copy_(hu, non_blocking=True)
                ops.sample(logits, b["f"][0, :n], b["k"][:n], b["f"][1, :n], b["f"][2, :n], b["u"][:n], out, self.sample_vocab)
            b["host_out"].copy_(b["out"], non_blocking=True)     # all of the small buffer: no views to make
            b["done"].record()
        return Ticket(slot, n, b["out"], b["done"])

    def fetch(self, ticket: Ticket) -> List[int]:
        if ticket.rows == 0:
            return []
        ticket.done.synchronize()
        return self._sets[ticket.slot]["host_out_np"][:ticket.rows].tolist()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], uniforms: Sequence[float]) -> List[int]:
        """logits float32 [n, vocab] on the device -> n token ids on the host."""
        return self.fetch(self.launch(logits, params, uniforms))
