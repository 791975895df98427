"""Decoding parameters, with the reference's names, meanings, defaults and checks.

src/main/java/org/robomiri/jllm/sampling/SamplingParams.java:19-44 (fields and validation) and
src/main/resources/jllm.properties:191-204 (defaults: temperature 0.6, top-k 20, top-p 0.95,
min-p 0, seed -1, max-tokens 1024). Penalties, logit bias, stop strings and constraints need
a tokenizer or token history that this engine does not carry and are not built.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.6               # 0 means greedy (argmax)
    top_k: int = 20                        # 0 disables top-k; 1 means greedy
    top_p: float = 0.95                    # 1 disables nucleus sampling
    min_p: float = 0.0                     # 0 disables; keep tokens with p >= min_p * p_max
    seed: int = -1                         # -1 for a random seed
    max_tokens: int = 1024                 # most generated tokens
    ignore_eos: bool = False               # benchmarks: keep going past a stop token
    stop_token_ids: Tuple[int, ...] = ()   # besides the model's eos ids

    def __post_init__(self):
        for name in ("temperature", "top_p", "min_p"):
            if not math.isfinite(float(getattr(self, name))):
                raise ValueError(f"sampling parameters must be finite numbers: {self.describe()}")
        if self.temperature < 0 or self.top_k < 0 or self.top_p <= 0 or self.top_p > 1 or self.min_p < 0 \
                or self.min_p > 1:
            raise ValueError("invalid sampling parameters (temperature >= 0, top_k >= 0, 0 < top_p <= 1, "
                             f"0 <= min_p <= 1): {self.describe()}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be at least 1, got {self.max_tokens}")

    def describe(self) -> str:
        return (f"temperature={self.temperature}, top_k={self.top_k}, top_p={self.top_p}, min_p={self.min_p}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0 or self.top_k == 1

    @classmethod
    def greedy_params(cls, max_tokens: int = 1024, **kw) -> "SamplingParams":
        return cls(temperature=0.0, top_k=0, top_p=1.0, max_tokens=max_tokens, **kw)
