"""The dense gated feed-forward: x += Wdown (silu(Wgate xb) * (Wup xb)).

Formula from the reference (src/main/java/org/robomiri/jllm/cpu/CpuBackend.java:661-669,
silu at cpu/VectorKernels.java:637-639). As the reference's converter does
(model/ModelConverter.java:380-382), gate and up are stacked into one [2 * hidden, dim]
matrix at load, rows [0, hidden) gate and [hidden, 2 hidden) up, so one product feeds both.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import TensorWant
from .base import FeedForward, register_feed_forward
from .linear import Linear


class DenseGlu(FeedForward):
    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.hidden, self.dim, self.rt = spec.hidden, dim, runtime
        gate, up = tensors.pop(prefix + "gate_proj.weight"), tensors.pop(prefix + "up_proj.weight")
        # bfloat16: blocks of 8 gate rows followed by their 8 up rows, so that the product's epilogue holds a
        # gate value and its up value together and applies SwiGLU itself (no [rows, 2 hidden] round trip)
        self.fused = gate.dtype == torch.bfloat16 and dim % 8 == 0 and spec.hidden % 8 == 0
        if self.fused:
            stacked = torch.stack([gate.view(spec.hidden // 8, 8, dim), up.view(spec.hidden // 8, 8, dim)], dim=1)
            self.gate_up = Linear(stacked.reshape(2 * spec.hidden, dim).contiguous())
            del stacked
        else:
            self.gate_up = Linear(torch.cat([gate, up], dim=0).contiguous())
        del gate, up
        self.down = Linear(tensors.pop(prefix + "down_proj.weight"))

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        return {prefix + "gate_proj.weight": TensorWant((spec.hidden, dim)),
                prefix + "up_proj.weight": TensorWant((spec.hidden, dim)),
                prefix + "down_proj.weight": TensorWant((dim, spec.hidden))}

    def forward(self, xb, x, batch) -> None:
        rows = xb.shape[0]
        h = self.rt.buffer("ffn_hidden", self.hidden)[:rows]
        if self.fused:
            self.gate_up.forward(xb, h, swiglu=True)
        else:
            gate_up = self.rt.buffer("gate_up", 2 * self.hidden)[:rows]
            self.gate_up.forward(xb, gate_up)
            ops.swiglu(gate_up, h)
        self.down.forward(h, x, accumulate=True)


register_feed_forward("dense_glu", DenseGlu, replace=True)
