"""RMSNorm as a part: y = (x * (1 / sqrt(mean(x^2) + eps))) * gain.

Formula and order of the multiplications from the reference
(src/main/java/org/robomiri/jllm/cpu/VectorKernels.java:630-634,675-685). The input is the
float32 residual stream; the output has the compute dtype. The gain stays in the dtype it
was stored in (bfloat16 or float32): the kernel reads either.
"""
from __future__ import annotations

from ..csrc import ops
from ..weights.loader import TensorWant
from .base import Norm, register_norm


class RmsNorm(Norm):
    def __init__(self, spec, dim: int, tensors: dict, prefix: str, runtime):
        self.eps = float(spec.eps)
        self.dim = dim
        self.gain = tensors[prefix + "weight"]

    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        return {prefix + "weight": TensorWant((dim,), "vector", init="gain")}

    def forward(self, x, out, row_index=None, rows=None):
        ops.rmsnorm(x, self.gain, self.eps, out, row_index, rows)


register_norm("rmsnorm", RmsNorm, replace=True)
