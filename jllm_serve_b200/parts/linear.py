"""out (+)= a @ W^T (+ bias): the matrix product every part uses, choosing the kernel by dtype and shape.

float32: always the CUDA-core kernel with true 32-bit products and sums (no tensor cores).
bfloat16: the tensor-core kernels where the shape fits them, else the same CUDA-core kernel
reading bfloat16 and summing in float32. Weights are [out, in] row-major, as stored in the
checkpoint (src/main/java/org/robomiri/jllm/cpu/CpuMatmul.java:390-396).
"""
from __future__ import annotations

import torch

from ..csrc import ops


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None):
        assert weight.dim() == 2 and weight.is_contiguous()
        self.weight, self.bias = weight, bias
        self.out_features, self.in_features = weight.shape

    def forward(self, a: torch.Tensor, out: torch.Tensor, accumulate: bool = False, swiglu: bool = False) -> None:
        """a [rows, in] (compute dtype) -> out [rows, out]; `accumulate` adds into out (the float32 residual);
        `swiglu`: the weight's rows are interleaved gate / up blocks and out is [rows, out / 2]."""
        if a.shape[0] == 0:
            return
        if self.weight.dtype == torch.bfloat16 and ops.gemm_bf16_fits(a, self.weight, out):
            ops.gemm_bf16(a, self.weight, out, self.bias, accumulate, swiglu)
        elif swiglu:
            raise ops.KernelError("the fused SwiGLU epilogue exists in the tensor-core kernels only")
        else:
            ops.gemm_plain(a, self.weight, out, self.bias, accumulate)
