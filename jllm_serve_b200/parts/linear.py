"""out (+)= a @ W^T (+ bias): the matrix product every part uses, choosing the kernel by dtype and shape.

float32: always the CUDA-core kernel with true 32-bit products and sums (no tensor cores).
bfloat16: the tensor-core kernels where the shape fits them (K a multiple of 8), else the same CUDA-core kernel
reading bfloat16 and summing in float32. Weights are [out, in] row-major in the checkpoint
(src/main/java/org/robomiri/jllm/cpu/CpuMatmul.java:390-396); for the tensor-core kernels a bfloat16 weight is
PACKED once, when the part is built (`ops.pack_weight`: tiles of 128 rows x 64 k in the shared-memory image the
tensor cores read, so a tile is one contiguous bulk copy), and the row-major copy is let go.
"""
from __future__ import annotations

import torch

from ..csrc import ops


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, keep_plain: bool = False):
        """`keep_plain`: the row-major matrix stays beside the packed one (it is someone else's too: an embedding
        table that serves as the head is gathered row by row)."""
        assert weight.dim() == 2 and weight.is_contiguous()
        self.bias = bias
        self.out_features, self.in_features = weight.shape
        self.packed = None
        if weight.dtype == torch.bfloat16 and weight.is_cuda and self.in_features % 8 == 0 and self.in_features >= 8:
            self.packed = ops.pack_weight(weight)
        self.weight = weight if (self.packed is None or keep_plain) else None

    def rows(self, lo: int, hi: int) -> "Linear":
        """The product with rows [lo, hi) of the weight only (a view where the packed tiles allow it, else a copy)."""
        bias = self.bias[lo:hi] if self.bias is not None else None
        if self.packed is None:
            return Linear(self.weight[lo:hi].contiguous(), bias)
        out = Linear.__new__(Linear)
        out.bias, out.out_features, out.in_features, out.weight = bias, hi - lo, self.in_features, None
        if lo % 128 == 0:
            out.packed = ops.PackedWeight(self.packed.data[lo // 128: -(-hi // 128)], hi - lo, self.in_features)
        else:
            out.packed = ops.pack_weight(self.packed.unpack()[lo:hi].contiguous())
        return out

    def forward(self, a: torch.Tensor, out: torch.Tensor, accumulate: bool = False, swiglu: bool = False) -> None:
        """a [rows, in] (compute dtype) -> out [rows, out]; `accumulate` adds into out (the float32 residual);
        `swiglu`: the weight's rows are interleaved gate / up blocks and out is [rows, out / 2]."""
        if a.shape[0] == 0:
            return
        if self.packed is not None and ops.gemm_bf16_fits(a, self.packed, out):
            ops.gemm_bf16(a, self.packed, out, self.bias, accumulate, swiglu)
        elif swiglu:
            raise ops.KernelError("the fused SwiGLU epilogue exists in the tensor-core kernels only")
        else:
            weight = self.weight if self.weight is not None else self.packed.unpack()
            ops.gemm_plain(a, weight, out, self.bias, accumulate)
