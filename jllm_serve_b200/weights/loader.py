"""Weights by tensor name, checked against what the model's parts want.

Every part lists the tensors it wants (`TensorWant`: shape and role) under its checkpoint
names; `load_checked` compares that list with the file once and raises ONE error that
names every missing tensor, every unexpected tensor and every wrong shape. The reference
checks each tensor against its spec as it loads and stops at the first mismatch
(src/main/java/org/robomiri/jllm/model/ModelWeights.java:28-84, DecoderLayer.java:35-44,
AttnWeights.java:52-64).

Precision policy. `bfloat16`: tensors stay in bfloat16; a tensor stored in 32-bit stays
so if it is a vector (norm gains, biases: the kernels read either), and is rounded to
bfloat16 (nearest even) if it is a matrix that feeds the tensor cores; float16 becomes
bfloat16 (matrix) or float32 (vector). `float32`: everything is widened to float32, which
is exact for bfloat16 and float16. Integer tables become int32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch

from .safetensors_io import TensorSource


class WeightError(ValueError):
    """The checkpoint does not fit the configuration; the message lists every difference."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)


@dataclass(frozen=True)
class TensorWant:
    shape: Tuple[int, ...]
    role: str = "matrix"                   # matrix | vector | int_table
    optional: bool = False
    init: str = "normal"                   # random-weights mode: normal = N(0, 0.02), gain = 1 + N(0, 0.1)


def target_dtype(stored: torch.dtype, role: str, compute: torch.dtype) -> torch.dtype:
    if role == "int_table" or not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if role == "matrix":
        return torch.bfloat16
    return torch.bfloat16 if stored == torch.bfloat16 else torch.float32


def compare(source_meta: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]], wants: Dict[str, TensorWant], where: str):
    """Raises WeightError if the names or shapes differ; returns nothing otherwise."""
    missing = sorted(n for n, w in wants.items() if n not in source_meta and not w.optional)
    unexpected = sorted(n for n in source_meta if n not in wants)
    wrong = sorted((n, tuple(source_meta[n][1]), tuple(w.shape)) for n, w in wants.items()
                   if n in source_meta and tuple(source_meta[n][1]) != tuple(w.shape))
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not match the configuration"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): "
                     + ", ".join(f"{n} is {list(has)}, config wants {list(want)}" for n, has, want in wrong))
    raise WeightError("\n".join(lines), missing, unexpected, wrong)


def load_checked(source: TensorSource, wants: Dict[str, TensorWant], compute: torch.dtype, device,
                 notes: list | None = None) -> Dict[str, torch.Tensor]:
    meta = {n: source.meta(n) for n in source.names()}
    compare(meta, wants, str(source.dir))
    out = {}
    for name, want in wants.items():
        if name not in meta:
            continue
        stored = meta[name][0]
        to = target_dtype(stored, want.role, compute)
        if notes is not None and stored == torch.float32 and to == torch.bfloat16:
            notes.append(f"{name}: stored in float32, rounded to bfloat16 for the tensor-core path")
        out[name] = source.tensor(name).to(device=device, dtype=to).contiguous()
    return out


def convert_checked(tensors: Dict[str, torch.Tensor], wants: Dict[str, TensorWant], compute: torch.dtype, device):
    """The same check and policy for tensors that are in memory already (random weights made on the device)."""
    compare({n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()}, wants, "in-memory weights")
    return {n: tensors[n].to(device=device, dtype=target_dtype(tensors[n].dtype, wants[n].role, compute)).contiguous()
            for n in wants if n in tensors}
