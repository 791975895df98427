"""Weights by tensor name, checked against what the model's parts want.

Every part lists the tensors it wants (`TensorWant`: shape and role) under its checkpoint
names; `load_checked` compares that list with the file once and raises ONE error that
names every missing tensor, every wrong shape and every unexpected tensor. The reference
checks each tensor against its spec as it loads and stops at the first mismatch
(src/main/java/org/robomiri/jllm/model/ModelWeights.java:28-84, DecoderLayer.java:35-44,
AttnWeights.java:52-64); tensors it does not ask for it never looks at, and so here: they
are listed in the error when there is one, and noted otherwise.

Precision policy. `bfloat16`: tensors stay in bfloat16; a tensor stored in 32-bit stays
so if it is a vector (norm gains, biases: the kernels read either), and is rounded to
bfloat16 (nearest even) if it is a matrix that feeds the tensor cores; float16 becomes
bfloat16 (matrix) or float32 (vector). A matrix whose part needs it in 32 bits whatever the
compute dtype (a router, a state transition) is wanted with the role `matrix_fp32`. `float32`: everything is widened to float32, which
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
    role: str = "matrix"                   # matrix | matrix_fp32 | vector | int_table
    optional: bool = False
    init: str = "normal"                   # random-weights mode: normal = N(0, 0.02), gain = 1 + N(0, 0.1)


def target_dtype(stored: torch.dtype, role: str, compute: torch.dtype) -> torch.dtype:
    if role == "int_table" or not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32 or role == "matrix_fp32":
        return torch.float32
    if role == "matrix":
        return torch.bfloat16
    return torch.bfloat16 if stored == torch.bfloat16 else torch.float32


# Prefixes of multimodal checkpoints mapped onto the plain names, as the reference's converter maps them
# (model/ModelConverter.java:977-988): `language_model.model.X` and `model.language_model.X` become `model.X`,
# `language_model.lm_head.X` becomes `lm_head.X`. Other tensors of such a file (vision tower, projector) keep their
# names and are never read.
PREFIX_ALIASES = (("language_model.model.", "model."), ("model.language_model.", "model."),
                  ("language_model.lm_head.", "lm_head."))


def canonical_name(name: str) -> str:
    for prefix, plain in PREFIX_ALIASES:
        if name.startswith(prefix):
            return plain + name[len(prefix):]
    return name


def canonical_names(stored) -> Dict[str, str]:
    """{canonical name: stored name}. Two stored tensors that map onto one name are an error."""
    out: Dict[str, str] = {}
    for n in stored:
        c = canonical_name(n)
        if c in out:
            raise WeightError(f"tensors {out[c]!r} and {n!r} are both {c!r} once their prefixes are dropped")
        out[c] = n
    return out


def compare(source_meta: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]], wants: Dict[str, TensorWant], where: str,
            strict: bool = False) -> list:
    """Raises ONE WeightError that lists every missing tensor, every wrong shape and every unexpected tensor, if a
    wanted tensor is missing or has a wrong shape. Tensors that the model does not ask for are no error by
    themselves (the reference reads what it needs by name and leaves the rest alone: a tied checkpoint that still
    ships `lm_head.weight`, an old one with `rotary_emb.inv_freq`, a multimodal one with its vision tower); they
    are returned so that the caller can note them. With `strict` they are an error too."""
    missing = sorted(n for n, w in wants.items() if n not in source_meta and not w.optional)
    unexpected = sorted(n for n in source_meta if n not in wants)
    wrong = sorted((n, tuple(source_meta[n][1]), tuple(w.shape)) for n, w in wants.items()
                   if n in source_meta and tuple(source_meta[n][1]) != tuple(w.shape))
    if not (missing or wrong or (strict and unexpected)):
        return unexpected
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
                 notes: list | None = None, strict: bool = False) -> Dict[str, torch.Tensor]:
    stored = canonical_names(source.names())
    meta = {c: source.meta(n) for c, n in stored.items()}
    ignored = compare(meta, wants, str(source.dir), strict)
    if notes is not None and ignored:
        shown = ", ".join(ignored[:8]) + (f" and {len(ignored) - 8} more" if len(ignored) > 8 else "")
        notes.append(f"{len(ignored)} tensors of the checkpoint are not used by this model and were not read: {shown}")
    out = {}
    for name, want in wants.items():
        if name not in meta:
            continue
        stored_dtype = meta[name][0]
        to = target_dtype(stored_dtype, want.role, compute)
        if notes is not None and stored_dtype == torch.float32 and to == torch.bfloat16:
            notes.append(f"{name}: stored in float32, rounded to bfloat16 for the tensor-core path")
        out[name] = source.tensor(stored[name]).to(device=device, dtype=to).contiguous()
    return out


def convert_checked(tensors: Dict[str, torch.Tensor], wants: Dict[str, TensorWant], compute: torch.dtype, device):
    """The same check and policy for tensors that are in memory already (random weights made on the device)."""
    compare({n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()}, wants, "in-memory weights", strict=True)
    return {n: tensors[n].to(device=device, dtype=target_dtype(tensors[n].dtype, wants[n].role, compute)).contiguous()
            for n in wants if n in tensors}
