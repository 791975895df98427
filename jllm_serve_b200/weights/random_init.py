"""Random weights from a configuration and a seed.

The reference has no random mode in the engine; its tiny test checkpoints come from a
script that writes a safetensors file (scripts/make-tiny-model.py:1-75). Here the mode is
part of the framework: matrices and biases are N(0, 0.02), norm gains 1 + N(0, 0.1), every
tensor drawn from a generator seeded by (seed, tensor name), so a tensor's values do not
depend on which other tensors exist. `write_model_folder` writes config.json and
model.safetensors; `random_tensors` makes the tensors in memory on any device (a model of
several GB never has to pass through a file).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict

import torch

from .loader import TensorWant
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
GAIN_STD = 0.1


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(wants: Dict[str, TensorWant], seed: int, device="cpu", dtype: torch.dtype = torch.bfloat16,
                   vector_dtype: torch.dtype | None = None) -> Dict[str, torch.Tensor]:
    """One tensor per wanted name (optional ones included), stored as `dtype` (vectors as `vector_dtype`)."""
    out = {}
    gen = torch.Generator(device=device)
    for name, want in wants.items():
        gen.manual_seed(_seed_for(seed, name))
        t = torch.randn(want.shape, generator=gen, device=device, dtype=torch.float32)
        t = t * GAIN_STD + 1.0 if want.init == "gain" else t * MATRIX_STD
        to = (vector_dtype or dtype) if want.role == "vector" else dtype
        out[name] = t.to(torch.int32) if want.role == "int_table" else t.to(to)
    return out


def write_model_folder(config: dict, seed: int, out_dir, dtype: torch.dtype = torch.bfloat16,
                       vector_dtype: torch.dtype | None = None) -> Path:
    """config.json + model.safetensors of random weights for `config` (a dict with the architecture's own keys)."""
    from ..config.registry import architecture_entry, parse_config
    from ..engine.model import model_wants

    spec = parse_config(config)
    wants = model_wants(architecture_entry(config["model_type"]), spec)
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "config.json").write_text(json.dumps(config, indent=2))
    tensors = random_tensors(wants, seed, "cpu", dtype, vector_dtype)
    write_safetensors(out_dir / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return out_dir
