"""Reading and writing safetensors files, without any library for the format.

File = u64 little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}
(plus an optional "__metadata__"), then the raw little-endian data. The checks are the
reference's (src/main/java/org/robomiri/jllm/safetensors/SafeTensors.java:269-362): header
length sanity, known dtype, well-formed entry, no negative dimension, byte count equal to
shape x element size, no duplicate name, no overlapping ranges. Sharded checkpoints are
read through `model.safetensors.index.json` (`weight_map`, :207-225), whose shard names
must stay inside the model folder.

Tensors are views of a memory map: nothing is copied until a tensor is moved to a device.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path
from typing import Dict, Iterable, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 << 20


def _no_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise SafetensorsError(f"duplicate tensor name {k!r} in the header")
        out[k] = v
    return out


class SafetensorsFile:
    """One memory-mapped file; `entries` maps a name to (dtype, shape, begin, end) in file offsets."""

    def __init__(self, path):
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to be a safetensors file ({size} bytes)")
        self._file = open(self.path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen < 2 or hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: header length {hlen} does not fit a file of {size} bytes")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"), object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: the header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: the header must be a JSON object")
        base = 8 + hlen
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        ranges = []
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype_name, shape, (lo, hi) = meta["dtype"], meta["shape"], meta["data_offsets"]
                shape = tuple(int(s) for s in shape)
                lo, hi = int(lo), int(hi)
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: malformed header entry for {name!r}: {meta!r}") from None
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {dtype_name!r} "
                                       f"(supported: {', '.join(sorted(_DTYPES))})")
            if any(s < 0 for s in shape):
                raise SafetensorsError(f"{self.path}: tensor {name!r} has a negative dimension {shape}")
            dtype, width = _DTYPES[dtype_name]
            count = 1
            for s in shape:
                count *= s
            if lo < 0 or hi < lo or base + hi > size or hi - lo != count * width:
                raise SafetensorsError(f"{self.path}: tensor {name!r} of shape {shape} and dtype {dtype_name} needs "
                                       f"{count * width} bytes, data_offsets give [{lo}, {hi}) in {size - base}")
            self.entries[name] = (dtype, shape, base + lo, base + hi)
            if hi > lo:
                ranges.append((lo, hi, name))
        ranges.sort()
        for (_, hi_a, a), (lo_b, _, b) in zip(ranges, ranges[1:]):
            if lo_b < hi_a:
                raise SafetensorsError(f"{self.path}: the data of {a!r} and {b!r} overlap")

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, lo, hi = self.entries[name]
        if hi == lo:
            return torch.empty(shape, dtype=dtype)
        count = (hi - lo) // _DTYPES[_NAMES[dtype]][1]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the map is read-only; the tensors are only ever read
            return torch.frombuffer(self._map, dtype=dtype, count=count, offset=lo).reshape(shape)


class TensorSource:
    """All tensors of a model folder by name: `model.safetensors`, or the shards its index names."""

    def __init__(self, model_dir):
        self.dir = Path(model_dir)
        single, index = self.dir / "model.safetensors", self.dir / "model.safetensors.index.json"
        self.files = []
        self.where: Dict[str, SafetensorsFile] = {}
        if single.is_file():
            self._add(SafetensorsFile(single))
        elif index.is_file():
            try:
                weight_map = json.loads(index.read_text())["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise SafetensorsError(f"{index}: no readable 'weight_map'") from None
            opened = {}
            for name, shard in weight_map.items():
                if not isinstance(shard, str) or "/" in shard or "\\" in shard or shard.startswith("."):
                    raise SafetensorsError(f"{index}: shard name {shard!r} must be a plain file name in the model folder")
                if shard not in opened:
                    opened[shard] = SafetensorsFile(self.dir / shard)
                    self.files.append(opened[shard])
                if name not in opened[shard].entries:
                    raise SafetensorsError(f"{index}: tensor {name!r} is not in shard {shard!r}")
                self.where[name] = opened[shard]
        else:
            raise SafetensorsError(f"{self.dir}: neither model.safetensors nor model.safetensors.index.json")

    def _add(self, f: SafetensorsFile):
        self.files.append(f)
        for name in f.entries:
            self.where[name] = f

    def names(self) -> Iterable[str]:
        return self.where.keys()

    def has(self, name: str) -> bool:
        return name in self.where

    def meta(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self.where[name].entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self.where:
            raise SafetensorsError(f"tensor {name!r} not found in {self.dir}")
        return self.where[name].tensor(name)


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Writes CPU tensors in the order given, each aligned to 8 bytes through header padding."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot write tensor {name!r} of dtype {t.dtype}")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
