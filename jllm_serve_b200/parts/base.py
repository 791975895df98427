"""The interfaces of the parts a layer is put together from, and the registry that picks them.

A part is built from its spec (sizes and constants), the model's width, its tensors and
the `Runtime`; it never learns which model it is in. The kinds:

* `Norm`:             `forward(x, out, row_index=None, rows=None)`; x float32 [rows, dim] -> out (compute dtype).
* `PositionEncoding`: made once per position table (`spec.kind` picks the class) and context, as
                      `cls(spec, max_positions, device)`, with `tensors=` and `dim=` too if its `wants` names
                      tensors (full checkpoint names; the prefix it is given is empty); a mixer that rotates asks
                      it for `cos`, `sin`, `rotary_dim`; one that adds to the embedding overrides
                      `on_embedding(x, batch)`.
* `Mixer`:            `cache_need(spec)` says what it keeps between steps (one need, a tuple of needs, or None);
                      `forward(xb, x, batch, cache)` reads the normed rows `xb` and ADDS its result into the
                      float32 residual stream `x`.
* `FeedForward`:      `forward(xb, x, batch)`, same contract.
* `Block`:            the arrangement of norm, mixer and feed-forward in one layer.

Every part class has `wants(spec, dim, prefix) -> {checkpoint name: TensorWant}`: the tensors
it needs, which is also what the loader checks the file against and what the random-weights
mode generates.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

import torch


@dataclass
class Runtime:
    """Where and how a model runs: the same for every part of one model."""
    device: torch.device
    dtype: torch.dtype                     # compute dtype: torch.float32 or torch.bfloat16
    max_positions: int                     # the context: positions 0 .. max_positions - 1 can be cached
    max_rows: int                          # most rows (tokens) in one step
    page_size: int

    def __post_init__(self):
        self._buffers: Dict[str, torch.Tensor] = {}
        self.notes: list = []              # what a part wants the user to know about how it was built

    def buffer(self, name: str, cols: int, dtype: Optional[torch.dtype] = None, rows: Optional[int] = None):
        """A persistent [rows or max_rows, cols] scratch tensor: the same memory at every step, so that a
        captured step can be replayed. Parts slice the rows they use. Buffers of one name are shared by all
        layers, which run one after the other."""
        dtype = dtype or self.dtype
        key = f"{name}:{cols}:{dtype}:{rows}"
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.empty((rows or self.max_rows, cols), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf


class Part:
    @classmethod
    def wants(cls, spec, dim: int, prefix: str) -> dict:
        return {}


class Norm(Part):
    graph_safe = True

    def forward(self, x, out, row_index=None, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    graph_safe = True

    def on_embedding(self, x, batch) -> None:
        """Hook for encodings that add to the embedded rows; rotary tables leave them alone."""


class Mixer(Part):
    # False for a part whose forward decides on the host from values that change between steps of the same
    # shape (it cannot be captured once and replayed); decode steps then run launch by launch
    graph_safe = True

    @classmethod
    def cache_need(cls, spec):
        """A `cache.CacheNeed` (or None): what a run of this mixer keeps between steps."""
        return None

    def decode_bucket_cap(self, rows: int) -> int:
        """The smallest `batch.kv_bucket` (the longest request's keys in units of 256, at most 32) from which on a step of
        `rows` single rows launches the same kernels in the same shapes however long the context is; 32: the launches
        may change up to the largest bucket (the safe answer, and the default). The step function clamps a decode
        step's bucket to the largest cap among the model's parts: a context that grows then asks for a newly captured
        step a few times in its life and not every 256 tokens."""
        return 32

    def forward(self, xb, x, batch, cache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    graph_safe = True

    def forward(self, xb, x, batch) -> None:
        raise NotImplementedError


class Block(Part):
    # an arrangement says itself whether its step can be captured and replayed (usually: whether all its parts
    # can); one that does not say is run launch by launch
    graph_safe = False

    def decode_bucket_cap(self, rows: int) -> int:
        """See `Mixer.decode_bucket_cap`: the largest cap among the arrangement's parts."""
        return 32

    def forward(self, x, batch, cache) -> None:
        raise NotImplementedError


@dataclass
class RunCache:
    """What one layer run sees of the cache in a step."""
    run: int                               # schedule index whose cache this is
    writes: bool                           # False: the run reads another run's cache and stores nothing
    group: int = -1                        # paged group index (block tables and write slots of the batch), -1 = none
    keys: Optional[torch.Tensor] = None    # [pages, kv_heads, page_size, head_dim]
    values: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None   # [slots, ...] for a fixed-state mixer (the first of `states`)
    states: tuple = ()                     # every fixed-size state the mixer named, in its order; a mixer may hold
                                           # these beside paged keys and values


_REGISTRIES: Dict[str, Dict[str, Callable]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def _register(family: str, kind: str, cls, replace: bool):
    table = _REGISTRIES[family]
    if kind in table and not replace:
        raise ValueError(f"{family} part {kind!r} is registered already")
    table[kind] = cls


def register_mixer(kind: str, cls, replace: bool = False):
    _register("mixer", kind, cls, replace)


def register_feed_forward(kind: str, cls, replace: bool = False):
    _register("feed_forward", kind, cls, replace)


def register_norm(kind: str, cls, replace: bool = False):
    _register("norm", kind, cls, replace)


def register_position_encoding(kind: str, cls, replace: bool = False):
    _register("position", kind, cls, replace)


def register_block(kind: str, cls, replace: bool = False):
    _register("block", kind, cls, replace)


def part_class(family: str, kind: str):
    table = _REGISTRIES[family]
    if kind not in table:
        raise KeyError(f"no {family} part of kind {kind!r} (registered: {', '.join(sorted(table)) or 'none'})")
    return table[kind]
