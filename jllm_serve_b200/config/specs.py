"""The typed configuration: what a model is made of, as plain immutable data.

The vocabulary follows the reference's: a decoder is a core (sizes shared by the whole
model), a list of layer specs and a list of rotary tables
(src/main/java/org/robomiri/jllm/model/Decoder.java:15-33, LayerSpec.java:11-19,
Attention.java:48-50, Mlp.java:7-22, RopeTable.java:20-51, Architecture.java:61-67).
Every size and constant that a part needs is a field here; parts never read
`model_type` and never see config.json.

Two things go beyond the reference's vocabulary, because the order of layers is data:
`Decoder.schedule` lists the layer runs, and a run may name a layer a second time or
read the keys and values of an earlier run instead of writing its own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model: the message names the key and its value."""


@dataclass(frozen=True)
class RopeScaling:
    """How the inverse frequencies of a rotary table are stretched (Scaling.java:6-78)."""
    kind: str = "none"                     # none | linear | yarn
    factor: float = 1.0
    original_max_positions: int = 0        # yarn: the trained length
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    attention_factor: float = 0.0          # 0 = derive from factor
    truncate: bool = True


@dataclass(frozen=True)
class RopeTableSpec:
    """One rotary table: `rotary_dim` values of each head are rotated, paired as (i, i + rotary_dim / 2)."""
    rotary_dim: int
    theta: float
    scaling: RopeScaling = RopeScaling()
    pairing: str = "half"                  # half: (i, i + rotary_dim/2)
    kind: str = field(default="rotary", init=False)   # which registered position encoding builds the table

    def __post_init__(self):
        if self.rotary_dim < 2 or self.rotary_dim % 2:
            raise ConfigError(f"rotary_dim={self.rotary_dim} must be even and at least 2")
        if not self.theta > 0:
            raise ConfigError(f"rope_theta={self.theta} must be positive")
        if self.pairing != "half":
            raise ConfigError(f"rope pairing {self.pairing!r} is not built (built: half)")


@dataclass(frozen=True)
class NormSpec:
    kind: str = "rmsnorm"
    eps: float = 1e-6


@dataclass(frozen=True)
class MixerSpec:
    """Base of every token mixer's spec; `kind` picks the part from the parts registry."""
    kind: str = field(default="", init=False)


@dataclass(frozen=True)
class GqaAttentionSpec(MixerSpec):
    """Grouped-query causal attention over a paged cache (Attention.java:48-50,68-71)."""
    kind: str = field(default="gqa_attention", init=False)
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0                        # 0 = all keys; else the last `window` keys
    rope_table: int = 0                    # index into Decoder.rope_tables, -1 = no rotation
    qk_norm: bool = False                  # per-head RMSNorm of q and k before the rotation
    qk_norm_eps: float = 1e-6
    bias: bool = False                     # q, k, v biases
    out_bias: bool = False                 # o_proj bias
    scale: float = 0.0                     # multiplier of q . k

    def __post_init__(self):
        if self.heads <= 0:
            raise ConfigError(f"num_attention_heads={self.heads} must be positive")
        if self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ConfigError(f"num_key_value_heads={self.kv_heads} must be positive and divide "
                              f"num_attention_heads={self.heads}")
        if self.head_dim <= 0:
            raise ConfigError(f"head_dim must be positive, got {self.head_dim}")
        if self.window < 0:
            raise ConfigError(f"sliding_window={self.window} must not be negative")


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str = field(default="", init=False)


@dataclass(frozen=True)
class DenseGluSpec(FeedForwardSpec):
    """down(act(gate x) * (up x)) (Mlp.java:21)."""
    kind: str = field(default="dense_glu", init=False)
    hidden: int = 0
    activation: str = "silu"

    def __post_init__(self):
        if self.hidden <= 0:
            raise ConfigError(f"intermediate_size must be positive for a dense feed-forward, got {self.hidden}")
        if self.activation != "silu":
            raise ConfigError(f"unsupported hidden_act {self.activation!r}: only silu (SwiGLU) is built")


@dataclass(frozen=True)
class LayerNames:
    """Checkpoint names of a layer's pieces, relative to the layer's prefix (DecoderLayer.java:20-32)."""
    mixer: str = "self_attn."
    feed_forward: str = "mlp."
    mixer_norm: str = "input_layernorm."
    feed_forward_norm: str = "post_attention_layernorm."


@dataclass(frozen=True)
class ModelNames:
    """Checkpoint names of the model's own tensors (ModelWeights.java:36-37,68,74-77)."""
    embedding: str = "model.embed_tokens.weight"
    layer: str = "model.layers.{}."
    final_norm: str = "model.norm."
    head: str = "lm_head.weight"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer, a feed-forward, the norm before each, and how they are arranged."""
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    norm: NormSpec
    arrangement: str = "pre_norm"          # x += mixer(norm(x)); x += ffn(norm(x))
    names: LayerNames = LayerNames()


@dataclass(frozen=True)
class LayerRun:
    """One entry of the schedule: run `layer`; `cache_of` = the index of the earlier run whose
    cache this run's mixer reads instead of keeping one of its own (None = its own)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class Core:
    """Sizes and switches of the whole model (Architecture.java:61-67)."""
    architecture: str
    model_type: str
    dim: int
    layers: int
    vocab: int
    norm_eps: float
    tied: bool
    bos: int
    eos: Tuple[int, ...]
    max_positions: int
    description: str = ""


@dataclass(frozen=True)
class Decoder:
    core: Core
    layers: Tuple[LayerSpec, ...]
    rope_tables: Tuple[object, ...]       # position tables: RopeTableSpec, or any spec with a registered `kind`
    final_norm: NormSpec
    schedule: Tuple[LayerRun, ...] = ()
    names: ModelNames = ModelNames()

    def __post_init__(self):
        if len(self.layers) != self.core.layers or self.core.layers <= 0:
            raise ConfigError(f"num_hidden_layers={self.core.layers} but {len(self.layers)} layer specs")
        if not self.schedule:
            object.__setattr__(self, "schedule", tuple(LayerRun(l) for l in range(len(self.layers))))
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"schedule entry {i} names layer {run.layer} of {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {run.cache_of}, "
                                      f"which does not run before it")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {run.cache_of}, "
                                      f"which keeps none of its own")
        for t in self.rope_tables:
            if not getattr(t, "kind", ""):
                raise ConfigError(f"position table {t!r} names no kind of position encoding")
        for spec in self.layers:
            t = getattr(spec.mixer, "rope_table", -1)
            if t >= len(self.rope_tables):
                raise ConfigError(f"a layer names rope table {t} of {len(self.rope_tables)}")

    def with_schedule(self, schedule) -> "Decoder":
        runs = tuple(r if isinstance(r, LayerRun) else LayerRun(*r) for r in schedule)
        return Decoder(self.core, self.layers, self.rope_tables, self.final_norm, runs, self.names)
