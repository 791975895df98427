"""Family parsers: config.json of one `model_type` -> a `Decoder` spec.

As in the reference, a family is a generic decoder reader (`DecoderDraft`) plus a few switches
that the family sets (src/main/java/org/robomiri/jllm/model/Families.java:166-171 for qwen3, the
shared reader at :611-916). Adding a dense family means writing one function of a few lines,
as `parse_qwen3` below, and one `register_architecture` line.
"""
from __future__ import annotations

import math

from .reader import ConfigReader
from .specs import (ConfigError, Core, Decoder, DenseGluSpec, GqaAttentionSpec, LayerSpec, NormSpec, RopeScaling,
                    RopeTableSpec)


def parse_rope_scaling(rs: ConfigReader | None, c: ConfigReader) -> RopeScaling:
    """`rope_scaling`: default/none, linear and yarn (Families.java:1001-1072); the others are refused by name."""
    if rs is None:
        return RopeScaling()
    kind = rs.string("rope_type", rs.string("type", "default"))
    factor = rs.number("factor", 1.0)
    if kind in ("default", "none"):
        return RopeScaling()
    if kind == "linear":
        if factor <= 0:
            raise ConfigError(f"invalid linear rope_scaling: factor={factor}")
        return RopeScaling(kind="linear", factor=factor)
    if kind == "yarn":
        orig = rs.integer("original_max_position_embeddings", c.integer("max_position_embeddings", 0))
        beta_fast, beta_slow = rs.number("beta_fast", 32.0), rs.number("beta_slow", 1.0)
        attention = rs.number("attention_factor", 0.0)
        if not factor > 0 or orig <= 0 or not beta_fast > beta_slow or not beta_slow > 0 or attention < 0:
            raise ConfigError(f"invalid yarn rope_scaling: {dict(rs.values)}")
        mscale, all_dim = rs.number("mscale", 0.0), rs.number("mscale_all_dim", 0.0)
        both = mscale != 0 and all_dim != 0
        return RopeScaling(kind="yarn", factor=factor, original_max_positions=orig, beta_fast=beta_fast,
                           beta_slow=beta_slow, mscale=mscale if both else 1.0, mscale_all_dim=all_dim if both else 0.0,
                           attention_factor=attention, truncate=rs.boolean("truncate", True))
    raise ConfigError(f"unsupported rope_scaling type {kind!r} (supported: default, linear, yarn)")


class DecoderDraft:
    """The keys every dense decoder family reads, and the switches a family sets before `build` reads the rest with
    the family's defaults, validates and resolves the layer specs and the canonical description (the reference's
    `Draft`, Families.java:611-733, with the switches of :639-668 that dense families use). The defaults are Llama's.

    Switches:
      bias      "reject"      `attention_bias=true` is an error (the family has no such key)
                "always"      q, k and v have biases whatever the config says; o_proj has none
                "config_qkvo" the config's value, false when absent: biases on q, k, v and o_proj
      qk_norm   per-head RMSNorm of queries and keys before the rotation
      window    "none" | "all" (every layer gets `sliding_window`) | "from_max_window_layers" (layers >=
                `max_window_layers`, and only with `use_sliding_window`)
      theta_default, norm_eps_default, partial_rotary_default, tied_default, max_positions_default
    """

    def __init__(self, values: dict, model_type: str, architecture: str):
        self.values, self.model_type, self.architecture = values, model_type, architecture
        self.c = c = ConfigReader(values)
        archs = values.get("architectures")
        if isinstance(archs, list) and archs and archs[0] != architecture:
            raise ConfigError(f"model_type {model_type!r} goes with architecture {architecture}, "
                              f"config.json names {archs[0]!r}")
        self.dim = c.positive("hidden_size")
        self.layers = c.positive("num_hidden_layers")
        self.vocab = c.positive("vocab_size")
        self.heads = c.positive("num_attention_heads")
        self.kv_heads = c.integer("num_key_value_heads", self.heads)
        self.head_dim = c.integer("head_dim", self.dim // self.heads)
        self.hidden = c.integer("intermediate_size", 0)
        # newer configs nest rope_theta, partial_rotary_factor and the scaling keys in rope_parameters; the top-level
        # keys win when both are there (Families.java:716-731)
        self.rope_parameters = c.mapping("rope_parameters")
        scaling = c.mapping("rope_scaling")
        rp = self.rope_parameters
        if scaling is None and rp is not None and (rp.has("rope_type") or rp.has("type")):
            scaling = rp
        self.scaling_map = scaling
        # the family's switches
        self.bias = "reject"
        self.qk_norm = False
        self.window = "none"
        self.theta_default = 10000.0
        self.norm_eps_default = 1e-6
        self.partial_rotary_default = 1.0
        self.tied_default = False
        self.max_positions_default = 4096

    def _rope_number(self, key: str, default: float) -> float:
        if self.c.has(key) or self.rope_parameters is None:
            return self.c.number(key, default)
        return self.rope_parameters.number(key, default)

    def build(self) -> Decoder:
        c, dim, layers, heads, kv_heads, head_dim = self.c, self.dim, self.layers, self.heads, self.kv_heads, self.head_dim
        if head_dim <= 0:
            raise ConfigError(f"head_dim must be positive, got {head_dim}")
        if kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(f"num_key_value_heads={kv_heads} must be positive and divide num_attention_heads={heads}")
        if c.has("num_experts") and c.integer("num_experts") > 0:
            raise ConfigError("num_experts > 0: expert feed-forwards belong to another architecture, not built")
        if self.hidden <= 0:
            raise ConfigError(f"intermediate_size must be positive for a dense feed-forward, got {self.hidden}")
        if c.boolean("mlp_bias", False):
            raise ConfigError("models with an MLP bias (mlp_bias=true) are not supported")
        act = c.string("hidden_act", "silu")
        eps = c.number("rms_norm_eps", self.norm_eps_default)
        if not eps >= 0:
            raise ConfigError(f"rms_norm_eps={eps} must not be negative")
        configured = c.boolean("attention_bias", False)
        if self.bias == "reject":
            if configured:
                raise ConfigError(f"attention_bias=true is not a key of model_type {self.model_type!r}")
            bias = out_bias = False
        elif self.bias == "always":
            bias, out_bias = True, False
        elif self.bias == "config_qkvo":
            bias = out_bias = configured
        else:
            raise ValueError(f"unknown bias switch {self.bias!r}")
        partial = self._rope_number("partial_rotary_factor", self.partial_rotary_default)
        if partial <= 0 or partial > 1 or int(head_dim * partial) < 2:
            raise ConfigError(f"invalid partial_rotary_factor {partial}")
        rotary_dim = int(head_dim * partial) & ~1
        theta = self._rope_number("rope_theta", self.theta_default)
        scaling = parse_rope_scaling(self.scaling_map, c)
        window, window_from = 0, 0
        sw = c.integer("sliding_window", 0) if c.has("sliding_window") else 0
        if self.window == "all" and sw > 0:
            window = sw
        elif self.window == "from_max_window_layers" and sw > 0 and c.boolean("use_sliding_window", False):
            window, window_from = sw, c.integer("max_window_layers", layers)
        elif self.window not in ("none", "all", "from_max_window_layers"):
            raise ValueError(f"unknown window switch {self.window!r}")
        norm = NormSpec("rmsnorm", eps)
        scale = float(1.0 / math.sqrt(head_dim))
        specs = []
        for l in range(layers):
            attn = GqaAttentionSpec(heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                    window=window if window > 0 and l >= window_from else 0, rope_table=0,
                                    qk_norm=self.qk_norm, qk_norm_eps=eps, bias=bias, out_bias=out_bias, scale=scale)
            specs.append(LayerSpec(attn, DenseGluSpec(hidden=self.hidden, activation=act), norm))
        extra = (" bias" if bias else "") + (" obias" if out_bias else "") \
            + (f" window={window}@{window_from}" if window else "") \
            + (f" rope={scaling.kind}x{scaling.factor:g}" if scaling.kind != "none" else "") \
            + (f" rotary={rotary_dim}" if rotary_dim != head_dim else "")
        description = (f"{self.architecture} dim={dim} ffn={self.hidden} layers={layers} heads={heads}/{kv_heads} "
                       f"headDim={head_dim} vocab={self.vocab} theta={theta:.0f}{extra}")
        core = Core(architecture=self.architecture, model_type=self.model_type, dim=dim, layers=layers, vocab=self.vocab,
                    norm_eps=eps, tied=c.boolean("tie_word_embeddings", self.tied_default),
                    bos=c.integer("bos_token_id", -1), eos=c.int_list("eos_token_id"),
                    max_positions=c.positive("max_position_embeddings", self.max_positions_default),
                    description=description)
        return Decoder(core, tuple(specs), (RopeTableSpec(rotary_dim, theta, scaling, "half"),), norm)


def parse_qwen3(values: dict) -> Decoder:
    """Qwen3 dense: per-head q/k RMSNorm, the window rule of Qwen2 (`use_sliding_window`, from layer
    `max_window_layers` on), no biases unless `attention_bias` (then q, k, v and o_proj) (Families.java:166-171)."""
    d = DecoderDraft(values, "qwen3", "Qwen3ForCausalLM")
    d.bias, d.qk_norm, d.window = "config_qkvo", True, "from_max_window_layers"
    return d.build()
