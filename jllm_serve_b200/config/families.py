"""Family parsers: config.json of one `model_type` -> a `Decoder` spec.

As in the reference, a family is a generic decoder reader plus a few switches that the
family sets (src/main/java/org/robomiri/jllm/model/Families.java:166-171 for qwen3, the
shared reader at :611-916). Adding a family means writing one such function and one
`register_architecture` line.
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


def parse_qwen3(values: dict) -> Decoder:
    """Qwen3 dense: per-head q/k RMSNorm, the window rule of Qwen2 (`use_sliding_window`, from layer
    `max_window_layers` on), no biases unless `attention_bias` (then q, k, v and o_proj)
    (Families.java:166-171; keys and defaults :711-719,735-800,861,913-914)."""
    c = ConfigReader(values)
    arch = "Qwen3ForCausalLM"
    archs = values.get("architectures")
    if isinstance(archs, list) and archs and archs[0] != arch:
        raise ConfigError(f"model_type 'qwen3' goes with architecture {arch}, config.json names {archs[0]!r}")
    dim = c.positive("hidden_size")
    layers = c.positive("num_hidden_layers")
    vocab = c.positive("vocab_size")
    heads = c.positive("num_attention_heads")
    kv_heads = c.integer("num_key_value_heads", heads)
    head_dim = c.integer("head_dim", dim // heads)
    if head_dim <= 0:
        raise ConfigError(f"head_dim must be positive, got {head_dim}")
    if kv_heads <= 0 or heads % kv_heads:
        raise ConfigError(f"num_key_value_heads={kv_heads} must be positive and divide num_attention_heads={heads}")
    if c.has("num_experts") and c.integer("num_experts") > 0:
        raise ConfigError("num_experts > 0: expert feed-forwards belong to another architecture (qwen3_moe), not built")
    hidden = c.integer("intermediate_size", 0)
    if c.boolean("mlp_bias", False):
        raise ConfigError("models with an MLP bias (mlp_bias=true) are not supported")
    act = c.string("hidden_act", "silu")
    eps = c.number("rms_norm_eps", 1e-6)
    if not eps >= 0:
        raise ConfigError(f"rms_norm_eps={eps} must not be negative")
    bias = c.boolean("attention_bias", False)
    partial = c.number("partial_rotary_factor", 1.0)
    if partial <= 0 or partial > 1 or int(head_dim * partial) < 2:
        raise ConfigError(f"invalid partial_rotary_factor {partial}")
    rotary_dim = int(head_dim * partial) & ~1
    theta = c.number("rope_theta", 10000.0)
    scaling = parse_rope_scaling(c.mapping("rope_scaling"), c)
    window, window_from = 0, 0
    sw = c.integer("sliding_window", 0) if c.has("sliding_window") else 0
    if sw > 0 and c.boolean("use_sliding_window", False):
        window = sw
        window_from = c.integer("max_window_layers", layers)
    norm = NormSpec("rmsnorm", eps)
    scale = float(1.0 / math.sqrt(head_dim)) if head_dim > 0 else 0.0
    specs = []
    for l in range(layers):
        attn = GqaAttentionSpec(heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                window=window if window > 0 and l >= window_from else 0, rope_table=0, qk_norm=True,
                                qk_norm_eps=eps, bias=bias, out_bias=bias, scale=scale)
        specs.append(LayerSpec(attn, DenseGluSpec(hidden=hidden, activation=act), norm))
    extra = (" bias obias" if bias else "") + (f" window={window}@{window_from}" if window else "") \
        + (f" rope={scaling.kind}x{scaling.factor:g}" if scaling.kind != "none" else "") \
        + (f" rotary={rotary_dim}" if rotary_dim != head_dim else "")
    description = (f"{arch} dim={dim} ffn={hidden} layers={layers} heads={heads}/{kv_heads} headDim={head_dim} "
                   f"vocab={vocab} theta={theta:.0f}{extra}")
    core = Core(architecture=arch, model_type="qwen3", dim=dim, layers=layers, vocab=vocab, norm_eps=eps,
                tied=c.boolean("tie_word_embeddings", False), bos=c.integer("bos_token_id", -1),
                eos=c.int_list("eos_token_id"), max_positions=c.positive("max_position_embeddings", 4096),
                description=description)
    return Decoder(core, tuple(specs), (RopeTableSpec(rotary_dim, theta, scaling, "half"),), norm)
