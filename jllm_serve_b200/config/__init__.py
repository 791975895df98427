"""Typed configuration and the architecture registry."""
from .specs import (ConfigError, Core, Decoder, DenseGluSpec, FeedForwardSpec, GqaAttentionSpec, LayerNames, LayerRun, LayerSpec, ModelNames,
                    MixerSpec, NormSpec, RopeScaling, RopeTableSpec)
from .reader import ConfigReader
from .registry import (architecture_entry, load_config, parse_config, register_architecture, supported_architectures,
                       unregister_architecture)
from .families import DecoderDraft, parse_qwen3, parse_rope_scaling

register_architecture("qwen3", parse_qwen3, replace=True)
