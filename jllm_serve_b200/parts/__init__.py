"""The parts a model is put together from. Importing the package registers the built-in kinds."""
from .base import (Block, FeedForward, Mixer, Norm, Part, PositionEncoding, RunCache, Runtime, part_class,
                   register_block, register_feed_forward, register_mixer, register_norm, register_position_encoding)
from .linear import Linear
from .norm import RmsNorm
from .rope import RotaryTable
from .attention import GqaAttention
from .mlp import DenseGlu
from .block import PreNormBlock
