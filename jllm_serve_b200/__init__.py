"""A B200-native inference engine for the Qwen3 dense architecture.

Typed configuration and an architecture registry (`config`), weights by tensor name
(`weights`), layers put together from parts (`parts`), a paged cache manager (`cache`),
one step function, a scheduler and generation (`engine`), sampling (`sampling`), and the
hand-written sm_100a kernels (`csrc`). There is no CPU path: the engine needs a B200.
"""
__version__ = "0.1.0"

from . import config  # registers the architectures
