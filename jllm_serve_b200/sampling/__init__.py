"""Sampling: parameters and the device sampler."""
from .params import SamplingParams
from .sampler import RequestRng, Sampler
