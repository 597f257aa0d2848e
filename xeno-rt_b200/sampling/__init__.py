"""Sampling: the options of the reference's sampler and the device kernels that apply them."""
from .params import SamplerConfig, GREEDY_THRESHOLD
from .sampler import Sampler, sequence_key

__all__ = ["SamplerConfig", "GREEDY_THRESHOLD", "Sampler", "sequence_key"]
