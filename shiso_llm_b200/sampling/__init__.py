"""Sampling: parameters, the device sampler and host samplers."""

from .device import DeviceSampler
from .host import Xorshift64Star, argmax, candidate_mask, keyed_sample, keyed_uniform, stream_sample, suppress
from .params import SamplingParams

__all__ = [
    "DeviceSampler", "SamplingParams", "Xorshift64Star", "argmax", "candidate_mask",
    "keyed_sample", "keyed_uniform", "stream_sample", "suppress",
]
