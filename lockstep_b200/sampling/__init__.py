"""Sampling: the counter-based random numbers and the device sampler."""

from . import philox
from .sampler import Sampler, SamplingParams

__all__ = ["Sampler", "SamplingParams", "philox"]
