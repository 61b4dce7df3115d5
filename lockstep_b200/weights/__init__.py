"""Weights: reading a model folder by tensor name, and the random-weights mode."""

from .loader import WeightError, load_weights
from .random_init import random_tensors, write_random_model

__all__ = ["WeightError", "load_weights", "random_tensors", "write_random_model"]
