"""Parts a layer is put together from, and their registries."""

from .base import (Block, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime,
                   WeightSpec, build_part, known_parts, register_part, unregister_part)
from . import attention, block, embedding, mlp, norm, position  # register the built-in parts

__all__ = [
    "Block", "CacheNeed", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime",
    "WeightSpec", "build_part", "known_parts", "register_part", "unregister_part",
]
