"""Typed configurations and the architecture registry."""

from .registry import (architecture_name, config_from_dict, known_architectures, load_config,
                       register_architecture, unregister_architecture)
from .spec import ConfigError, LayerRun, LayerSpec, ModelSpec, PartSpec
from . import qwen3 as _qwen3  # registers Qwen3ForCausalLM
from .qwen3 import Qwen3Config

__all__ = [
    "ConfigError", "LayerRun", "LayerSpec", "ModelSpec", "PartSpec", "Qwen3Config",
    "architecture_name", "config_from_dict", "known_architectures", "load_config",
    "register_architecture", "unregister_architecture",
]
