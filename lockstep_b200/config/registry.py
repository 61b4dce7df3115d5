"""One registry from an architecture's name to its configuration class.

``config.json`` names its architecture in ``architectures[0]`` (``model_type``
is accepted where that list is absent).  The configuration class reads the
architecture's own keys and builds the ``ModelSpec``; the generic model in
``engine.model`` is assembled from that spec, so registering an architecture
means registering a configuration class and, if it needs them, new parts.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Callable, Mapping

from .spec import ConfigError, ModelSpec

_ARCHITECTURES: dict[str, type] = {}
_MODEL_TYPES: dict[str, str] = {}


def register_architecture(name: str, model_type: str | None = None) -> Callable[[type], type]:
    """Class decorator: ``name`` is what ``architectures[0]`` holds."""

    def wrap(cls: type) -> type:
        if name in _ARCHITECTURES and _ARCHITECTURES[name] is not cls:
            raise ValueError(f"architecture {name!r} is already registered")
        _ARCHITECTURES[name] = cls
        if model_type:
            _MODEL_TYPES[model_type] = name
        cls.architecture = name
        return cls

    return wrap


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)
    for k in [k for k, v in _MODEL_TYPES.items() if v == name]:
        del _MODEL_TYPES[k]


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_name(raw: Mapping[str, Any]) -> str:
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        return str(archs[0])
    mt = raw.get("model_type")
    if mt in _MODEL_TYPES:
        return _MODEL_TYPES[mt]
    raise ConfigError(
        "config.json names no architecture: give \"architectures\": [\"<name>\"] "
        f"(known: {known_architectures()})")


def config_from_dict(raw: Mapping[str, Any]):
    """The typed configuration for a ``config.json`` dictionary."""
    name = architecture_name(raw)
    cls = _ARCHITECTURES.get(name)
    if cls is None:
        raise ConfigError(f"unknown architecture {name!r}; known: {known_architectures()}")
    return cls.from_dict(raw)


def load_config(folder: str | Path):
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    return config_from_dict(raw)


def model_spec(config) -> ModelSpec:
    return config.model_spec()
