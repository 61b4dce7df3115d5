"""What a model is made of, as plain data.

An architecture's configuration class turns its ``config.json`` keys into a
``ModelSpec``: one ``LayerSpec`` per layer (which mixer, feed-forward, norm and
position encoding, each with its sizes and constants as parameters) and a
``schedule`` that says in which order layers run and whose cache each run uses.
Nothing below the configuration class knows which architecture it serves.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


def _freeze(params: Mapping[str, Any] | None) -> Mapping[str, Any]:
    return MappingProxyType(dict(params or {}))


@dataclass(frozen=True)
class PartSpec:
    """A part by the name it is registered under, and its parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "params", _freeze(self.params))

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default=None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer and a feed-forward.

    ``prefix`` is the tensor-name prefix of the layer's weights
    (``model.layers.3``); each part adds its own suffixes.  ``extra`` holds whatever further
    parts the layer's block arrangement asks for, by the name it asks under (norms after the
    mixer or the feed-forward, a second feed-forward branch, ...): the block receives the whole
    ``LayerSpec`` and builds them, nothing else reads them.
    """

    prefix: str
    block: PartSpec            # arrangement, e.g. pre_norm
    mixer: PartSpec            # e.g. gqa_attention
    feed_forward: PartSpec     # e.g. swiglu
    mixer_norm: PartSpec       # norm in front of the mixer
    feed_forward_norm: PartSpec
    position: PartSpec         # position encoding the mixer applies
    extra: Mapping[str, PartSpec] = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "extra", _freeze(self.extra))


@dataclass(frozen=True)
class LayerRun:
    """One entry of the schedule: run layer ``layer`` on cache entry ``cache``.

    A layer may be run more than once (give each run its own ``cache``), and a
    run may read a cache entry that an earlier run wrote (``writes_cache``
    False): it then adds nothing to the cache.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[LayerRun, ...]
    # tensor-name prefixes of the parts that are not layers
    names: Mapping[str, str] = field(default_factory=lambda: {
        "embedding": "model.embed_tokens", "final_norm": "model.norm", "head": "lm_head"})

    def __post_init__(self):
        object.__setattr__(self, "names", _freeze(self.names))
        object.__setattr__(self, "layers", tuple(self.layers))
        object.__setattr__(self, "schedule", tuple(self.schedule))
        writers: dict[int, int] = {}
        for run in self.schedule:
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule names layer {run.layer}, the model has {len(self.layers)}")
            if run.writes_cache:
                if run.cache in writers:
                    raise ValueError(f"cache entry {run.cache} is written by two runs of the schedule")
                writers[run.cache] = run.layer
            elif run.cache not in writers:
                raise ValueError(f"a run reads cache entry {run.cache} before any run wrote it")

    @property
    def cache_entries(self) -> int:
        return 1 + max((run.cache for run in self.schedule), default=-1)


class ConfigError(ValueError):
    """config.json is missing a key, has a wrong value, or asks for what the engine lacks."""
