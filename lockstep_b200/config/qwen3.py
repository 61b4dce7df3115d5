"""Qwen3 dense: typed configuration read from the architecture's own config.json keys.

Keys and meanings follow LockStep's ``Qwen3Config`` (engine/model/qwen3.py:49-80);
what LockStep ignores but would change the result if set is refused here
(attention_bias, rope_scaling, a hidden_act other than silu).  The window keys
(``use_sliding_window``, ``sliding_window``, ``max_window_layers``) are read:
layers at or past ``max_window_layers`` then attend to the last
``sliding_window`` positions only, and live in a cache group of their own.
"""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Mapping

from .registry import register_architecture
from .spec import ConfigError, LayerRun, LayerSpec, ModelSpec, PartSpec

_REQUIRED = (
    "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
    "num_key_value_heads", "vocab_size", "rms_norm_eps", "rope_theta", "max_position_embeddings",
)


@register_architecture("Qwen3ForCausalLM", model_type="qwen3")
@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int = 0

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        if raw.get("model_type", "qwen3") != "qwen3":
            raise ConfigError(f"expected model_type \"qwen3\", got {raw.get('model_type')!r}")
        missing = [k for k in _REQUIRED if k not in raw]
        if missing:
            raise ConfigError(f"config.json lacks the keys {missing}")
        if raw.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported (Qwen3 dense has no projection biases)")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is not supported")
        if raw.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {raw.get('hidden_act')!r} is not supported (silu only)")
        heads = int(raw["num_attention_heads"])
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if int(raw["hidden_size"]) % heads:
                raise ConfigError("head_dim is absent and hidden_size is no multiple of num_attention_heads")
            head_dim = int(raw["hidden_size"]) // heads
        use_window = bool(raw.get("use_sliding_window", False))
        window = raw.get("sliding_window")
        cfg = cls(
            hidden_size=int(raw["hidden_size"]),
            intermediate_size=int(raw["intermediate_size"]),
            num_hidden_layers=int(raw["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=int(raw["num_key_value_heads"]),
            head_dim=int(head_dim),
            vocab_size=int(raw["vocab_size"]),
            rms_norm_eps=float(raw["rms_norm_eps"]),
            rope_theta=float(raw["rope_theta"]),
            max_position_embeddings=int(raw["max_position_embeddings"]),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            use_sliding_window=use_window,
            sliding_window=int(window) if (use_window and window is not None) else None,
            max_window_layers=int(raw.get("max_window_layers", 0)) if use_window else 0,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for f in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"{f} must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim must be even for the rotary encoding, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be positive")
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            raise ConfigError("use_sliding_window is set but sliding_window is not a positive number")

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3"}
        for f in fields(self):
            out[f.name] = getattr(self, f.name)
        out["attention_bias"] = False
        out["hidden_act"] = "silu"
        return out

    def layer_window(self, layer: int) -> int:
        if self.use_sliding_window and self.sliding_window and layer >= self.max_window_layers:
            return int(self.sliding_window)
        return 0

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"width": self.hidden_size, "eps": self.rms_norm_eps})
        position = PartSpec("rotary", {"dim": self.head_dim, "theta": self.rope_theta})
        layers = []
        for l in range(self.num_hidden_layers):
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qk_norm_eps": self.rms_norm_eps,
                "window": self.layer_window(l),
                "scale": self.head_dim ** -0.5,
            })
            ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                      "intermediate_size": self.intermediate_size})
            layers.append(LayerSpec(
                prefix=f"model.layers.{l}", block=PartSpec("pre_norm"), mixer=mixer, feed_forward=ffn,
                mixer_norm=norm, feed_forward_norm=norm, position=position))
        return ModelSpec(
            architecture="Qwen3ForCausalLM",
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size,
                                                   "width": self.hidden_size}),
            final_norm=norm,
            head=PartSpec("linear_head", {"vocab_size": self.vocab_size, "width": self.hidden_size,
                                          "tied": self.tie_word_embeddings}),
            layers=tuple(layers),
            schedule=tuple(LayerRun(layer=l, cache=l) for l in range(self.num_hidden_layers)),
        )
