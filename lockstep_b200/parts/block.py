"""Arrangement of a layer's parts.  "pre_norm":
h += mixer(norm_a(h)); h += feed_forward(norm_b(h))  (LockStep: engine/model/qwen3.py:242-287).
The names under which the layer's tensors are stored are parameters of the
arrangement, so the same arrangement serves architectures that name them otherwise."""

from __future__ import annotations

from .base import Block, Runtime, build_part, register_part

_DEFAULT_NAMES = {
    "mixer_norm": "input_layernorm",
    "mixer": "self_attn",
    "feed_forward_norm": "post_attention_layernorm",
    "feed_forward": "mlp",
}


class PreNormBlock(Block):
    def __init__(self, layer_spec, runtime: Runtime):
        names = dict(_DEFAULT_NAMES)
        names.update(layer_spec.block.get("names", {}) or {})
        self.names = names
        self.position = build_part("position", layer_spec.position, runtime)
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime, position=self.position)
        self.feed_forward_norm = build_part("norm", layer_spec.feed_forward_norm, runtime)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, runtime)

    def _children(self):
        return [(self.names[k], getattr(self, k)) for k in _DEFAULT_NAMES]

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return all(part.graph_safe for _, part in self._children()) and self.position.graph_safe

    def attention_windows(self):
        return set().union(*(part.attention_windows() for _, part in self._children()))

    def weight_specs(self):
        out = {}
        for name, part in self._children():
            for local, spec in part.weight_specs().items():
                out[f"{name}.{local}"] = spec
        return out

    def bind(self, tensors):
        for name, part in self._children():
            own = {k[len(name) + 1:]: v for k, v in tensors.items() if k.startswith(name + ".")}
            if own or part.weight_specs():
                part.bind(own)

    @staticmethod
    def _normed(norm, consumer, h):
        """Rows for ``consumer``: still to be normalised where it can fuse the norm, else the tensor."""
        if consumer.accepts_normed_rows and hasattr(norm, "lazy"):
            return norm.lazy(h)
        return norm.forward(h)

    def _mix(self, h, ctx, cache):
        self.mixer.forward(self._normed(self.mixer_norm, self.mixer, h), ctx, cache, h)

    def _feed_forward(self, h, ctx, cache):
        self.feed_forward.forward(self._normed(self.feed_forward_norm, self.feed_forward, h), ctx, h)

    def steps(self):
        return [(bool(self.mixer_norm.graph_safe and self.mixer.graph_safe and self.position.graph_safe), self._mix),
                (bool(self.feed_forward_norm.graph_safe and self.feed_forward.graph_safe), self._feed_forward)]

    def forward(self, h, ctx, cache):
        self._mix(h, ctx, cache)
        self._feed_forward(h, ctx, cache)


@register_part("block", "pre_norm")
def _build(spec, runtime, layer_spec=None, **_):
    return PreNormBlock(layer_spec, runtime)
