"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * gain, all in float32
(LockStep: engine/kernels/rmsnorm.py:30-38)."""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import Norm, Runtime, WeightSpec, register_part


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, runtime: Runtime):
        self.width, self.eps, self.rt = int(width), float(eps), runtime
        self.gain: torch.Tensor | None = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.width,), "gain")}

    def bind(self, tensors):
        self.gain = tensors["weight"]

    def forward(self, h, row_index=None):
        rows = h.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((rows, self.width), dtype=self.rt.dtype, device=h.device)
        K.rmsnorm(h, self.gain, out, self.eps, self.rt.err, row_index)
        return out


@register_part("norm", "rmsnorm")
def _build(spec, runtime, **_):
    return RMSNorm(spec["width"], spec["eps"], runtime)
