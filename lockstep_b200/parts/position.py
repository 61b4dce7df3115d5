"""Position encodings.

"rotary": the half-rotation of LockStep (engine/kernels/rope.py:38-56) with
tables cos/sin[pos, i] of angle pos * theta^(-2i/dim), built in float64 on the
host and kept in float32 (engine/model/qwen3.py:117-129).  ``dim`` may be
smaller than the head size; the dimensions past it are left as they are.
"none": no position encoding.
"""

from __future__ import annotations

import torch

from .base import PositionEncoding, Runtime, register_part


class Rotary(PositionEncoding):
    graph_safe = True

    def __init__(self, dim: int, theta: float, runtime: Runtime):
        if dim % 2:
            raise ValueError(f"rotary dimension must be even, got {dim}")
        self.dim, self.theta = int(dim), float(theta)
        half = self.dim // 2
        exponent = torch.arange(0, half, dtype=torch.float64) * 2.0 / self.dim
        inv_freq = 1.0 / (self.theta ** exponent)
        pos = torch.arange(runtime.max_positions, dtype=torch.float64)
        ang = pos[:, None] * inv_freq[None, :]
        self.cos = ang.cos().to(torch.float32).to(runtime.device).contiguous()
        self.sin = ang.sin().to(torch.float32).to(runtime.device).contiguous()

    def rotary(self):
        return self.cos, self.sin, self.dim


class NoPosition(PositionEncoding):
    graph_safe = True


@register_part("position", "rotary")
def _build_rotary(spec, runtime, **_):
    return Rotary(spec["dim"], spec["theta"], runtime)


@register_part("position", "none")
def _build_none(spec, runtime, **_):
    return NoPosition()
