"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases, added into the
residual stream (LockStep: engine/model/qwen3.py:285-287, engine/kernels/swiglu.py:25-29).
gate and up are one product over the row-concatenated weights, with the
activation in that product's epilogue."""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import FeedForward, Runtime, WeightSpec, register_part
from .norm import NormedRows


class SwiGLU(FeedForward):
    graph_safe = True
    accepts_normed_rows = True

    def __init__(self, hidden_size: int, intermediate_size: int, runtime: Runtime):
        self.h, self.i, self.rt = int(hidden_size), int(intermediate_size), runtime
        self.w_gate_up = self.w_down = None

    def weight_specs(self):
        return {
            "gate_proj.weight": WeightSpec((self.i, self.h)),
            "up_proj.weight": WeightSpec((self.i, self.h)),
            "down_proj.weight": WeightSpec((self.h, self.i)),
        }

    def bind(self, tensors):
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def forward(self, x, ctx, residual):
        act = self.rt.rows(residual.shape[0], self.i)
        if isinstance(x, NormedRows):
            x.linear(self.w_gate_up, act, K.EPILOGUE_SILU_MUL, self.rt.err)
        else:
            K.gemm_nt(x, self.w_gate_up, act, K.EPILOGUE_SILU_MUL, err=self.rt.err)
        K.gemm_nt(act, self.w_down, residual, K.EPILOGUE_RESIDUAL, err=self.rt.err)


@register_part("feed_forward", "swiglu")
def _build(spec, runtime, **_):
    return SwiGLU(spec["hidden_size"], spec["intermediate_size"], runtime)
