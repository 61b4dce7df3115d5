"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * gain, all in float32
(LockStep: engine/kernels/rmsnorm.py:30-38)."""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import Norm, Runtime, WeightSpec, register_part


class NormedRows:
    """Rows that are still to be normalised: a mixer or feed-forward that can make the
    norm inside its first product takes ``h``, ``gain`` and ``eps`` from here; any other
    calls ``materialize()`` and gets the tensor ``Norm.forward`` would have returned."""

    def __init__(self, norm: "RMSNorm", h: torch.Tensor, row_index=None):
        self.norm, self.h, self.row_index = norm, h, row_index
        self.gain, self.eps = norm.gain, norm.eps
        self._out = None

    def pending(self) -> bool:
        """True while nobody has asked for the normalised tensor (a product may still make it)."""
        return self._out is None

    def materialize(self) -> torch.Tensor:
        if self._out is None:
            self._out = self.norm.forward(self.h, self.row_index)
        return self._out

    def linear(self, w: torch.Tensor, out: torch.Tensor, epilogue: int, err: torch.Tensor) -> None:
        """out = epilogue(norm(h) @ w.T): fused where the kernel allows, else norm, then product."""
        if self._out is None and K.gemm_nt_tc_rmsnorm(self.h, self.gain, self.eps, w, out, epilogue, err,
                                                      self.row_index):
            return
        K.gemm_nt(self.materialize(), w, out, epilogue, err=err)


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, runtime: Runtime):
        self.width, self.eps, self.rt = int(width), float(eps), runtime
        self.gain: torch.Tensor | None = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.width,), "gain")}

    def bind(self, tensors):
        self.gain = tensors["weight"]

    def lazy(self, h, row_index=None) -> NormedRows:
        """The rows of ``h`` to be normalised, for a part that sets ``accepts_normed_rows``."""
        return NormedRows(self, h, row_index)

    def forward(self, h, row_index=None):
        rows = h.shape[0] if row_index is None else row_index.numel()
        out = self.rt.rows(rows, self.width)
        K.rmsnorm(h, self.gain, out, self.eps, self.rt.err, row_index)
        return out


@register_part("norm", "rmsnorm")
def _build(spec, runtime, **_):
    return RMSNorm(spec["width"], spec["eps"], runtime)
