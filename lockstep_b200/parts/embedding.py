"""Token embedding (a gather into the float32 residual stream; LockStep:
engine/model/qwen3.py:319) and the output head (logits = y @ W^T, float32 out;
engine/model/qwen3.py:373), whose weight may be the embedding table itself."""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import Part, Runtime, WeightSpec, register_part


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, width: int, runtime: Runtime):
        self.vocab, self.width, self.rt = int(vocab_size), int(width), runtime
        self.table = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.vocab, self.width), "table")}

    def bind(self, tensors):
        self.table = tensors["weight"]

    def forward(self, ctx) -> torch.Tensor:
        """The float32 residual stream [tokens, width] of the step's tokens.  An
        embedding that encodes absolute positions would add them here (``ctx.positions``)."""
        ids = ctx.token_ids
        h = self.rt.rows(ids.numel(), self.width, dtype=torch.float32)
        K.embed_gather(ids, self.table, h, self.rt.err)
        return h


class LinearHead(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, width: int, tied: bool, runtime: Runtime):
        self.vocab, self.width, self.tied, self.rt = int(vocab_size), int(width), bool(tied), runtime
        self.weight = None

    def weight_specs(self):
        return {} if self.tied else {"weight": WeightSpec((self.vocab, self.width))}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        logits = self.rt.rows(y.shape[0], self.vocab, dtype=torch.float32)
        K.gemm_nt(y, self.weight, logits, err=self.rt.err)
        return logits


@register_part("embedding", "token_embedding")
def _build_embedding(spec, runtime, **_):
    return TokenEmbedding(spec["vocab_size"], spec["width"], runtime)


@register_part("head", "linear_head")
def _build_head(spec, runtime, **_):
    return LinearHead(spec["vocab_size"], spec["width"], spec.get("tied", False), runtime)
