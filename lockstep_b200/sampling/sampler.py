"""Sampling of next tokens on the device.

Greedy (temperature <= 0): argmax with ties to the lowest id.  Otherwise
temperature and nucleus (top-p) sampling as LockStep defines it
(engine/sampler/philox.py:71-98): softmax(logits / T), rank by (-p, id), keep
the shortest head whose mass reaches top_p, inverse CDF over the head with the
Philox draw for (seed, uid, position).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from . import philox


@dataclass
class SamplingParams:
    uid: str
    seed: int = 0
    temperature: float = 0.0
    top_p: float = 1.0
    position: int = 0        # position of the last context token


def _as_int32(words: list[int]) -> list[int]:
    return [w - (1 << 32) if w >= (1 << 31) else w for w in words]


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._probs = None

    def sample(self, logits: torch.Tensor, params: list[SamplingParams]) -> list[int]:
        """One token per row of ``logits`` [rows, vocab] (float32, on the device)."""
        if logits.shape[0] == 0:
            return []
        return self.sample_device(logits, params).tolist()

    def sample_device(self, logits: torch.Tensor, params: list[SamplingParams]) -> torch.Tensor:
        """As ``sample``, but the tokens stay on the device (int32 [rows])."""
        rows, vocab = logits.shape
        if rows != len(params):
            raise ValueError("one SamplingParams per row of logits")
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if rows == 0:
            return out
        if all(p.temperature <= 0 for p in params):
            K.argmax(logits, out)
            return out
        for p in params:
            if p.temperature > 0 and not 0 < p.top_p <= 1:
                raise ValueError(f"{p.uid}: top_p must lie in (0, 1], got {p.top_p}")
        flat = []
        for p in params:
            k0, k1 = philox.key_words(p.seed, p.uid)
            flat.extend(_as_int32([k0, k1, p.position & 0xFFFFFFFF, (p.position >> 32) & 0xFFFFFFFF]))
        words = torch.tensor(flat, dtype=torch.int32).view(rows, 4)
        keys = words[:, :2].contiguous().to(self.device)
        positions = words[:, 2:].contiguous().to(self.device)
        temperature = torch.tensor([max(0.0, p.temperature) for p in params], dtype=torch.float32,
                                   device=self.device)
        top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32, device=self.device)
        if self._probs is None or self._probs.shape[0] < rows or self._probs.shape[1] != vocab:
            self._probs = torch.empty((rows, vocab), dtype=torch.float32, device=self.device)
        K.sample(logits, self._probs[:rows], temperature, top_p, keys, positions, out)
        return out
