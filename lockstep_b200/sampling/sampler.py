"""Sampling of next tokens on the device.

Greedy (temperature <= 0): argmax with ties to the lowest id.  Otherwise
temperature and nucleus (top-p) sampling as LockStep defines it
(engine/sampler/philox.py:71-98): softmax(logits / T), rank by (-p, id), keep
the shortest head whose mass reaches top_p, inverse CDF over the head with the
Philox draw for (seed, uid, position).
"""

from __future__ import annotations

import functools
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
        self._host = None                     # pinned: one row of parameters a request, copied in one go
        self._copied = None                   # the last copy out of it

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
        # keys, positions, temperatures and nucleus sizes in one pinned buffer and one copy
        if self._host is None or self._host.numel() < 6 * rows:
            self._host = torch.empty(6 * max(rows, 64), dtype=torch.int32).pin_memory()
            self._copied = torch.cuda.Event()
        else:
            self._copied.synchronize()        # the copy before this one has read the buffer
        host = self._host[:6 * rows]
        words = host.numpy()
        reals = words.view("float32")
        for i, p in enumerate(params):
            k0, k1 = _key_words(p.seed, p.uid)
            words[2 * i], words[2 * i + 1] = _as_int32([k0, k1])
            words[2 * rows + 2 * i], words[2 * rows + 2 * i + 1] = _as_int32(
                [p.position & 0xFFFFFFFF, (p.position >> 32) & 0xFFFFFFFF])
            reals[4 * rows + i] = max(0.0, p.temperature)
            reals[5 * rows + i] = p.top_p
        dev = host.to(self.device, non_blocking=True)
        self._copied.record()
        keys, positions = dev[:2 * rows].view(rows, 2), dev[2 * rows:4 * rows].view(rows, 2)
        temperature, top_p = dev[4 * rows:5 * rows].view(torch.float32), dev[5 * rows:].view(torch.float32)
        need = K.sample_scratch_floats(rows, vocab)
        if need and (self._probs is None or self._probs.numel() < need):
            self._probs = torch.empty(need, dtype=torch.float32, device=self.device)
        K.sample(logits, self._probs if need else None, temperature, top_p, keys, positions, out)
        return out


@functools.lru_cache(maxsize=4096)
def _key_words(seed: int, uid: str) -> tuple[int, int]:
    return philox.key_words(seed, uid)
