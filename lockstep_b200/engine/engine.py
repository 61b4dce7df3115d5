"""The Python entry point: a model folder in, generated tokens out.

    engine = Engine("path/to/model", dtype="bfloat16")
    tokens = engine.generate([Request(uid="a", prompt=[1, 2, 3], max_new_tokens=16)])

``Engine`` puts the step function (``ModelRunner``), the device sampler and the
scheduler together.  ``generate_greedy`` and ``forward_batch`` keep the shape of
LockStep's ``Qwen3.generate_greedy`` and ``Qwen3.forward_batch``
(engine/model/qwen3.py:294-402).
"""

from __future__ import annotations

import torch

from .. import kernels as K
from ..sampling import Sampler
from .batch import StepEntry
from .policy import Policy
from .runner import ModelRunner
from .scheduler import Request, Scheduler


class Engine:
    def __init__(self, model_dir, dtype="bfloat16", device="cuda:0", num_pages: int | None = None,
                 page_size: int = 16, max_running: int = 32, max_step_tokens: int = 2048,
                 max_seq_len: int | None = None, enable_prefix_cache: bool = False,
                 eos_token_ids=None, policy: Policy | None = None, audit: bool = False,
                 trajectory: bool = False, poison_freed_pages: bool = False):
        if num_pages is None:
            num_pages = 4096
        self.runner = ModelRunner(model_dir, dtype=dtype, device=device, num_pages=num_pages,
                                  page_size=page_size, max_live=max_running, max_seq_len=max_seq_len,
                                  poison_freed_pages=poison_freed_pages)
        self.sampler = Sampler(self.runner.device)
        # two pinned buffers in turn (a step may be launched before the last one is collected):
        # sampled ids, then the two words of the device error word
        self._pinned = [torch.zeros(max_running + 2, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._pinned_turn = 0
        self.cache = self.runner.cache
        self.config = self.runner.config
        self._options = dict(max_step_tokens=max_step_tokens, policy=policy, eos_token_ids=eos_token_ids,
                             audit=audit, enable_prefix_cache=enable_prefix_cache, max_running=max_running,
                             trajectory=trajectory)
        self.scheduler = self._new_scheduler()

    def _new_scheduler(self) -> Scheduler:
        return Scheduler(self, **self._options)

    # backend interface of the scheduler
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        # the device error word is read after sampling, in one wait for the whole step
        return self.runner.step(entries, check=False, static_logits=True)

    def sample(self, logits, params) -> list[int]:
        tokens = self.sampler.sample(logits, params)
        K.raise_on_fault(self.runner.err)
        return tokens

    # run-ahead: the sampled tokens and the error word go to pinned memory by a copy that the
    # host waits for later, and the next decode step may take the tokens on the device
    supports_run_ahead = True

    def sample_async(self, logits, params) -> dict:
        tokens = self.sampler.sample_device(logits, params)
        n = tokens.numel()
        host = self._pinned[self._pinned_turn]
        self._pinned_turn ^= 1
        if n:
            host[:n].copy_(tokens, non_blocking=True)
        host[-2:].copy_(self.runner.err, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return {"tokens": tokens, "host": host, "n": n, "done": done}

    def collect(self, pending) -> list[int]:
        pending["done"].synchronize()
        host = pending["host"]
        code, detail = host[-2:].tolist()
        if code != 0:
            K.raise_on_fault(self.runner.err)
        return host[:pending["n"]].tolist()

    def can_step_ahead(self, entries) -> bool:
        return self.runner.can_step_ahead(entries)

    def step_ahead(self, entries, pending) -> torch.Tensor:
        return self.runner.step(entries, check=False, static_logits=True, tokens_device=pending["tokens"])

    # -- generation -------------------------------------------------------------
    def weight_cast_report(self) -> dict:
        """What the cast of the model folder's tensors to the engine's element types cost."""
        return self.runner.weight_cast_report()

    def submit(self, request: Request) -> None:
        self.scheduler.submit(request)

    def run(self, max_steps: int = 1 << 30) -> dict[str, list[int]]:
        return self.scheduler.run(max_steps)

    def generate(self, requests: list[Request], max_steps: int = 1 << 30) -> dict[str, list[int]]:
        """Run ``requests`` to completion with continuous batching; uid -> generated ids."""
        for r in requests:
            self.scheduler.submit(r)
        self.scheduler.run(max_steps)
        out = {r.uid: list(r.generated) for r in requests}
        self.scheduler.done = [r for r in self.scheduler.done if r not in requests]
        return out

    def generate_greedy(self, prompt_ids: list[int], max_new_tokens: int, eos_token_ids=None) -> list[int]:
        saved = self.scheduler.eos
        self.scheduler.eos = set(eos_token_ids or saved)
        try:
            uid = f"greedy-{self.scheduler.step_index}-{len(self.scheduler.done)}"
            return self.generate([Request(uid=uid, prompt=list(prompt_ids), max_new_tokens=max_new_tokens)])[uid]
        finally:
            self.scheduler.eos = saved

    def forward_batch(self, work: list[tuple[str, list[int], int]]) -> dict[str, torch.Tensor]:
        """One step over (uid, tokens, start) with logits for every fed position,
        as LockStep's ``forward_batch``; requests are opened on first use and stay
        open until ``release``."""
        entries = []
        for uid, tokens, start in work:
            if uid not in self.cache.slots:
                self.runner.open(uid)
            entries.append(StepEntry(uid=uid, tokens=list(tokens), start=start, want=list(range(len(tokens)))))
        logits = self.runner.step(entries)
        out, r = {}, 0
        for e in entries:
            out[e.uid] = logits[r:r + len(e.tokens)]
            r += len(e.tokens)
        return out

    def release(self, uid: str) -> None:
        self.runner.close(uid)
