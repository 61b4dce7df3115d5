"""A record of what the engine did, step by step, as one running sha256
(after LockStep's engine/audit/trajectory.py:15-59).

Each step absorbs its index, its work list (request, start, tokens), the tokens
it emitted, the raw bytes of the logits rows they were sampled from and the
digests of the cache manager and of the prefix index.  Two runs with the same
digest were the same execution: same batches, same bits, same pages.
``first_divergence`` names the first step at which two records part.
"""

from __future__ import annotations

import hashlib


class Trajectory:
    def __init__(self, constants_digest: str = ""):
        self._digest = hashlib.sha256()
        self.per_step: list[str] = []
        if constants_digest:
            self._absorb("constants", constants_digest.encode("ascii"))

    def _absorb(self, label: str, payload: bytes) -> None:
        self._digest.update(label.encode("utf-8"))
        self._digest.update(len(payload).to_bytes(8, "big"))
        self._digest.update(payload)

    def observe_step(self, step: int, work, emitted, logits_bytes: bytes, cache_state) -> None:
        """work: [(uid, start, token ids)]; emitted: [(uid, token)]; logits_bytes: the rows the
        tokens were sampled from, in the order of ``emitted``; cache_state: anything with a
        stable ``repr`` (the managers' digests)."""
        self._absorb("step", str(int(step)).encode())
        self._absorb("work", repr([(u, int(s), [int(t) for t in toks]) for u, s, toks in work]).encode())
        self._absorb("emitted", repr([(u, int(t)) for u, t in emitted]).encode())
        self._absorb("logits", logits_bytes)
        self._absorb("cache", repr(cache_state).encode())
        self.per_step.append(self._digest.hexdigest())

    @property
    def steps(self) -> int:
        return len(self.per_step)

    def hexdigest(self) -> str:
        return self._digest.hexdigest()

    def first_divergence(self, other: "Trajectory") -> int | None:
        """The first step at which the two records differ; None if they agree throughout."""
        for i, (mine, theirs) in enumerate(zip(self.per_step, other.per_step)):
            if mine != theirs:
                return i
        if len(self.per_step) != len(other.per_step):
            return min(len(self.per_step), len(other.per_step))
        return None
