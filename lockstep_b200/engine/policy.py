"""The seam through which every scheduling decision goes
(names and meanings as in LockStep's engine/sched/policy.py:51-103)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SchedulerState:
    """What a policy may see when it decides."""

    step: int
    waiting: tuple[str, ...]
    running: tuple[str, ...]
    free_blocks: int
    total_blocks: int
    reclaimable_blocks: int = 0


class Policy:
    name = "base"
    # True if the policy's answers for a step of decoding requests do not depend on the
    # tokens of the step before: the scheduler may then launch that step before it has them
    allows_run_ahead = False

    def admit(self, state: SchedulerState, uid: str, blocks_needed: int) -> bool:
        raise NotImplementedError

    def chunk_boundary(self, state: SchedulerState, uid: str, remaining: int) -> int:
        """How many of the ``remaining`` context tokens to run in this step (before
        the step's token budget is applied)."""
        raise NotImplementedError

    def should_preempt(self, state: SchedulerState, uid: str) -> bool:
        return False

    def evict_victim(self, state: SchedulerState, candidates: tuple[int, ...]) -> int:
        return min(candidates)

    def honor_cache_hit(self, state: SchedulerState, uid: str, hit_length: int) -> bool:
        return True


class DefaultPolicy(Policy):
    """Admit while there is room; run the whole remainder of a prompt (the token
    budget of the step cuts it)."""

    name = "default"
    allows_run_ahead = True

    def __init__(self, max_running: int = 32):
        self.max_running = max_running

    def admit(self, state, uid, blocks_needed):
        if len(state.running) >= self.max_running:
            return False
        return blocks_needed <= state.free_blocks + state.reclaimable_blocks

    def chunk_boundary(self, state, uid, remaining):
        return remaining


class FixedChunkPolicy(DefaultPolicy):
    def __init__(self, chunk: int, max_running: int = 32):
        super().__init__(max_running)
        self.chunk = int(chunk)
        self.name = f"fixed-chunk({chunk})"

    def chunk_boundary(self, state, uid, remaining):
        return min(self.chunk, remaining)


class ScriptedPolicy(DefaultPolicy):
    """Portions from a cyclic plan, preemption of named requests at named steps."""

    allows_run_ahead = False          # it preempts at steps it names: every step is planned

    def __init__(self, chunk_plan=(), preempt_at=(), max_running: int = 32):
        super().__init__(max_running)
        self.chunk_plan = tuple(int(c) for c in chunk_plan)
        self.preempt_at = {(int(s), str(u)) for s, u in preempt_at}
        self._next: dict[str, int] = {}
        self.name = "scripted"

    def chunk_boundary(self, state, uid, remaining):
        if not self.chunk_plan or remaining == 1:
            return remaining
        i = self._next.get(uid, 0)
        self._next[uid] = i + 1
        return max(1, min(self.chunk_plan[i % len(self.chunk_plan)], remaining))

    def should_preempt(self, state, uid):
        if (state.step, uid) in self.preempt_at:
            self.preempt_at.discard((state.step, uid))
            return True
        return False
