"""Continuous batching above the step function (after LockStep's
engine/sched/scheduler.py, with a token budget and lazy page reservation).

Each step: admit waiting requests while slots and pages allow; give every
decoding request its one token first, then cut the prompts of the others into
portions under the step's token budget, oldest first; run the batch; sample for
the requests whose context is now complete; finish and free.

When pages run out: pages are taken step by step as a request grows, so a step
may find the pool short.  Then cached prefix pages that no request holds are
evicted first; if that is not enough the most recently admitted running request
is preempted (its pages are given back, its tokens kept, it returns to the front
of the queue and is computed again when readmitted); a request that cannot run
even alone raises ``OutOfPages``.  A request larger than the whole pool is
refused at ``submit``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..cache import OutOfPages, PrefixIndex
from ..sampling import SamplingParams
from .batch import StepEntry
from .lifecycle import Lifecycle
from .policy import DefaultPolicy, Policy, SchedulerState
from .trajectory import Trajectory


@dataclass(eq=False)
class Request:
    """r = (uid, prompt, sampling parameters, seed); names as in LockStep
    (engine/sched/scheduler.py:19-28).  A request is itself, not its fields: two requests
    are equal only if they are the same object, so membership in the scheduler's lists is a
    comparison of identities."""

    uid: str
    prompt: list[int]
    seed: int = 0
    max_new_tokens: int = 8
    temperature: float = 0.0
    top_p: float = 1.0

    generated: list[int] = field(default_factory=list)
    finished: bool = False
    kv_len: int = 0
    preempt_count: int = 0
    cache_hit_tokens: int = 0

    def context(self) -> list[int]:
        return self.prompt + self.generated

    def total_tokens(self) -> int:
        return len(self.prompt) + len(self.generated)

    def tokens(self, start: int, end: int) -> list[int]:
        """context()[start:end] without building the whole context."""
        n = len(self.prompt)
        if end <= n:
            return self.prompt[start:end]
        if start >= n:
            return self.generated[start - n:end - n]
        return self.prompt[start:] + self.generated[:end - n]


class OversizedRequest(ValueError):
    """A request that cannot fit even when the pool is empty."""


class Scheduler:
    """``backend`` gives ``cache`` (a CacheManager), ``step(entries) -> logits``
    and ``sample(logits, params) -> tokens``; ``ModelRunner`` with a ``Sampler``
    is one, a host-side fake is another (the scheduler's decisions are tested
    without a device).

    A backend with ``supports_run_ahead`` also gives ``sample_async(logits, params) ->
    pending`` (tokens stay on the device, their copy to the host is under way),
    ``collect(pending) -> tokens``, ``can_step_ahead(entries)`` and ``step_ahead(entries,
    pending) -> logits`` (a decode step whose token ids are the pending ones, taken on the
    device).  While every running request only decodes and none can end by its token count,
    the scheduler then launches step n + 1 before it waits for the tokens of step n, so the
    host's share of a step runs beside the device's.  A request that ends on an end token
    at step n has one more token computed at step n + 1, which is dropped; the other rows of
    that step do not depend on it."""

    def __init__(self, backend, max_step_tokens: int = 2048, policy: Policy | None = None,
                 eos_token_ids=None, audit: bool = False, enable_prefix_cache: bool = False,
                 max_running: int = 32, trajectory: bool = False):
        self.backend = backend
        self.cache = backend.cache
        self.max_step_tokens = int(max_step_tokens)
        if self.max_step_tokens < 1:
            raise ValueError("max_step_tokens must be at least 1")
        self.policy = policy or DefaultPolicy(max_running=max_running)
        self.eos = set(eos_token_ids or ())
        self.audit_enabled = audit
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self.done: list[Request] = []
        self.step_index = 0
        self.events: list[tuple] = []          # (step, event, uid, detail)
        self.lifecycle = Lifecycle()           # every event is checked against the table of legal ones
        # trajectory=True: every step's work, tokens, logits bytes and cache digests go into one
        # running hash (the logits rows are read back each step, so no step is launched ahead)
        self.trajectory = Trajectory() if trajectory else None
        self.stats = {"preemptions": 0, "evictions": 0, "steps": 0, "tokens_run": 0,
                      "mixed_steps": 0, "budget_cuts": 0, "launched_ahead": 0}
        self._ahead = None                     # a launched step whose tokens have not been collected
        self._step_limit = 1 << 62
        self.prefix = None
        if enable_prefix_cache:
            if self.cache.states or not self.cache.paged:
                raise ValueError("prefix reuse shares pages of keys and values: a model that keeps a "
                                 "fixed-size state per request cannot take part")
            self.prefix = PrefixIndex(page_size=self.cache.page_size)
            self.cache.keep_boundary_windows()

    # -- bookkeeping ----------------------------------------------------------
    def _event(self, name: str, uid: str, detail=()):
        self.lifecycle.observe(uid, name)
        self.events.append((self.step_index, name, uid, tuple(detail)))

    def _pages_for(self, tokens: int) -> int:
        return self.cache.peak_pages(tokens, min(tokens, self.max_step_tokens))

    def _reclaimable(self) -> int:
        """How many more pages evictions can add to ``cache.free_pages()`` (the scarcest group's count)."""
        if not self.prefix:
            return 0
        groups = self.cache.paged
        gain = self.prefix.reclaimable(groups)
        return min(g.allocator.free_pages + n for g, n in zip(groups, gain)) - self.cache.free_pages()

    def _state(self) -> SchedulerState:
        return SchedulerState(
            step=self.step_index, waiting=tuple(r.uid for r in self.waiting),
            running=tuple(r.uid for r in self.running), free_blocks=self.cache.free_pages(),
            total_blocks=self.cache.total_pages(), reclaimable_blocks=self._reclaimable())

    def submit(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"{request.uid}: the prompt is empty")
        total = len(request.prompt) + request.max_new_tokens
        if self._pages_for(total) > self.cache.total_pages() or total > self.cache.max_seq_len:
            raise OversizedRequest(
                f"{request.uid} needs {self._pages_for(total)} pages ({len(request.prompt)} prompt + "
                f"{request.max_new_tokens} new tokens at page size {self.cache.page_size}) but the pool "
                f"holds {self.cache.total_pages()} and a sequence at most {self.cache.max_seq_len} tokens")
        if any(r.uid == request.uid for r in self.waiting + self.running):
            raise ValueError(f"a request with uid {request.uid!r} is already queued")
        self.waiting.append(request)

    # -- admission ------------------------------------------------------------
    def _admit(self, request: Request, state: SchedulerState) -> None:
        self.cache.create(request.uid)
        request.kv_len = 0
        request.cache_hit_tokens = 0
        self._event("resume" if request.preempt_count else "admit", request.uid)
        if self.prefix is not None:
            context = request.context()
            # (at most all but the last token: something is left to compute)
            hit, pages = self.prefix.lookup(context, self.cache.paged, limit=len(context) - 1)
            if hit and self.policy.honor_cache_hit(state, request.uid, hit):
                for group, held in zip(self.cache.paged, pages):
                    group.adopt(request.uid, held)
                request.kv_len = request.cache_hit_tokens = hit
                self.cache.lengths[request.uid] = hit
                self._event("cache_hit", request.uid, (hit,))

    def _preempt(self, request: Request) -> None:
        self.cache.release(request.uid)
        request.kv_len = 0
        request.preempt_count += 1
        self.running.remove(request)
        self.waiting.insert(0, request)
        self.stats["preemptions"] += 1
        self._event("preempt", request.uid)

    def _make_room(self, request: Request, tokens: int, planned: list) -> bool:
        """Reserve pages so that ``request`` holds ``tokens``; evict, then preempt
        younger requests, as needed.  False if the request itself had to go."""
        while True:
            if self.cache.can_reserve(request.uid, tokens):
                self.cache.reserve(request.uid, tokens)
                return True
            if self.prefix is not None:
                candidates = self.prefix.evictable(self.cache.paged)
                if candidates:
                    victim = self.policy.evict_victim(self._state(), tuple(candidates))
                    if victim not in candidates:
                        raise ValueError(f"policy {self.policy.name} chose page {victim}, which is not evictable")
                    self.prefix.evict(victim, self.cache.paged)
                    self.stats["evictions"] += 1
                    self._event("evict", request.uid, (victim,))
                    continue
            victim = self.running[-1]
            if victim is request:
                if len(self.running) == 1:
                    raise OutOfPages(
                        f"{request.uid} needs {self.cache.pages_short(request.uid, tokens)} more pages, "
                        f"{self.cache.free_pages()} are free and no other request holds any")
                self._preempt(request)
                return False
            planned[:] = [p for p in planned if p[0] is not victim]
            self._preempt(victim)

    # -- one step ---------------------------------------------------------------
    def step(self) -> bool:
        if self._ahead is not None:
            launched, self._ahead = self._ahead, None
        else:
            launched = self._plan_and_launch()
            if launched is None:
                return False
            if launched is True:
                return True
        # the next step goes out before this one's tokens are waited for, where that is safe
        if self._can_run_ahead(launched):
            self._ahead = self._launch_ahead(launched)
        self._collect(launched)
        self.step_index += 1
        return True

    def _plan_and_launch(self):
        """Admission, preemption and the plan of one step, and its launch.  None: nothing is
        queued; True: a step went by without work for the device; else the launched step."""
        if not self.waiting and not self.running:
            return None
        state = self._state()
        for request in list(self.waiting):
            need = self._pages_for(request.total_tokens() + 1)
            if not self.cache.has_slot() or not self.policy.admit(state, request.uid, need):
                continue
            self.waiting.remove(request)
            self._admit(request, state)
            self.running.append(request)
            state = self._state()
        if not self.running:
            smallest = min(self._pages_for(r.total_tokens() + 1) for r in self.waiting)
            raise OutOfPages(
                f"{len(self.waiting)} requests waiting, the smallest needs {smallest} pages, "
                f"{self.cache.free_pages()} free, nothing running that could free more")

        for request in list(self.running):
            if request.kv_len and request.generated and self.policy.should_preempt(state, request.uid):
                self._preempt(request)
                state = self._state()
        if not self.running:
            self.step_index += 1
            return True

        # decoding requests first, then prompts, each group oldest first
        budget = self.max_step_tokens
        planned: list[tuple[Request, int]] = []
        order = [r for r in self.running if r.total_tokens() - r.kv_len == 1] + \
                [r for r in self.running if r.total_tokens() - r.kv_len > 1]
        for request in order:
            if request not in self.running or budget <= 0:
                continue
            remaining = request.total_tokens() - request.kv_len
            take = self.policy.chunk_boundary(state, request.uid, remaining)
            if not 1 <= take <= remaining:
                raise ValueError(f"policy {self.policy.name} returned a portion of {take} for "
                                 f"{request.uid} with {remaining} remaining")
            if take > budget:
                take = budget
                self.stats["budget_cuts"] += 1
            if self._make_room(request, request.kv_len + take, planned):
                planned.append((request, take))
                budget -= take
        planned = [(r, n) for r, n in planned if r in self.running]
        if not planned:
            self.step_index += 1
            return True
        return self._launch(planned)

    def _launch(self, planned, ahead_of=None):
        """Run the planned portions on the backend and start sampling; the tokens are taken
        in ``_collect``.  ``ahead_of``: the launched step whose tokens this one feeds on."""
        entries = []
        for request, take in planned:
            start = request.kv_len
            last = ahead_of is not None or start + take == request.total_tokens()
            tokens = [0] if ahead_of is not None else request.tokens(start, start + take)
            entries.append(StepEntry(uid=request.uid, tokens=tokens, start=start, want=[take - 1] if last else []))
            self._event("decode" if last else "chunk", request.uid, (start, take))
        kinds = {len(e.tokens) == 1 for e in entries}
        if len(kinds) == 2:
            self.stats["mixed_steps"] += 1
        if ahead_of is not None:
            logits = self.backend.step_ahead(entries, ahead_of["pending"])
        else:
            logits = self.backend.step(entries)
        self.stats["steps"] += 1
        self.stats["tokens_run"] += sum(len(e.tokens) for e in entries)

        params, owners = [], []
        for (request, take), e in zip(planned, entries):
            request.kv_len = e.start + take
            if e.want:
                # the position of the last token fed: the last context position
                params.append(SamplingParams(uid=request.uid, seed=request.seed,
                                             temperature=request.temperature, top_p=request.top_p,
                                             position=e.start + take - 1))
                owners.append(request)
        launched = {"planned": planned, "owners": owners, "params": params, "logits": logits, "pending": None,
                    "work": [(e.uid, e.start, list(e.tokens)) for e in entries]}
        if getattr(self.backend, "supports_run_ahead", False):
            launched["pending"] = self.backend.sample_async(logits, params)
        return launched

    def _collect(self, launched) -> None:
        """Take the tokens of a launched step, append them, finish what has ended."""
        if launched["pending"] is not None:
            tokens = self.backend.collect(launched["pending"])
        else:
            tokens = self.backend.sample(launched["logits"], launched["params"])   # also reports device faults
        owners = []
        for request, token in zip(launched["owners"], tokens):
            if request.finished or request not in self.running:
                continue                      # ended on an end token while this step was under way
            request.generated.append(int(token))
            owners.append(request)
        if self.trajectory is not None:
            rows = launched["logits"]
            raw = rows.detach().cpu().contiguous().numpy().tobytes() if hasattr(rows, "detach") else repr(rows).encode()
            self.trajectory.observe_step(
                self.step_index, launched["work"],
                [(r.uid, r.generated[-1]) for r in owners], raw,
                (self.cache.digest(), self.prefix.digest() if self.prefix is not None else ()))

        if self.audit_enabled:
            self.cache.audit()
            if self.prefix is not None:
                self.prefix.audit()

        for request in owners:
            if len(request.generated) >= request.max_new_tokens or request.generated[-1] in self.eos:
                request.finished = True
                self.running.remove(request)
                self.done.append(request)
                if self.prefix is not None:
                    self.prefix.insert(request.context()[:request.kv_len], self.cache.paged, request.uid)
                self.cache.release(request.uid)
                self._event("finish", request.uid)

    def _can_run_ahead(self, launched) -> bool:
        """True if the step after ``launched`` is known now: the same requests, one more token
        each, whatever the tokens turn out to be (but for an end token, see the class)."""
        if launched["pending"] is None or self.waiting or self.audit_enabled or self.prefix is not None:
            return False
        if self.trajectory is not None:
            return False
        if not self.policy.allows_run_ahead or self.step_index + 2 > self._step_limit:
            return False
        planned = launched["planned"]
        if len(launched["owners"]) != len(planned) or len(planned) != len(self.running):
            return False
        for request, take in planned:
            # after the token under way it must still want another
            if take != 1 or len(request.generated) + 2 > request.max_new_tokens:
                return False
            if request.kv_len + 1 > self.cache.max_seq_len:
                return False
        # and all of them together must fit without making room: several requests may cross a
        # page edge in the same step, so the pages are counted for the whole step, group by group
        if not self.cache.can_reserve_all([(request.uid, request.kv_len + 1) for request, _ in planned]):
            return False
        entries = [StepEntry(uid=r.uid, tokens=[0], start=r.kv_len, want=[0]) for r, _ in planned]
        return self.backend.can_step_ahead(entries)

    def _launch_ahead(self, launched):
        planned = [(request, 1) for request, _ in launched["planned"]]
        for request, _ in planned:
            self.cache.reserve(request.uid, request.kv_len + 1)
        self.stats["launched_ahead"] += 1
        return self._launch(planned, ahead_of=launched)

    def drain(self) -> None:
        """Collect a step that was launched ahead (its tokens are appended)."""
        if self._ahead is not None:
            launched, self._ahead = self._ahead, None
            self._collect(launched)
            self.step_index += 1

    def run(self, max_steps: int = 1 << 30) -> dict[str, list[int]]:
        self._step_limit = max_steps
        try:
            while self.step_index < max_steps and self.step():
                pass
            self.drain()
        finally:
            self._step_limit = 1 << 62
        if self.audit_enabled:
            self.cache.audit()
        return {r.uid: list(r.generated) for r in self.done}
