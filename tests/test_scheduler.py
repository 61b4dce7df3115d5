"""The scheduler's decisions, on the host: a fake step function stands in for the model.

The fake's next token depends on the request's whole context, so any token that
the scheduler loses, repeats or feeds at a wrong position changes the output.
"""

from __future__ import annotations

import pytest

from lockstep_b200.cache import CacheManager, OutOfPages
from lockstep_b200.engine import (FixedChunkPolicy, OversizedRequest, Request, Scheduler, ScriptedPolicy)
from lockstep_b200.parts import CacheNeed

VOCAB = 97


def next_token(context):
    h = 7
    for i, t in enumerate(context):
        h = (h * 31 + t * (i + 1)) % 1000003
    return h % VOCAB


class FakeBackend:
    def __init__(self, pages=64, page=4, live=8, seq=4096, window=0, windows=None):
        needs = [CacheNeed("paged_kv", kv_heads=1, head_dim=16, window=w) for w in (windows or [window])]
        self.cache = CacheManager(needs, num_pages=pages, page_size=page, max_live=live,
                                  max_seq_len=seq, allocate=False)
        self.history: dict[str, list[int]] = {}
        self.steps: list[list[tuple[str, int, int]]] = []
        self.sampled = []

    def step(self, entries):
        out = []
        self.steps.append([(e.uid, e.start, len(e.tokens)) for e in entries])
        for e in entries:
            hist = self.history.setdefault(e.uid, [])
            if e.start < len(hist):        # recomputed after a preemption or a prefix hit
                del hist[e.start:]
            if e.start > len(hist):        # a prefix hit: the shared pages hold these tokens
                hist.extend([None] * (e.start - len(hist)))
            assert e.start == len(hist) == self.cache.lengths[e.uid]
            hist.extend(e.tokens)
            self.cache.reserve(e.uid, e.start + len(e.tokens))
            self.cache.advance(e.uid, e.start + len(e.tokens))
            for w in e.want:
                assert w == len(e.tokens) - 1
                out.append(e.uid)
        return out

    def sample(self, logits, params):
        self.sampled.extend(params)
        return [next_token(self._context[p.uid]()) for p in params]


def run(requests, **kw):
    backend_kw = {k: kw.pop(k) for k in ("pages", "page", "live", "seq", "window", "windows") if k in kw}
    backend = FakeBackend(**backend_kw)
    sched = Scheduler(backend, audit=True, **kw)
    backend._context = {}
    for r in requests:
        backend._context[r.uid] = r.context
        sched.submit(r)
    out = sched.run(max_steps=10000)
    return out, sched, backend


def expected(prompt, n, eos=()):
    ctx, out = list(prompt), []
    for _ in range(n):
        t = next_token(ctx)
        out.append(t)
        ctx.append(t)
        if t in eos:
            break
    return out


def make(n=5, new=9):
    return [Request(uid=f"r{i}", prompt=[(3 * i + 5 * j) % VOCAB for j in range(3 + 11 * i)],
                    max_new_tokens=new + i) for i in range(n)]


def test_generation_is_right_and_budget_is_kept():
    for budget in (1, 3, 8, 64, 4096):
        out, sched, backend = run(make(), max_step_tokens=budget)
        for r in make():
            assert out[r.uid] == expected(r.prompt, r.max_new_tokens), (budget, r.uid)
        assert all(sum(n for _, _, n in step) <= budget for step in backend.steps)
        assert sched.cache.free_pages() == sched.cache.total_pages()


def test_decoding_requests_go_first_and_prompts_are_cut():
    reqs = [Request("short", [1, 2], max_new_tokens=20), Request("long", list(range(50)), max_new_tokens=2)]
    out, sched, backend = run(reqs, max_step_tokens=8)
    mixed = [s for s in backend.steps if {n == 1 for _, _, n in s} == {True, False}]
    assert mixed and sched.stats["mixed_steps"] == len(mixed)
    for step in mixed:
        assert step[0][0] == "short" and step[0][2] == 1     # the decoded token leads
        assert step[1][0] == "long" and step[1][2] <= 7      # the prompt gets the rest of the budget
    assert sum(step[1][2] == 7 for step in mixed) >= 5
    assert sched.stats["budget_cuts"] > 0
    assert out["long"] == expected(list(range(50)), 2)


def test_portions_follow_the_policy_down_to_two_tokens():
    reqs = [Request("a", list(range(40)), max_new_tokens=3)]
    out, sched, backend = run(reqs, policy=ScriptedPolicy(chunk_plan=(7, 2, 17, 2)))
    sizes = [n for step in backend.steps for _, _, n in step]
    assert sizes[:5] == [7, 2, 17, 2, 7] and out["a"] == expected(list(range(40)), 3)
    out2, _, b2 = run([Request("a", list(range(40)), max_new_tokens=3)], policy=FixedChunkPolicy(16))
    assert [n for s in b2.steps for _, _, n in s][:3] == [16, 16, 8] and out2 == out


def test_when_pages_run_out_the_youngest_is_preempted_and_recomputed():
    reqs = make(4, new=30)
    # 12 pages of 4 tokens: the four requests need far more together than the pool has
    out, sched, backend = run(reqs, pages=24, page=4, max_step_tokens=16)
    assert sched.stats["preemptions"] > 0
    for r in make(4, new=30):
        assert out[r.uid] == expected(r.prompt, r.max_new_tokens), r.uid
    victims = [e[2] for e in sched.events if e[1] == "preempt"]
    assert "r0" not in victims                     # the oldest request is never the victim
    resumed = [e[2] for e in sched.events if e[1] == "resume"]
    assert set(resumed) == set(victims)
    assert sched.cache.free_pages() == 24 and sched.cache.reused_pages() > 0


def test_oversized_request_is_refused_at_submit():
    backend = FakeBackend(pages=4, page=4)
    sched = Scheduler(backend)
    with pytest.raises(OversizedRequest, match="needs 5 pages"):
        sched.submit(Request("big", list(range(10)), max_new_tokens=8))
    with pytest.raises(ValueError, match="empty"):
        sched.submit(Request("none", []))


def test_a_request_that_cannot_run_alone_raises():
    backend = FakeBackend(pages=4, page=4)
    sched = Scheduler(backend)
    backend._context = {}
    r = Request("a", list(range(10)), max_new_tokens=6)
    backend._context["a"] = r.context
    sched.submit(r)
    backend.cache.paged[0].allocator.take()        # a page that nothing will give back
    with pytest.raises(OutOfPages):
        sched.run()


def test_requests_wait_for_a_slot():
    out, sched, backend = run(make(6, new=4), live=2)
    assert max(len(s) for s in backend.steps) <= 2
    for r in make(6, new=4):
        assert out[r.uid] == expected(r.prompt, r.max_new_tokens)


def test_eos_finishes_early():
    r = Request("a", [5, 6, 7], max_new_tokens=50)
    full = expected(r.prompt, 50)
    eos = full[4]
    out, _, _ = run([r], eos_token_ids={eos})
    assert out["a"] == full[:full.index(eos) + 1]


def test_sampling_parameters_and_position():
    r = Request("a", [1, 2, 3, 4], seed=9, max_new_tokens=3, temperature=0.7, top_p=0.9)
    _, _, backend = run([r])
    assert [(p.position, p.seed, p.temperature, p.top_p) for p in backend.sampled] == \
        [(3, 9, 0.7, 0.9), (4, 9, 0.7, 0.9), (5, 9, 0.7, 0.9)]


def test_scripted_preemption_recomputes_the_context():
    reqs = [Request("a", list(range(9)), max_new_tokens=8), Request("b", [4, 4], max_new_tokens=8)]
    out, sched, backend = run(reqs, policy=ScriptedPolicy(preempt_at=[(3, "a")]))
    assert [e[2] for e in sched.events if e[1] == "preempt"] == ["a"]
    assert out["a"] == expected(list(range(9)), 8) and out["b"] == expected([4, 4], 8)
    again = [s for s in backend.steps if any(u == "a" and start == 0 for u, start, _ in s)]
    assert len(again) == 2                         # the prompt and, later, the whole context again


def test_prefix_reuse_skips_shared_pages_and_evicts_under_pressure():
    shared = list(range(20))
    first = Request("a", shared + [50, 51], max_new_tokens=4)
    out, sched, backend = run([first], pages=16, page=4, enable_prefix_cache=True)
    second = Request("b", shared + [60], max_new_tokens=4)
    backend._context["b"] = second.context
    sched.submit(second)
    sched.run()
    starts = [start for step in backend.steps for u, start, _ in step if u == "b"]
    assert starts[0] == 20 and second.cache_hit_tokens == 20     # five whole pages were adopted
    assert second.generated == expected(second.prompt, 4)
    big = Request("c", [9] * 40, max_new_tokens=8)               # needs the cached pages' room
    backend._context["c"] = big.context
    sched.submit(big)
    sched.run()
    assert sched.stats["evictions"] > 0 and big.generated == expected(big.prompt, 8)
    sched.cache.audit()


@pytest.mark.parametrize("new", [11, 14])       # the first turn ends on a page's edge, or three tokens past it
def test_prefix_reuse_with_a_windowed_group_serves_the_next_turn(new):
    """Layers that keep every key beside layers that keep a window of 12: a finished request's
    pages are indexed in both groups, the windowed one only has its last pages left.  The next
    turn of the same conversation adopts the whole prefix (all pages of the one group, the
    window's pages of the other); a request that shares only the beginning gets nothing, since
    the window's pages at that point were given back long ago."""
    first = Request("a", list(range(30)), max_new_tokens=new)
    out, sched, backend = run([first], pages=24, page=4, windows=[0, 12], seq=256, enable_prefix_cache=True)
    full, win = sched.cache.paged
    assert full.window == 0 and win.window == 12
    held = first.kv_len // 4                                    # whole pages of the 40 or 43 tokens it fed
    assert held == 10
    assert sched.prefix.reclaimable(sched.cache.paged) == [held, 3]   # keys 28.. of the window: pages 7, 8, 9
    turn = Request("b", first.context() + [70, 71, 72], max_new_tokens=5)
    backend._context["b"] = turn.context
    sched.submit(turn)
    sched.run()
    assert turn.cache_hit_tokens == held * 4
    starts = [start for step in backend.steps for u, start, _ in step if u == "b"]
    assert starts[0] == held * 4 and turn.generated == expected(turn.prompt, 5)
    other = Request("c", list(range(20)) + [80, 81], max_new_tokens=3)
    backend._context["c"] = other.context
    sched.submit(other)
    sched.run()
    assert other.cache_hit_tokens == 0 and other.generated == expected(other.prompt, 3)
    # under pressure the index gives everything back, in both groups
    big = Request("d", [9] * 70, max_new_tokens=8)
    backend._context["d"] = big.context
    sched.submit(big)
    sched.run()
    assert sched.stats["evictions"] > 0 and big.generated == expected(big.prompt, 8)
    sched.cache.audit()
    sched.prefix.audit()
    while sched.prefix.evictable(sched.cache.paged):
        sched.prefix.evict(sched.prefix.evictable(sched.cache.paged)[0], sched.cache.paged)
    assert not sched.prefix.entries
    assert full.allocator.free_pages == win.allocator.free_pages == 24


def test_prefix_reuse_is_refused_for_a_model_with_state_slots():
    backend = FakeBackend()
    backend.cache = CacheManager([CacheNeed("paged_kv", kv_heads=1, head_dim=16),
                                  CacheNeed("state", state_shape=(4,))], num_pages=8, page_size=4, max_live=2,
                                 max_seq_len=64, allocate=False)
    with pytest.raises(ValueError, match="fixed-size state"):
        Scheduler(backend, enable_prefix_cache=True)
    Scheduler(backend)


def test_windowed_group_frees_pages_while_decoding():
    r = Request("a", list(range(30)), max_new_tokens=60)
    out, sched, backend = run([r], pages=8, page=4, window=12, seq=128, max_step_tokens=16)
    assert out["a"] == expected(r.prompt, 60)      # 90 tokens went through 8 pages of 4
    with pytest.raises(OversizedRequest):          # a portion of 64 beside the window needs more
        run([Request("a", list(range(30)), max_new_tokens=60)], pages=8, page=4, window=12, seq=128,
            max_step_tokens=64)
    assert sched.cache.reused_pages() > 0


# -- run-ahead: the next decode step is launched before the last one's tokens are collected ----

class FakeAsyncBackend(FakeBackend):
    """A backend whose tokens "stay on the device": ``sample_async`` works them out from the
    tokens that were really fed (the fake's own history), ``step_ahead`` feeds them to the next
    step without the scheduler having seen them, ``collect`` hands them over."""

    supports_run_ahead = True

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.ahead_steps = 0
        self.uncollected = 0

    def sample_async(self, logits, params):
        self.sampled.extend(params)
        for p in params:                       # the position the scheduler names is the last one fed
            assert p.position == len(self.history[p.uid]) - 1
        self.uncollected += 1
        return {"uids": [p.uid for p in params], "tokens": [next_token(self.history[p.uid]) for p in params]}

    def collect(self, pending):
        self.uncollected -= 1
        return list(pending["tokens"])

    def can_step_ahead(self, entries):
        return all(len(e.tokens) == 1 and e.want == [0] for e in entries)

    def step_ahead(self, entries, pending):
        assert self.uncollected == 1           # the step it feeds on is still under way
        assert [e.uid for e in entries] == pending["uids"]
        for e, t in zip(entries, pending["tokens"]):
            assert e.tokens == [0]
            e.tokens = [t]
        self.ahead_steps += 1
        return self.step(entries)


def run_ahead(requests, late=(), **kw):
    backend_kw = {k: kw.pop(k) for k in ("pages", "page", "live", "seq", "window", "windows") if k in kw}
    backend = FakeAsyncBackend(**backend_kw)
    sched = Scheduler(backend, **kw)
    for r in requests:
        sched.submit(r)
    late = dict(late)
    while sched.step():
        for r in late.pop(sched.step_index, []):
            sched.submit(r)
    sched.drain()
    assert backend.uncollected == 0
    return {r.uid: list(r.generated) for r in sched.done}, sched, backend


def test_run_ahead_gives_the_same_tokens():
    reqs = [Request(uid=f"r{i}", prompt=[3 + i, 5, 8 + i] * (i + 1), max_new_tokens=4 + 3 * i) for i in range(4)]
    out, sched, backend = run_ahead(reqs)
    for r in reqs:
        assert out[r.uid] == expected(r.prompt, r.max_new_tokens)
    assert backend.ahead_steps > 0
    # no step after a request's last token: the count of tokens decides, and it is known ahead
    assert sched.stats["tokens_run"] == sum(len(r.prompt) + r.max_new_tokens - 1 for r in reqs)
    sched.cache.audit()
    assert sched.cache.free_pages() == sched.cache.total_pages()


def test_run_ahead_drops_the_token_after_an_end_token():
    prompt = [4, 9, 2, 7]
    full = expected(prompt, 40)
    eos = full[5]
    want = expected(prompt, 40, eos=(eos,))
    assert len(want) < 40
    other = Request(uid="other", prompt=[1, 2, 3], max_new_tokens=30)
    reqs = [Request(uid="ends", prompt=prompt, max_new_tokens=40), other]
    out, sched, backend = run_ahead(reqs, eos_token_ids=[eos])
    assert out["ends"] == want
    assert out["other"] == expected(other.prompt, 30, eos=(eos,))
    assert backend.ahead_steps > 0
    sched.cache.audit()
    assert sched.cache.free_pages() == sched.cache.total_pages()


def test_run_ahead_stops_for_arrivals_and_for_pages():
    first = Request(uid="a", prompt=[5, 6, 7], max_new_tokens=20)
    late = Request(uid="b", prompt=[9, 8, 7, 6, 5], max_new_tokens=6)
    out, sched, backend = run_ahead([first], late={6: [late]})
    assert out["a"] == expected(first.prompt, 20) and out["b"] == expected(late.prompt, 6)
    # b's prompt ran beside one of a's decoded tokens: that step was planned, not launched ahead
    assert any(len(step) == 2 and {n for _, _, n in step} == {1, 5} for step in backend.steps)
    # so few pages that a request is preempted: whatever is launched ahead, the tokens are the same
    reqs = [Request(uid=f"p{i}", prompt=[2 + i, 3, 4, 5], max_new_tokens=12) for i in range(3)]
    out, sched, backend = run_ahead(reqs, pages=9, page=4)
    for r in reqs:
        assert out[r.uid] == expected(r.prompt, 12)
    assert sched.stats["preemptions"] > 0
    sched.cache.audit()


def test_run_ahead_counts_pages_for_the_whole_step():
    """Two requests of equal length cross a page edge in the same step with one page free:
    the step is not launched ahead (each alone would fit, both do not); the planned path
    preempts and the tokens are those of a run without run-ahead."""
    def reqs():
        return [Request(uid=f"p{i}", prompt=[2 + i, 3, 4, 5], max_new_tokens=12) for i in range(2)]
    want, plain_sched, _ = run(reqs(), pages=5, page=4)
    out, sched, backend = run_ahead(reqs(), pages=5, page=4)
    assert out == want
    for r in reqs():
        assert out[r.uid] == expected(r.prompt, 12)
    assert sched.stats["preemptions"] > 0 and sched.stats["preemptions"] == plain_sched.stats["preemptions"]
    sched.cache.audit()
    assert sched.cache.free_pages() == sched.cache.total_pages()


# -- the debugging aids: lifecycle table, trajectory record ------------------------------------

def test_every_event_is_a_legal_transition_and_an_illegal_one_raises():
    from lockstep_b200.engine.lifecycle import TRANSITIONS, IllegalTransition, Lifecycle

    taken = set()
    # plenty of room; so few pages that requests are preempted; prefix reuse with evictions; portions
    reqs = [Request(uid=f"p{i}", prompt=[2 + i, 3, 4, 5] * (1 + i), max_new_tokens=12) for i in range(4)]
    for kw in ({}, {"pages": 9, "page": 4}, {"pages": 14, "page": 4, "enable_prefix_cache": True},
               {"policy": FixedChunkPolicy(3)}):
        fresh = [Request(uid=r.uid, prompt=list(r.prompt), max_new_tokens=r.max_new_tokens) for r in reqs]
        out, sched, _ = run(fresh, **kw)
        assert all(out[r.uid] == expected(r.prompt, 12) for r in reqs)
        taken |= sched.lifecycle.taken
        assert not sched.lifecycle.state              # every request reached its end
    shared = [Request(uid=f"s{i}", prompt=list(range(8)) + [20 + i], max_new_tokens=3) for i in range(3)]
    out, sched, _ = run(shared, pages=5, page=4, enable_prefix_cache=True, max_running=1)
    taken |= sched.lifecycle.taken
    assert ("admitted", "cache_hit") in taken and ("decoding", "preempt") in taken
    assert any(event == "evict" for _, event in taken)
    assert taken <= set(TRANSITIONS)
    life = Lifecycle()
    life.observe("x", "admit")
    with pytest.raises(IllegalTransition, match="cannot follow"):
        life.observe("x", "finish")                   # nothing was decoded yet
    with pytest.raises(IllegalTransition):
        Lifecycle().observe("y", "decode")            # never admitted


def test_trajectory_names_the_first_step_that_differs():
    def go(prompt_of_b, **kw):
        reqs = [Request(uid="a", prompt=[5, 6, 7, 8, 9], max_new_tokens=9),
                Request(uid="b", prompt=prompt_of_b, max_new_tokens=6)]
        out, sched, _ = run(reqs, trajectory=True, policy=FixedChunkPolicy(2), **kw)
        return sched.trajectory

    one, two = go([1, 2, 3, 4, 5, 6, 7]), go([1, 2, 3, 4, 5, 6, 7])
    assert one.steps > 5 and one.hexdigest() == two.hexdigest() and one.first_divergence(two) is None
    other = go([1, 2, 3, 4, 5, 6, 99])                # b's prompt differs in its fourth portion
    assert other.hexdigest() != one.hexdigest() and one.first_divergence(other) == 3
    pages = go([1, 2, 3, 4, 5, 6, 7], pages=32)      # the same tokens from another pool: the cache digest differs
    assert one.first_divergence(pages) == 0
