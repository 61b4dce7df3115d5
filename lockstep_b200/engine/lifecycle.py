"""The life of a request as a state machine (after LockStep's engine/sched/lifecycle.py:11-40).

The scheduler records an event for everything that happens to a request; this
table says which event may follow in which state, and ``Lifecycle.observe``
raises on one that may not.  It differs from LockStep's table where this
scheduler differs: pages are taken step by step, so a request may see an
eviction (made on its behalf) in any running state, and the youngest running
request may be preempted before it has run a token.
"""

from __future__ import annotations

WAITING, ADMITTED, PREFILLING, DECODING, PREEMPTED, DONE = (
    "waiting", "admitted", "prefilling", "decoding", "preempted", "done")

# events: admit, resume, cache_hit (pages of an indexed prefix adopted), chunk (a portion that
# does not reach the end of the context), decode (a portion that does: a token is sampled),
# evict (a cached page evicted to make room for this request), preempt, finish
TRANSITIONS: dict[tuple[str, str], str] = {
    (WAITING, "admit"): ADMITTED,
    (PREEMPTED, "resume"): ADMITTED,
    (ADMITTED, "cache_hit"): PREFILLING,
    (ADMITTED, "chunk"): PREFILLING,
    (ADMITTED, "decode"): DECODING,
    (ADMITTED, "evict"): ADMITTED,
    (ADMITTED, "preempt"): PREEMPTED,
    (PREFILLING, "chunk"): PREFILLING,
    (PREFILLING, "decode"): DECODING,
    (PREFILLING, "evict"): PREFILLING,
    (PREFILLING, "preempt"): PREEMPTED,
    (DECODING, "decode"): DECODING,
    (DECODING, "evict"): DECODING,
    (DECODING, "preempt"): PREEMPTED,
    (DECODING, "finish"): DONE,
}


class IllegalTransition(AssertionError):
    """An event that cannot follow in the request's state: the scheduler's books are wrong."""


class Lifecycle:
    def __init__(self):
        self.state: dict[str, str] = {}
        self.taken: set[tuple[str, str]] = set()      # (state, event) pairs seen: coverage of the table

    def observe(self, uid: str, event: str) -> str:
        state = self.state.get(uid, WAITING)
        nxt = TRANSITIONS.get((state, event))
        if nxt is None:
            legal = sorted(e for (s, e) in TRANSITIONS if s == state)
            raise IllegalTransition(f"request {uid!r} is {state}: event {event!r} cannot follow "
                                    f"(legal here: {legal})")
        self.taken.add((state, event))
        if nxt == DONE:
            self.state.pop(uid, None)         # a later request may use the uid again
        else:
            self.state[uid] = nxt
        return nxt
