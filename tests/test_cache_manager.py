"""The cache manager's books (no device): no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; slots; prefix reuse."""

from __future__ import annotations

import random

import pytest

from lockstep_b200.cache import AuditFailure, CacheManager, OutOfPages, PageAllocator, PrefixIndex
from lockstep_b200.parts import CacheNeed

FULL = CacheNeed("paged_kv", kv_heads=2, head_dim=16, window=0)
WIN = CacheNeed("paged_kv", kv_heads=2, head_dim=16, window=40)
STATE = CacheNeed("state", state_shape=(3, 4))


def manager(needs, pages=32, page=8, live=4, seq=512):
    return CacheManager(needs, num_pages=pages, page_size=page, max_live=live, max_seq_len=seq, allocate=False)


def test_allocator_lowest_first_and_reuse():
    a = PageAllocator(4)
    assert [a.take() for _ in range(3)] == [0, 1, 2]
    a.release(1)
    assert a.take() == 1 and a.stats["reused"] == 1
    a.take()
    with pytest.raises(OutOfPages):
        a.take()
    a.release(0)
    with pytest.raises(AuditFailure):
        a.release(0)          # freed twice


def test_audit_catches_lost_and_double_held_pages():
    m = manager([FULL, FULL])
    m.create("a")
    m.reserve("a", 20)
    m.audit()
    g = m.paged[0]
    g.allocator.refcount[g.seqs["a"].pages[0]] += 1        # a reference nobody holds
    with pytest.raises(AuditFailure):
        m.audit()
    g.allocator.refcount[g.seqs["a"].pages[0]] -= 1
    g.seqs["a"].pages[1] = g.seqs["a"].pages[0]             # one page under two logical places
    with pytest.raises(AuditFailure):
        m.audit()


def test_groups_by_need_have_pages_of_their_own():
    m = manager([FULL, WIN, WIN, FULL, STATE, None])
    assert len(m.paged) == 2 and len(m.states) == 1
    assert sorted(tuple(g.entries) for g in m.paged) == [(0, 3), (1, 2)]
    m.create("a")
    m.reserve("a", 100)
    full = next(g for g in m.paged if not g.window)
    win = next(g for g in m.paged if g.window)
    assert full.allocator.free_pages == 32 - 13 and win.allocator.free_pages == 32 - 13
    freed = m.advance("a", 100)
    # positions < 100 - 40 + 1 = 61 are behind every later query: pages 0..6 (7 * 8 = 56 <= 61)
    assert freed == 7 and win.allocator.free_pages == 32 - 6 and full.allocator.free_pages == 32 - 13
    assert win.seqs["a"].pages[:7] == [-1] * 7
    m.audit()
    m.reserve("a", 101)
    m.release("a")
    m.audit()
    assert m.free_pages() == 32 and m.live == 0


def test_reserve_takes_nothing_when_a_group_is_short():
    m = manager([FULL, WIN], pages=4, page=8)
    m.create("a")
    m.reserve("a", 30)
    m.create("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 9)
    m.audit()
    assert all(len(g.seqs["b"].pages) == 0 for g in m.paged)


def test_slots_are_unique_and_returned():
    m = manager([FULL], live=3)
    slots = [m.create(u) for u in "abc"]
    assert sorted(slots) == [0, 1, 2] and not m.has_slot()
    with pytest.raises(OutOfPages):
        m.create("d")
    m.release("b")
    assert m.create("d") == slots[1]
    m.audit()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = manager([FULL, WIN, FULL], pages=24, page=8, live=4, seq=400)
    live: dict[str, int] = {}
    n = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.has_slot():
            uid = f"r{n}"
            n += 1
            m.create(uid)
            live[uid] = 0
        elif op < 0.8 and live:
            uid = rng.choice(sorted(live))
            grow = live[uid] + rng.choice([1, 1, 1, 2, 7, 19, 40])
            if grow <= 400 and m.can_reserve(uid, grow):
                m.reserve(uid, grow)
                m.advance(uid, grow)
                live[uid] = grow
            elif grow <= 400:
                with pytest.raises(OutOfPages):
                    m.reserve(uid, grow)
        elif live:
            uid = rng.choice(sorted(live))
            m.release(uid)
            del live[uid]
        m.audit()
        for g in m.paged:
            held = sum(1 for s in g.seqs.values() for p in s.pages if p >= 0)
            assert held + g.allocator.free_pages == g.allocator.num_pages
    for uid in list(live):
        m.release(uid)
    m.audit()
    assert m.free_pages() == 24 and m.reused_pages() > 0


def test_prefix_index_shares_whole_pages():
    m = manager([FULL], pages=16, page=4)
    g = m.paged[0]
    idx = PrefixIndex(page_size=4)
    toks = list(range(11))
    m.create("a")
    m.reserve("a", 11)
    assert idx.insert(toks, g, "a") == 2                    # two whole pages
    m.release("a")
    m.audit()
    assert g.allocator.free_pages == 14 and idx.evictable(g) == [1] and idx.reclaimable(g) == [2]
    hit, pages = idx.lookup(toks[:9] + [99, 98], g)
    assert hit == 8 and pages == [[0, 1]]
    assert idx.lookup(toks[:8], g, limit=7)[0] == 4          # something is left to compute
    m.create("b")
    g.adopt("b", pages[0])
    m.reserve("b", 11)
    m.audit()
    assert idx.evictable(g) == []                          # a running request holds them
    m.release("b")
    with pytest.raises(ValueError):
        idx.evict(0, g)                                    # page 1 comes after it in the chain
    assert idx.evict(1, g) and idx.evictable(g) == [0] and idx.evict(0, g)
    m.audit()
    assert g.allocator.free_pages == 16
    assert idx.lookup(toks, g)[0] == 0


def test_prefix_eviction_leaves_no_unreachable_page():
    """Chains that share their first pages are evicted from their ends: whatever the order,
    every indexed page stays reachable by ``lookup`` and no page stays pinned for nothing."""
    rng = random.Random(4)
    m = manager([FULL], pages=32, page=4)
    g = m.paged[0]
    idx = PrefixIndex(page_size=4)
    stem = list(range(8))
    chains = [stem + [50 + i] * 4 + [60 + i] * 4 for i in range(3)]
    for i, toks in enumerate(chains):
        uid = f"r{i}"
        m.create(uid)
        hit, pages = idx.lookup(toks, g)
        g.adopt(uid, pages[0])
        m.lengths[uid] = hit
        m.reserve(uid, len(toks))
        idx.insert(toks, g, uid)
        m.release(uid)
    idx.audit()
    assert len(idx.entries) == 2 + 3 * 2 and idx.reclaimable(g) == [8]
    while idx.entries:
        offered = idx.evictable(g)
        assert offered, "pages are indexed but none is offered"
        idx.evict(rng.choice(offered), g)
        idx.audit()
        m.audit()
        for toks in chains:                 # what lookup finds is exactly what is still indexed
            hit, pages = idx.lookup(toks, g)
            assert len(pages[0]) == hit // 4
        reachable = set()
        for toks in chains:
            reachable.update(idx.lookup(toks, g)[1][0])
        assert reachable == {e.page for e in idx.entries.values()}
    assert g.allocator.free_pages == 32


def test_prefix_index_over_a_group_that_keeps_all_keys_and_one_with_a_window():
    win = CacheNeed("paged_kv", kv_heads=1, head_dim=16, window=8)
    m = manager([FULL, win], pages=16, page=4)
    full, windowed = m.paged
    idx = PrefixIndex(page_size=4)
    toks = list(range(100, 141))
    m.create("a")
    for n in range(4, 42, 4):                       # grows by a page a step; the window lets pages go
        m.reserve("a", min(n, 41))
        m.advance("a", min(n, 41))
    m.reserve("a", 41)
    m.advance("a", 41)
    assert windowed.seqs["a"].pages[:8] == [-1] * 8 and min(windowed.seqs["a"].pages[8:]) >= 0
    assert idx.insert(toks, m.paged, "a") == 10     # ten whole pages; the windowed group has two of them
    m.release("a")
    m.audit()
    idx.audit()
    assert idx.reclaimable(m.paged) == [10, 2]
    hit, pages = idx.lookup(toks + [7], m.paged)
    assert hit == 40 and min(pages[0]) >= 0
    assert pages[1][:8] == [-1] * 8 and min(pages[1][8:]) >= 0      # keys 33.. are what position 40 reads
    # one page less: position 36 reads keys 29.., that is page 7, which was given back
    assert idx.lookup(toks[:36] + [1, 2, 3, 4, 5], m.paged)[0] == 0
    assert idx.lookup(toks, m.paged, limit=39)[0] == 0
    # the all-keys group alone could use any of it
    assert idx.lookup(toks[:22], [full])[0] == 20
    m.create("b")
    for g, held in zip(m.paged, pages):
        g.adopt("b", held)
    m.lengths["b"] = hit
    m.reserve("b", 50)
    m.advance("b", 50)                              # gives back the adopted pages behind its window
    m.audit()
    assert idx.evictable(m.paged) == []             # "b" holds the chain's last page in the first group
    assert idx.insert(toks + list(range(9)), m.paged, "b") == 2     # pages 10 and 11 are new
    m.release("b")
    m.audit()
    idx.audit()
    order = []
    while idx.entries:
        offered = idx.evictable(m.paged)
        assert len(offered) == 1                    # one chain: only its end
        order.append(offered[0])
        idx.evict(offered[0], m.paged)
        m.audit()
    assert len(order) == 12
    assert full.allocator.free_pages == windowed.allocator.free_pages == 16


def test_freed_pages_are_poisoned_and_shared_pages_are_not_written():
    m = CacheManager([FULL], num_pages=8, page_size=4, max_live=4, max_seq_len=64, allocate=False,
                     poison_freed_pages=True)
    g = m.paged[0]
    idx = PrefixIndex(page_size=4)
    m.create("a")
    m.reserve("a", 10)
    m.assert_exclusive("a", 0, 9)
    idx.insert(list(range(10)), g, "a")
    with pytest.raises(AuditFailure, match="holders"):
        m.assert_exclusive("a", 4, 9)                  # its first two pages are now the index's too
    m.assert_exclusive("a", 8, 9)
    m.release("a")
    assert g.poisoned == 1                             # the third page; the index keeps the other two
    m.create("b")
    g.adopt("b", idx.lookup(list(range(8)), g)[1][0])
    m.lengths["b"] = 8
    m.reserve("b", 12)
    m.assert_exclusive("b", 8, 11)
    with pytest.raises(AuditFailure):
        m.assert_exclusive("b", 7, 8)                  # token 7 lies in a shared page
    with pytest.raises(AuditFailure, match="does not hold"):
        m.assert_exclusive("b", 8, 12)
    m.release("b")
    while idx.evictable(g):
        idx.evict(idx.evictable(g)[0], g)
    m.audit()
    assert g.poisoned == 4 and g.allocator.free_pages == 8


def test_constants_table_has_a_stable_digest():
    from lockstep_b200 import constants

    table = constants.table()
    assert table["attention.split_keys"] == 256 and table["gemm_tc.share_rule.blocks_per_round"] == 148
    assert constants.digest() == constants.digest() and len(constants.digest()) == 64
    assert "attention.split_keys=256" in constants.describe()
