"""The cache manager: everything a request keeps between steps.

Layers are sorted into groups by what their mixer declares (``CacheNeed``):
- a paged group keeps keys and values in pages of ``page_size`` tokens, with a
  block table per request; layers that read all keys and layers that read a
  window of them are different groups with pages of their own; a windowed
  group gives a page back as soon as every position in it lies behind the
  window;
- a state group keeps one tensor of fixed size per request in a slot.
A live request owns one slot id; it is its row in every group's block table
and its index in every state tensor.  Pages are handed out lowest-first,
given back when a request ends or is preempted, and used again.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import CacheNeed
from .pages import AuditFailure, OutOfPages, PageAllocator


@dataclass
class LayerCache:
    """What a mixer sees of the cache in one run of a layer."""

    kind: str
    writes: bool
    pages: torch.Tensor | None = None         # [num_pages, 2, kv_heads, page_size, head_dim]
    block_table: torch.Tensor | None = None   # [max_live, max_pages_per_seq] int32 (device)
    state: torch.Tensor | None = None         # [max_live, *state_shape]
    group: object | None = None


@dataclass
class _Seq:
    slot: int
    pages: list[int] = field(default_factory=list)   # logical -> physical, -1 once given back
    shared: int = 0                                  # leading pages adopted from the prefix index


# What a freed page is filled with when ``poison_freed_pages`` is on: finite and far outside
# anything a model computes.  A key or value of a page that was given back, read with any
# weight but zero, then shows in the result at once.  (Not NaN, as in LockStep's
# engine/kv/paged.py:103-113: these kernels load whole tiles and give the keys past a
# request's length the weight zero, and 0 x NaN would flag a read that is harmless.)
POISON = 1.0e30


class PagedGroup:
    def __init__(self, need: CacheNeed, entries: list[int], num_pages: int, page_size: int,
                 max_live: int, max_pages_per_seq: int, dtype, device, allocate: bool = True,
                 poison_freed_pages: bool = False):
        self.need, self.entries = need, list(entries)
        self.page_size, self.window = int(page_size), int(need.window)
        self.allocator = PageAllocator(num_pages)
        self.max_pages_per_seq = int(max_pages_per_seq)
        # One row and one page more than requests can hold: the padding row (index max_live) maps
        # every position to the padding page (index num_pages, outside the allocator's range).
        # Rows that pad a recorded decode step to its batch size write their keys there.
        self.table_host = np.full((max_live + 1, self.max_pages_per_seq), -1, dtype=np.int32)
        self.table_host[max_live, :] = num_pages
        self.device = device
        self.table = None
        self.pages = None
        if allocate:
            self.table = torch.from_numpy(self.table_host).to(device)
            self.pages = torch.zeros(
                (len(self.entries), num_pages + 1, 2, need.kv_heads, self.page_size, need.head_dim),
                dtype=dtype, device=device)
        self.seqs: dict[str, _Seq] = {}
        self._dirty: set[int] = set()
        self.pinned: dict[int, int] = {}
        self.poison = bool(poison_freed_pages)
        self.poisoned = 0
        # True (prefix reuse is on): a windowed group keeps what the last whole-page boundary's
        # window reads, not only what the next position's does, so that a finished request's
        # whole pages can be adopted by a request that goes on from that boundary
        self.keep_boundary_window = False

    def _give_back(self, page: int) -> None:
        """Drop one reference on ``page``; a page nobody holds any more is poisoned (debug option)."""
        if self.allocator.release(page) and self.poison:
            self.poisoned += 1
            if self.pages is not None:
                self.pages[:, page].fill_(POISON)

    def assert_exclusive(self, uid: str, first_token: int, last_token: int) -> None:
        """The pages ``uid`` is about to write (tokens first..last) are held by it alone: sharing
        is by whole pages of a prefix, so a write never lands in a shared page
        (LockStep: engine/kv/paged.py:162-181)."""
        seq = self.seqs[uid]
        for logical in range(first_token // self.page_size, last_token // self.page_size + 1):
            page = seq.pages[logical] if logical < len(seq.pages) else -1
            if page < 0:
                raise AuditFailure(f"{uid} is about to write token {first_token}.. into logical page {logical}, "
                                   "which it does not hold")
            if self.allocator.refcount[page] != 1:
                raise AuditFailure(
                    f"{uid} is about to write physical page {page}, which has {self.allocator.refcount[page]} "
                    f"holders ({self.pinned.get(page, 0)} of them the prefix index)")

    # -- accounting ---------------------------------------------------------
    def first_needed_page(self, kv_len_after: int, first_query_pos: int | None = None) -> int:
        """First logical page a query at ``first_query_pos`` (default: the next
        position) can still read."""
        if not self.window:
            return 0
        q = kv_len_after if first_query_pos is None else first_query_pos
        lo = q - self.window + 1
        return max(0, lo) // self.page_size

    def pages_short(self, uid: str, total_tokens: int) -> int:
        """How many new pages ``reserve(uid, total_tokens)`` would take."""
        seq = self.seqs[uid]
        need = -(-total_tokens // self.page_size)
        return max(0, need - len(seq.pages))

    def reserve(self, uid: str, total_tokens: int) -> None:
        seq = self.seqs[uid]
        need = -(-total_tokens // self.page_size)
        if need > self.max_pages_per_seq:
            raise ValueError(
                f"{uid}: {total_tokens} tokens need {need} pages, the block table holds "
                f"{self.max_pages_per_seq} (raise max_seq_len)")
        while len(seq.pages) < need:
            page = self.allocator.take()
            self.table_host[seq.slot, len(seq.pages)] = page
            seq.pages.append(page)
            self._dirty.add(seq.slot)

    def advance(self, uid: str, kv_len: int) -> int:
        """Give back the pages that every later query's window has passed."""
        if not self.window:
            return 0
        seq = self.seqs[uid]
        first = self.first_needed_page(kv_len // self.page_size * self.page_size if self.keep_boundary_window
                                       else kv_len)
        freed = 0
        for logical in range(min(first, len(seq.pages))):
            page = seq.pages[logical]
            if page >= 0:
                self._give_back(page)
                seq.pages[logical] = -1
                self.table_host[seq.slot, logical] = -1
                self._dirty.add(seq.slot)
                freed += 1
        return freed

    def create(self, uid: str, slot: int) -> None:
        self.seqs[uid] = _Seq(slot=slot)
        self.table_host[slot, :] = -1
        self._dirty.add(slot)

    def adopt(self, uid: str, pages: list[int]) -> None:
        seq = self.seqs[uid]
        if seq.pages:
            raise AuditFailure("adopt expects a request that holds no pages yet")
        for page in pages:                    # -1: a page behind the window, which nobody reads any more
            if page >= 0:
                self.allocator.retain(page)
            self.table_host[seq.slot, len(seq.pages)] = page
            seq.pages.append(page)
        seq.shared = len(pages)
        self._dirty.add(seq.slot)

    def release(self, uid: str) -> None:
        seq = self.seqs.pop(uid)
        for page in seq.pages:
            if page >= 0:
                self._give_back(page)
        self.table_host[seq.slot, :] = -1
        self._dirty.add(seq.slot)

    def pin(self, page: int) -> None:
        self.allocator.retain(page)
        self.pinned[page] = self.pinned.get(page, 0) + 1

    def unpin(self, page: int) -> None:
        held = self.pinned.get(page, 0)
        if held <= 0:
            raise AuditFailure(f"unpinning page {page}, which the prefix index does not hold")
        if held == 1:
            del self.pinned[page]
        else:
            self.pinned[page] = held - 1
        self._give_back(page)

    def sync(self) -> None:
        """Bring the device block table up to date (rows that changed)."""
        if self.table is None or not self._dirty:
            self._dirty.clear()
            return
        rows = sorted(self._dirty)
        if len(rows) > 8:
            self.table.copy_(torch.from_numpy(self.table_host))
        else:
            for r in rows:
                self.table[r].copy_(torch.from_numpy(self.table_host[r]))
        self._dirty.clear()

    def audit(self) -> None:
        holders: dict[int, int] = dict(self.pinned)
        for uid, seq in self.seqs.items():
            seen = set()
            for logical, page in enumerate(seq.pages):
                if page < 0:
                    continue
                if page in seen:
                    raise AuditFailure(f"{uid} maps two logical pages to physical page {page}")
                seen.add(page)
                holders[page] = holders.get(page, 0) + 1
                if self.table_host[seq.slot, logical] != page:
                    raise AuditFailure(f"{uid}: block table row disagrees at logical page {logical}")
        self.allocator.audit(holders)


class StateGroup:
    def __init__(self, need: CacheNeed, entries: list[int], max_live: int, device, allocate: bool = True):
        self.need, self.entries = need, list(entries)
        self.state = None
        if allocate:
            # (one slot more than requests can hold: the padding rows of a recorded step)
            self.state = torch.zeros((len(self.entries), max_live + 1, *need.state_shape),
                                     dtype=need.state_dtype, device=device)

    def clear(self, slot: int) -> None:
        if self.state is not None:
            self.state[:, slot].zero_()


class CacheManager:
    """Pages, block tables and state slots of all live requests.

    ``needs``: for every cache entry of the model's schedule (index = entry),
    the ``CacheNeed`` of the mixer that writes it (None for a mixer that keeps
    nothing).  ``allocate=False`` builds the books without device memory (for
    host-side tests and planning).  ``poison_freed_pages`` (a debugging aid) fills a page
    with ``POISON`` when its last holder gives it back.
    """

    def __init__(self, needs: list[CacheNeed | None], num_pages: int, page_size: int, max_live: int,
                 max_seq_len: int, dtype=torch.float32, device="cpu", allocate: bool = True,
                 poison_freed_pages: bool = False):
        self.page_size, self.max_live = int(page_size), int(max_live)
        self.max_seq_len = int(max_seq_len)
        self.device = torch.device(device)
        self.paged: list[PagedGroup] = []
        self.states: list[StateGroup] = []
        self._entry: dict[int, tuple[object, int]] = {}
        by_key: dict[tuple, list[int]] = {}
        need_of: dict[tuple, CacheNeed] = {}
        for entry, need in enumerate(needs):
            if need is None:
                continue
            by_key.setdefault(need.group_key(), []).append(entry)
            need_of[need.group_key()] = need
        max_pages_per_seq = -(-self.max_seq_len // self.page_size)
        for key, entries in by_key.items():
            need = need_of[key]
            if need.kind == "paged_kv":
                group = PagedGroup(need, entries, num_pages, page_size, max_live, max_pages_per_seq,
                                   dtype, self.device, allocate, poison_freed_pages)
                self.paged.append(group)
            elif need.kind == "state":
                group = StateGroup(need, entries, max_live, self.device, allocate)
                self.states.append(group)
            else:
                raise ValueError(f"unknown cache need {need.kind!r}")
            for i, entry in enumerate(entries):
                self._entry[entry] = (group, i)
        self.pad_slot = self.max_live          # the row of padding rows in every block table and state tensor
        self._free_slots = list(range(self.max_live - 1, -1, -1))
        self.slots: dict[str, int] = {}
        self.lengths: dict[str, int] = {}

    # -- requests -----------------------------------------------------------
    @property
    def live(self) -> int:
        return len(self.slots)

    def has_slot(self) -> bool:
        return bool(self._free_slots)

    def create(self, uid: str) -> int:
        if uid in self.slots:
            raise KeyError(f"request {uid!r} already holds a slot")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_live} request slots are taken")
        slot = self._free_slots.pop()
        self.slots[uid] = slot
        self.lengths[uid] = 0
        for g in self.paged:
            g.create(uid, slot)
        for g in self.states:
            g.clear(slot)
        return slot

    def peak_pages(self, total_tokens: int, max_portion: int) -> int:
        """The most pages a request of ``total_tokens`` holds in any group at any
        time when no step runs more than ``max_portion`` of its tokens: all of
        them where every key is kept; the window, the portion and one page of
        slack where pages behind the window are given back."""
        worst = 0
        for g in self.paged:
            need = -(-total_tokens // self.page_size)
            if g.window and total_tokens > max_portion:
                need = min(need, -(-(g.window - 1 + max_portion) // self.page_size) + 1 + g.keep_boundary_window)
            worst = max(worst, need)
        return worst

    def keep_boundary_windows(self, on: bool = True) -> None:
        """Windowed groups keep the pages that the window of the last whole-page boundary reads
        (at most one page more per request): what a request that adopts the whole pages needs."""
        for g in self.paged:
            g.keep_boundary_window = bool(on)

    def pages_short(self, uid: str, total_tokens: int) -> int:
        """The most new pages any group needs to hold ``total_tokens`` of ``uid``."""
        return max((g.pages_short(uid, total_tokens) for g in self.paged), default=0)

    def can_reserve(self, uid: str, total_tokens: int) -> bool:
        return all(g.pages_short(uid, total_tokens) <= g.allocator.free_pages for g in self.paged)

    def can_reserve_all(self, wants) -> bool:
        """True if every (uid, total_tokens) of ``wants`` can be reserved, one after the
        other, from the pages that are free now."""
        return all(sum(g.pages_short(uid, total) for uid, total in wants) <= g.allocator.free_pages
                   for g in self.paged)

    def reserve(self, uid: str, total_tokens: int) -> None:
        """Make room for ``total_tokens`` of ``uid`` in every paged group, or take nothing."""
        if total_tokens > self.max_seq_len:
            raise ValueError(f"{uid}: {total_tokens} tokens exceed max_seq_len {self.max_seq_len}")
        if not self.can_reserve(uid, total_tokens):
            short = {i: g.pages_short(uid, total_tokens) - g.allocator.free_pages
                     for i, g in enumerate(self.paged)}
            raise OutOfPages(f"{uid}: not enough free pages for {total_tokens} tokens (short by group: {short})")
        for g in self.paged:
            g.reserve(uid, total_tokens)

    def assert_exclusive(self, uid: str, first_token: int, last_token: int) -> None:
        """Every page that tokens first..last of ``uid`` are written to is held by ``uid`` alone."""
        for g in self.paged:
            g.assert_exclusive(uid, first_token, last_token)

    def advance(self, uid: str, kv_len: int) -> int:
        """Record that ``uid`` now holds ``kv_len`` tokens; windowed groups give
        back the pages behind the window.  Returns the number of pages freed."""
        self.lengths[uid] = kv_len
        return sum(g.advance(uid, kv_len) for g in self.paged)

    def release(self, uid: str) -> None:
        slot = self.slots.pop(uid)
        self.lengths.pop(uid, None)
        for g in self.paged:
            g.release(uid)
        self._free_slots.append(slot)
        self._free_slots.sort(reverse=True)

    # -- numbers ------------------------------------------------------------
    def free_pages(self) -> int:
        return min((g.allocator.free_pages for g in self.paged), default=0)

    def total_pages(self) -> int:
        return min((g.allocator.num_pages for g in self.paged), default=0)

    def reused_pages(self) -> int:
        return sum(g.allocator.stats["reused"] for g in self.paged)

    # -- device -------------------------------------------------------------
    def sync(self) -> None:
        for g in self.paged:
            g.sync()

    def view(self, entry: int, writes: bool = True) -> LayerCache:
        if entry not in self._entry:
            return LayerCache(kind="none", writes=False)
        group, index = self._entry[entry]
        if isinstance(group, PagedGroup):
            return LayerCache(kind="paged_kv", writes=writes,
                              pages=None if group.pages is None else group.pages[index],
                              block_table=group.table, group=group)
        return LayerCache(kind="state", writes=writes,
                          state=None if group.state is None else group.state[index], group=group)

    def audit(self) -> None:
        taken = sorted(self.slots.values())
        if len(set(taken)) != len(taken):
            raise AuditFailure("two requests hold the same slot")
        if sorted(taken + self._free_slots) != list(range(self.max_live)):
            raise AuditFailure("a request slot was lost or is held twice")
        for g in self.paged:
            if set(g.seqs) != set(self.slots):
                raise AuditFailure("a paged group and the slot table disagree on the live requests")
            g.audit()

    def digest(self) -> tuple:
        return tuple(
            (g.allocator.digest(), tuple((u, tuple(s.pages)) for u, s in sorted(g.seqs.items())))
            for g in self.paged)
