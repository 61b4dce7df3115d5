"""Exact-prefix reuse of whole pages (LockStep: engine/cache/prefix.py).

A chain of sha256 keys over whole pages of tokens maps a prompt's prefix to the
physical pages that hold its keys and values.  A finished request's whole pages
are indexed (the index takes a reference on each); a new request with the same
prefix adopts them and computes only the rest.

A cache may have several paged groups (layers that keep every key, layers that
keep a window of them, layers with other head counts).  An entry stands for one
page of tokens and names the page that holds them in each group, or -1 where the
request had already given that page back (it lay behind a window).  A prefix of
n pages can be adopted if every group still has the pages that the first new
token can read: all n where every key is kept, those that reach into the window
of position n x page_size elsewhere.  ``lookup`` returns the longest such prefix,
with -1 in a group's list for the pages that group does not need.  So a model with
windowed layers reuses a prefix where its window's pages were kept (the end of a
finished request's context: the next turn of the same conversation), and one
without windows reuses any shared prefix.  A fixed-size state cannot be shared by
page: models with state slots get no prefix reuse (the scheduler refuses the option).

Only entries whose pages the index alone holds can be evicted, and a chain is evicted
from its end: an entry with an indexed entry after it is not offered, so that no
page stays pinned for a prefix that ``lookup`` can no longer use.  An entry is named
by its ``handle``: the number of its page in the first group that has one (plus
``HANDLE_STRIDE`` x that group's index), which for a cache of one group is the page
number itself.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

_ROOT = b"lockstep-b200-prefix-root"
HANDLE_STRIDE = 1 << 32


def page_key(parent: bytes, tokens: tuple[int, ...]) -> bytes:
    h = hashlib.sha256()
    h.update(parent)
    h.update(b"|")
    h.update(",".join(str(t) for t in tokens).encode("ascii"))
    return h.digest()


@dataclass
class _Entry:
    pages: list[int]                 # one per paged group, -1 where the group holds none
    tokens: tuple[int, ...]
    parent: bytes = _ROOT
    children: int = 0
    hits: int = 0

    @property
    def handle(self) -> int:
        for g, page in enumerate(self.pages):
            if page >= 0:
                return g * HANDLE_STRIDE + page
        raise AssertionError("an indexed entry holds no page")

    @property
    def page(self) -> int:
        """The entry's page in the first group (the only one of a cache with one group)."""
        return self.pages[0]


def _as_groups(groups):
    return list(groups) if isinstance(groups, (list, tuple)) else [groups]


@dataclass
class PrefixIndex:
    page_size: int
    entries: dict[bytes, _Entry] = field(default_factory=dict)
    stats: dict = field(default_factory=lambda: {"lookups": 0, "hit_pages": 0, "inserts": 0, "evictions": 0})

    def _chain(self, tokens):
        parent = _ROOT
        for i in range(len(tokens) // self.page_size):
            chunk = tuple(tokens[i * self.page_size:(i + 1) * self.page_size])
            parent = page_key(parent, chunk)
            yield parent, chunk

    def lookup(self, tokens, groups, limit: int | None = None) -> tuple[int, list[list[int]]]:
        """The longest indexed page-aligned prefix of ``tokens`` (of at most ``limit`` tokens)
        that every group of ``groups`` can still serve, as (token count, for each group its
        pages: -1 for a page that no later token reads in that group)."""
        groups = _as_groups(groups)
        self.stats["lookups"] += 1
        found: list[_Entry | None] = []
        for key, chunk in self._chain(tokens):
            e = self.entries.get(key)
            found.append(e if e is not None and e.tokens == chunk else None)
        n = len(found)
        if limit is not None:
            n = min(n, limit // self.page_size)
        while n > 0:
            first = [g.first_needed_page(n * self.page_size) for g in groups]
            if all(found[i] is not None and found[i].pages[gi] >= 0
                   for gi in range(len(groups)) for i in range(first[gi], n)):
                break
            n -= 1
        if n == 0:
            return 0, [[] for _ in groups]
        for e in found[:n]:
            if e is not None:
                e.hits += 1
        self.stats["hit_pages"] += n
        first = [g.first_needed_page(n * self.page_size) for g in groups]
        return n * self.page_size, [[found[i].pages[gi] if i >= first[gi] else -1 for i in range(n)]
                                    for gi in range(len(groups))]

    def insert(self, tokens, groups, uid: str) -> int:
        """Index the whole pages of ``tokens`` that request ``uid`` holds; returns how many
        entries were made or gained a page."""
        groups = _as_groups(groups)
        held = [g.seqs[uid].pages for g in groups]
        made = 0
        parent = _ROOT
        for i, (key, chunk) in enumerate(self._chain(tokens)):
            pages = [p[i] if i < len(p) else -1 for p in held]
            e = self.entries.get(key)
            if e is None:
                if any(p >= 0 for p in pages):
                    self.entries[key] = _Entry(pages=pages, tokens=chunk, parent=parent)
                    if parent in self.entries:
                        self.entries[parent].children += 1
                    for g, p in zip(groups, pages):
                        if p >= 0:
                            g.pin(p)
                    made += 1
            elif e.tokens == chunk:
                gained = False
                for gi, p in enumerate(pages):        # a page this entry lacked (it lay behind a window then)
                    if e.pages[gi] < 0 <= p:
                        e.pages[gi] = p
                        groups[gi].pin(p)
                        gained = True
                made += gained
            parent = key
        self.stats["inserts"] += made
        return made

    @staticmethod
    def _index_alone(e: _Entry, groups) -> bool:
        return all(p < 0 or g.allocator.refcount[p] == 1 for g, p in zip(groups, e.pages))

    def evictable(self, groups) -> list[int]:
        """Handles of the entries that can be evicted now: their pages are held by the index
        alone, and no indexed entry comes after them."""
        groups = _as_groups(groups)
        return sorted(e.handle for e in self.entries.values()
                      if e.children == 0 and self._index_alone(e, groups))

    def reclaimable(self, groups) -> list[int]:
        """For each group, how many pages evictions can free in the end: those of every entry
        whose pages the index alone holds (each is, or becomes, the end of its chain)."""
        groups = _as_groups(groups)
        out = [0] * len(groups)
        for e in self.entries.values():
            if self._index_alone(e, groups):
                for gi, p in enumerate(e.pages):
                    out[gi] += p >= 0
        return out

    def evict(self, handle: int, groups) -> bool:
        groups = _as_groups(groups)
        for key, e in list(self.entries.items()):
            if e.handle == handle:
                if e.children:
                    raise ValueError(f"entry {handle} has {e.children} indexed pages after it; evict those first")
                del self.entries[key]
                if e.parent in self.entries:
                    self.entries[e.parent].children -= 1
                for g, p in zip(groups, e.pages):
                    if p >= 0:
                        g.unpin(p)
                self.stats["evictions"] += 1
                return True
        return False

    def audit(self) -> None:
        """Child counts are right, every entry holds a page, and no page is indexed twice."""
        counts: dict[bytes, int] = {}
        seen: set[tuple[int, int]] = set()
        for key, e in self.entries.items():
            if e.parent in self.entries:
                counts[e.parent] = counts.get(e.parent, 0) + 1
            if not any(p >= 0 for p in e.pages):
                raise AssertionError("an entry that holds no page is indexed")
            for gi, p in enumerate(e.pages):
                if p >= 0:
                    if (gi, p) in seen:
                        raise AssertionError(f"page {p} of group {gi} is indexed twice")
                    seen.add((gi, p))
        for key, e in self.entries.items():
            if e.children != counts.get(key, 0):
                raise AssertionError(f"entry {e.handle}: {e.children} children on the books, "
                                     f"{counts.get(key, 0)} indexed")

    def digest(self) -> tuple:
        return tuple(sorted((k.hex()[:16], tuple(e.pages)) for k, e in self.entries.items()))
