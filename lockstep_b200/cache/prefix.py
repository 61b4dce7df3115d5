"""Exact-prefix reuse of whole pages (LockStep: engine/cache/prefix.py).

A chain of sha256 keys over whole pages of tokens maps a prompt's prefix to the
physical pages that hold its keys and values.  A finished request's whole pages
are indexed (the index takes a reference on each); a new request with the same
prefix adopts them and computes only the rest.  Only pages whose sole holder is
the index can be evicted, and a chain is evicted from its end: a page whose key
has a child entry is not offered, so no entry is ever left that ``lookup`` cannot
reach.  (A request that holds a page of a chain holds every page before it, so
a page held by the index alone has only such pages behind it, and each becomes
a leaf in turn.)  It serves models whose cache is one paged group that
keeps all keys: a window or a fixed-size state cannot be shared by page.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

_ROOT = b"lockstep-b200-prefix-root"


def page_key(parent: bytes, tokens: tuple[int, ...]) -> bytes:
    h = hashlib.sha256()
    h.update(parent)
    h.update(b"|")
    h.update(",".join(str(t) for t in tokens).encode("ascii"))
    return h.digest()


@dataclass
class _Entry:
    page: int
    tokens: tuple[int, ...]
    parent: bytes = _ROOT
    children: int = 0
    hits: int = 0


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

    def lookup(self, tokens) -> tuple[int, list[int]]:
        """Longest indexed page-aligned prefix as (token count, pages)."""
        self.stats["lookups"] += 1
        pages: list[int] = []
        for key, chunk in self._chain(tokens):
            e = self.entries.get(key)
            if e is None or e.tokens != chunk:
                break
            e.hits += 1
            pages.append(e.page)
        self.stats["hit_pages"] += len(pages)
        return len(pages) * self.page_size, pages

    def insert(self, tokens, pages: list[int], group) -> int:
        made = 0
        parent = _ROOT
        for i, (key, chunk) in enumerate(self._chain(tokens)):
            if i >= len(pages) or pages[i] < 0:
                break
            if key not in self.entries:
                self.entries[key] = _Entry(page=pages[i], tokens=chunk, parent=parent)
                if parent in self.entries:
                    self.entries[parent].children += 1
                group.pin(pages[i])
                made += 1
            parent = key
        self.stats["inserts"] += made
        return made

    def evictable(self, group) -> list[int]:
        """Pages that can be evicted now: held by the index alone, at the end of their chain."""
        return sorted(e.page for e in self.entries.values()
                      if e.children == 0 and group.allocator.refcount[e.page] == 1)

    def reclaimable(self, group) -> int:
        """How many pages evictions can free in the end: every page the index alone holds
        (each is, or becomes, the end of its chain)."""
        return sum(1 for e in self.entries.values() if group.allocator.refcount[e.page] == 1)

    def evict(self, page: int, group) -> bool:
        for key, e in list(self.entries.items()):
            if e.page == page:
                if e.children:
                    raise ValueError(f"page {page} has {e.children} indexed pages after it; evict those first")
                del self.entries[key]
                if e.parent in self.entries:
                    self.entries[e.parent].children -= 1
                group.unpin(page)
                self.stats["evictions"] += 1
                return True
        return False

    def audit(self) -> None:
        """Every entry's parent is indexed (or is the root) and child counts are right."""
        counts: dict[bytes, int] = {}
        for key, e in self.entries.items():
            if e.parent != _ROOT and e.parent not in self.entries:
                raise AssertionError(f"page {e.page} is indexed but the page before it is not: unreachable")
            counts[e.parent] = counts.get(e.parent, 0) + 1
        for key, e in self.entries.items():
            if e.children != counts.get(key, 0):
                raise AssertionError(f"page {e.page}: {e.children} children on the books, {counts.get(key, 0)} indexed")

    def digest(self) -> tuple:
        return tuple(sorted((k.hex()[:16], e.page) for k, e in self.entries.items()))
