"""Host-side page allocator: a min-heap free list (lowest page first, so that
allocation is a pure function of the order of requests) with reference counts
for pages shared between requests and the prefix index
(LockStep: engine/kv/paged.py:76-139)."""

from __future__ import annotations

import heapq


class OutOfPages(RuntimeError):
    """The pool has no free page left."""


class AuditFailure(AssertionError):
    """The allocator's books do not balance."""


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages))
        heapq.heapify(self._free)
        self.refcount = [0] * self.num_pages
        self.stats = {"taken": 0, "freed": 0, "reused": 0}
        self._ever_used = [False] * self.num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages(f"all {self.num_pages} pages are held")
        page = heapq.heappop(self._free)
        if self.refcount[page] != 0:
            raise AuditFailure(f"page {page} was on the free list with refcount {self.refcount[page]}")
        self.refcount[page] = 1
        self.stats["taken"] += 1
        if self._ever_used[page]:
            self.stats["reused"] += 1
        self._ever_used[page] = True
        return page

    def retain(self, page: int) -> None:
        if self.refcount[page] <= 0:
            raise AuditFailure(f"retaining free page {page}")
        self.refcount[page] += 1

    def release(self, page: int) -> bool:
        """Drop one reference; True if the page went back to the free list."""
        if not 0 <= page < self.num_pages or self.refcount[page] <= 0:
            raise AuditFailure(f"releasing page {page}, which is not held")
        self.refcount[page] -= 1
        if self.refcount[page] == 0:
            heapq.heappush(self._free, page)
            self.stats["freed"] += 1
            return True
        return False

    def audit(self, holders: dict[int, int]) -> None:
        """``holders``: page -> number of references that requests and the prefix
        index hold.  Raises if a page is lost, held twice or freed twice."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AuditFailure("a page is on the free list more than once")
        for page in range(self.num_pages):
            want = holders.get(page, 0)
            if self.refcount[page] != want:
                raise AuditFailure(
                    f"page {page}: refcount {self.refcount[page]} but {want} holders")
            if (self.refcount[page] == 0) != (page in free):
                raise AuditFailure(
                    f"page {page}: refcount {self.refcount[page]} but "
                    f"{'on' if page in free else 'not on'} the free list")

    def digest(self) -> tuple:
        return (tuple(self.refcount), tuple(sorted(self._free)))
