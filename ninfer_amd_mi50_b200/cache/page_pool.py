"""A pool of cache pages: a free stack with ownership checks.

The reference has no pages: each sequence owns a slab of ``max_context`` positions
(src/runtime/kv_cache.cpp:14-22) and slots are handed out round-robin and never freed
(src/api/ninfer_c_api.cpp:150).  Here pages are taken and given back one by one; a page
just freed is the next one handed out, so reuse happens as early as it can.
"""

from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """The pool cannot satisfy a reservation; nothing was taken."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))  # pop() gives page 0 first
        self._held = [False] * self.num_pages
        self._used_before = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int) -> List[int]:
        """Take `n` pages, or none at all."""
        if n < 0:
            raise ValueError("cannot take a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} of {self.num_pages} are free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._held[p]:
                raise AssertionError(f"page {p} handed out while held")
            self._held[p] = True
        return out

    def take_marking_reuse(self, n: int):
        """`take`, and which of the pages taken have been held before (they hold an earlier
        owner's entries; a page never handed out still has the zeros it was created with)."""
        out = self.take(n)
        again = [p for p in out if self._used_before[p]]
        for p in out:
            self._used_before[p] = True
        return out, again

    def give_back(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise AssertionError(f"page {p} does not belong to this pool")
            if not self._held[p]:
                raise AssertionError(f"page {p} freed twice")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free or held, never both, never neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free stack twice")
        for p in range(self.num_pages):
            if self._held[p] == (p in free):
                raise AssertionError(f"page {p}: held={self._held[p]} and free={p in free}")
