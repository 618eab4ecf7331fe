"""Free list of cache pages for one page group."""

from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """The pool has fewer free pages than a step needs."""


class PagePool:
    """Hands out page ids 0..num_pages-1. Last freed, first reused, so that pages are used again
    soon (a stale read then shows up in tests instead of hiding in never-touched memory)."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))
        self._held = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.pop()
        self._held[p] = True
        return p

    def free(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise ValueError(f"page {page} is not of this pool")
        if not self._held[page]:
            raise ValueError(f"page {page} freed twice (or never handed out)")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]
