"""Free-list of cache pages.

Same contract as the reference's BlockManager without its prefix-cache bookkeeping
(src/engine/block_manager.cpp:17-182): pages are handed out from a LIFO stack whose first
pops are 0, 1, 2, ...; a page given back is the next one handed out, so a finished
request's pages are used again at once; freeing a page twice, or one that was never taken,
is an error and changes nothing.
"""
from __future__ import annotations

from typing import Iterable, List


class OutOfPages(RuntimeError):
    """The pool has fewer free pages than were asked for; nothing was taken."""


class PagePoolError(RuntimeError):
    """A page id is out of range, freed twice or was never handed out."""


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._taken = bytearray(num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_taken(self) -> int:
        return self.num_pages - len(self._free)

    def is_taken(self, page: int) -> bool:
        return 0 <= page < self.num_pages and bool(self._taken[page])

    def take(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot take a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"asked for {n} pages, {len(self._free)} of {self.num_pages} are free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._taken[p] = 1
        return pages

    def give_back(self, pages: Iterable[int]) -> None:
        pages = list(pages)
        seen = set()
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise PagePoolError(f"page {p} is outside the pool of {self.num_pages}")
            if not self._taken[p] or p in seen:
                raise PagePoolError(f"page {p} is not held (freed twice?)")
            seen.add(p)
        for p in pages:
            self._taken[p] = 0
            self._free.append(p)
