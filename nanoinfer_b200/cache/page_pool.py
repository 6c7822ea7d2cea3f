"""Free-list of cache pages (the compiled PagePool of csrc/host_runtime.cpp behind a thin class).

Same contract as the reference's BlockManager without its prefix-cache bookkeeping
(src/engine/block_manager.cpp:17-182): pages are handed out from a LIFO stack whose first
pops are 0, 1, 2, ...; a page given back is the next one handed out, so a finished
request's pages are used again at once; freeing a page twice, or one that was never taken,
is an error and changes nothing.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, List

from . import native


class OutOfPages(RuntimeError):
    """The pool has fewer free pages than were asked for; nothing was taken."""


class PagePoolError(RuntimeError):
    """A page id is out of range, freed twice or was never handed out."""


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self._lib = native.lib()
        self.num_pages = num_pages
        self._h = self._lib.ni_pool_create(num_pages)

    def __del__(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ni_pool_destroy(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return self._lib.ni_pool_num_free(self._h)

    @property
    def num_taken(self) -> int:
        return self.num_pages - self.num_free

    def is_taken(self, page: int) -> bool:
        return bool(self._lib.ni_pool_is_taken(self._h, int(page)))

    def _message(self) -> str:
        return self._lib.ni_pool_last_error(self._h).decode()

    def take(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot take a negative number of pages")
        out = (ctypes.c_int32 * max(n, 1))()
        rc = self._lib.ni_pool_take(self._h, n, out)
        if rc == native.ERR_OUT_OF_PAGES:
            raise OutOfPages(self._message())
        if rc != 0:
            raise PagePoolError(self._message())
        return list(out[:n])

    def give_back(self, pages: Iterable[int]) -> None:
        pages = [int(p) for p in pages]
        arr = (ctypes.c_int32 * max(len(pages), 1))(*pages)
        if self._lib.ni_pool_give_back(self._h, arr, len(pages)) != 0:
            raise PagePoolError(self._message())
