"""The cache manager: paged keys/values per group of layers, block tables per request,
and fixed-size state slots.

A *group* is a set of layer runs with the same need (KV head count, head size, window).
Each group has a page pool and, per request, a block table of its own; a page id means
the same slot in the K and V tensors of every run of that group.  Pages are taken on
demand, portion by portion (``append``), given back when the request ends (``free``) and,
in a windowed group, as soon as the window has passed them (``release_passed``).  A
request also holds one *slot*: the row of its block tables in the host mirror that the
step function uploads, and the row of every per-request state tensor.

The reference has one group, takes the pages of a whole prompt when the request is added
and gives them back only at its end (src/engine/kv_cache_manager.cpp:120-220,
src/engine/engine.cpp:142-173); its block tables are rebuilt and copied every step
(src/engine/block_table.cpp:156-221).  It has no per-request state.

This is host-side bookkeeping only; the device tensors belong to the engine.  The books are
kept by compiled code (csrc/host_runtime.cpp, as the reference keeps them in C++); this class maps
request keys to integers, turns error codes into exceptions and exposes the mirror as arrays.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import native
from .page_pool import OutOfPages, PagePoolError


@dataclass(frozen=True)
class GroupSpec:
    """What the runs of one cache group share."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


class CacheError(RuntimeError):
    pass


class _PoolView:
    """The page pool of one group, as the manager's ``pools[g]``."""

    def __init__(self, lib, handle, group: int) -> None:
        self._lib, self._h, self._g = lib, handle, group
        self.num_pages = lib.ni_cache_pool_num_pages(handle, group)

    @property
    def num_free(self) -> int:
        return self._lib.ni_cache_pool_num_free(self._h, self._g)

    @property
    def num_taken(self) -> int:
        return self.num_pages - self.num_free

    def is_taken(self, page: int) -> bool:
        return bool(self._lib.ni_cache_pool_is_taken(self._h, self._g, int(page)))


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], pages_per_group: Sequence[int], page_size: int,
                 max_requests: int, max_tokens_per_request: int) -> None:
        if page_size <= 0 or max_requests <= 0 or max_tokens_per_request <= 0:
            raise ValueError("page_size, max_requests and max_tokens_per_request must be positive")
        if len(groups) != len(pages_per_group):
            raise ValueError("one page count per group is needed")
        if any(n <= 0 for n in pages_per_group):
            raise ValueError("a page pool needs at least one page")
        self.groups = list(groups)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_tokens_per_request = max_tokens_per_request
        self._lib = lib = native.lib()
        n = len(self.groups)
        pages = (ctypes.c_int32 * n)(*[int(p) for p in pages_per_group])
        windows = (ctypes.c_int32 * n)(*[-1 if g.window is None else int(g.window) for g in self.groups])
        self._h = lib.ni_cache_create(n, pages, windows, page_size, max_requests, max_tokens_per_request)
        if not self._h:
            raise ValueError("the cache manager could not be created from these sizes")
        self.table_width = lib.ni_cache_table_width(self._h)
        self.pools = [_PoolView(lib, self._h, g) for g in range(n)]
        self._windowed = any(g.window is not None for g in self.groups)
        # the compiled manager's mirror of the block tables, one row per slot; -1 = no page
        self.mirror = [np.ctypeslib.as_array(lib.ni_cache_mirror(self._h, g), shape=(max_requests, self.table_width))
                       for g in range(n)]
        # The compiled side knows requests by integers: a non-negative int key is used as it is
        # (so the compiled scheduler and this class mean the same request by an engine's request
        # id), any other key gets a number of its own from a range far above.
        self._keys: Dict[object, int] = {}
        self._next_key = 1 << 62
        self._needed = (ctypes.c_int32 * n)()

    def __del__(self) -> None:
        if getattr(self, "_h", None):
            self.mirror = []
            self._lib.ni_cache_destroy(self._h)
            self._h = None

    # ---- errors ---------------------------------------------------------------------------
    def _raise(self, rc: int, req=None):
        msg = self._lib.ni_cache_last_error(self._h).decode()
        if req is not None:
            msg = f"request {req!r}: {msg}"
        if rc == native.ERR_OUT_OF_PAGES:
            raise OutOfPages(msg)
        if rc == native.ERR_PAGE:
            raise PagePoolError(msg)
        raise CacheError(msg)

    @staticmethod
    def _is_plain(req) -> bool:
        return type(req) is int and 0 <= req < (1 << 62)

    def _key(self, req) -> int:
        if self._is_plain(req):
            if not self._lib.ni_cache_has(self._h, req):
                raise CacheError(f"request {req!r} is not admitted")
            return req
        try:
            return self._keys[req]
        except KeyError:
            raise CacheError(f"request {req!r} is not admitted") from None

    @property
    def table_version(self) -> int:
        """Bumped whenever any row of the mirror changes."""
        return self._lib.ni_cache_table_version(self._h)

    # ---- requests -------------------------------------------------------------------------
    def has(self, req) -> bool:
        if self._is_plain(req):
            return bool(self._lib.ni_cache_has(self._h, req))
        return req in self._keys

    @property
    def num_free_slots(self) -> int:
        return self._lib.ni_cache_num_free_slots(self._h)

    def admit(self, req) -> int:
        """Give ``req`` a slot and empty block tables; returns the slot."""
        if self.has(req):
            raise CacheError(f"request {req!r} is already admitted")
        plain = self._is_plain(req)
        key = req if plain else self._next_key
        slot = self._lib.ni_cache_admit(self._h, key)
        if slot < 0:
            self._raise(slot)
        if not plain:
            self._next_key += 1
            self._keys[req] = key
        return slot

    def slot(self, req) -> int:
        return self._lib.ni_cache_slot(self._h, self._key(req))

    def length(self, req) -> int:
        return self._lib.ni_cache_length(self._h, self._key(req))

    # ---- pages ----------------------------------------------------------------------------
    def pages_needed(self, req, n_new: int) -> List[int]:
        """Pages each group must still take so that ``n_new`` more tokens fit."""
        self._lib.ni_cache_pages_needed(self._h, self._key(req), n_new, self._needed)
        return list(self._needed)

    def pages_for_new_request(self, n_new: int) -> List[int]:
        return [-(-n_new // self.page_size) for _ in self.groups]

    def can_append(self, req, n_new: int, reserve: int = 0) -> bool:
        need = self.pages_needed(req, n_new)
        return all(n <= p.num_free - reserve for n, p in zip(need, self.pools))

    def needs_page_for_one(self, req) -> bool:
        """True if one more token of ``req`` starts a new page (in every group alike)."""
        return self._lib.ni_cache_needs_page_for_one(self._h, self._key(req)) == 1

    def append_one(self, req) -> None:
        """append(req, 1), for the decode loop."""
        rc = self._lib.ni_cache_append_one(self._h, self._key(req))
        if rc != 0:
            self._raise(rc, req)

    def append(self, req, n_new: int) -> None:
        """Take the pages for tokens [length, length + n_new).  All groups or none."""
        if n_new < 0:
            raise ValueError("n_new must not be negative")
        rc = self._lib.ni_cache_append(self._h, self._key(req), n_new)
        if rc != 0:
            self._raise(rc, req)

    def release_passed(self, req) -> int:
        """Give back the pages of windowed groups that no later query can see; returns how many."""
        if not self._windowed:
            return 0
        rc = self._lib.ni_cache_release_passed(self._h, self._key(req))
        if rc < 0:
            self._raise(rc, req)
        return rc

    def free(self, req) -> None:
        """Give back everything ``req`` holds: pages of all groups and its slot."""
        rc = self._lib.ni_cache_free(self._h, self._key(req))
        if rc != 0:
            self._raise(rc, req)
        self._keys.pop(req, None)

    def block_table(self, req, group: int = 0) -> List[int]:
        out = (ctypes.c_int32 * self.table_width)()
        n = self._lib.ni_cache_block_table(self._h, self._key(req), group, out, self.table_width)
        if n < 0:
            self._raise(n, req)
        return list(out[:n])

    def table_rows(self, group: int, slots: Sequence[int], width: Optional[int] = None) -> np.ndarray:
        """Rows of the host mirror for the given slots: int32 [len(slots), width]."""
        rows = self.mirror[group][np.asarray(slots, dtype=np.int64)]
        return rows if width is None else rows[:, :width]

    # ---- accounting -----------------------------------------------------------------------
    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def utilization(self, group: int = 0) -> float:
        return self.pools[group].num_taken / self.pools[group].num_pages

    def check_consistency(self) -> None:
        """Every taken page is held by exactly one request, and nothing else is taken."""
        if self._lib.ni_cache_check(self._h) != 0:
            raise CacheError(self._lib.ni_cache_last_error(self._h).decode())
