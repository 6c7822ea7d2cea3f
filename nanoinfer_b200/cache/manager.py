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

This class is host-side bookkeeping only; the device tensors belong to the engine.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from .page_pool import OutOfPages, PagePool


@dataclass(frozen=True)
class GroupSpec:
    """What the runs of one cache group share."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


class CacheError(RuntimeError):
    pass


class _Held:
    __slots__ = ("slot", "length", "tables", "first_live")

    def __init__(self, slot: int, n_groups: int) -> None:
        self.slot = slot
        self.length = 0                       # tokens whose keys/values are (being) cached
        self.tables: List[List[int]] = [[] for _ in range(n_groups)]
        self.first_live = [0] * n_groups      # index of the first page not yet released


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], pages_per_group: Sequence[int], page_size: int,
                 max_requests: int, max_tokens_per_request: int) -> None:
        if page_size <= 0 or max_requests <= 0 or max_tokens_per_request <= 0:
            raise ValueError("page_size, max_requests and max_tokens_per_request must be positive")
        if len(groups) != len(pages_per_group):
            raise ValueError("one page count per group is needed")
        self.groups = list(groups)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_tokens_per_request = max_tokens_per_request
        self.table_width = -(-max_tokens_per_request // page_size)
        self.pools = [PagePool(n) for n in pages_per_group]
        self._windowed = any(g.window is not None for g in self.groups)
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._held: Dict[object, _Held] = {}
        # host mirror of the block tables, one row per slot; -1 = no page
        self.mirror = [np.full((max_requests, self.table_width), -1, dtype=np.int32)
                       for _ in self.groups]
        self.table_version = 0     # bumped whenever any row of the mirror changes

    # ---- requests -------------------------------------------------------------------------
    def has(self, req) -> bool:
        return req in self._held

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self, req) -> int:
        """Give ``req`` a slot and empty block tables; returns the slot."""
        if req in self._held:
            raise CacheError(f"request {req!r} is already admitted")
        if not self._free_slots:
            raise CacheError("no free request slot")
        slot = self._free_slots.pop()
        self._held[req] = _Held(slot, len(self.groups))
        for m in self.mirror:
            m[slot, :] = -1
        self.table_version += 1
        return slot

    def slot(self, req) -> int:
        return self._get(req).slot

    def length(self, req) -> int:
        return self._get(req).length

    def _get(self, req) -> _Held:
        try:
            return self._held[req]
        except KeyError:
            raise CacheError(f"request {req!r} is not admitted") from None

    # ---- pages ----------------------------------------------------------------------------
    def _first_needed_page(self, g: int, length: int) -> int:
        """Index of the first page that a query at position >= ``length`` can still see."""
        w = self.groups[g].window
        if w is None:
            return 0
        return max(0, length - w + 1) // self.page_size

    def pages_needed(self, req, n_new: int) -> List[int]:
        """Pages each group must still take so that ``n_new`` more tokens fit."""
        h = self._get(req)
        total = -(-(h.length + n_new) // self.page_size)
        return [total - len(t) for t in h.tables]

    def pages_for_new_request(self, n_new: int) -> List[int]:
        return [-(-n_new // self.page_size) for _ in self.groups]

    def can_append(self, req, n_new: int, reserve: int = 0) -> bool:
        need = self.pages_needed(req, n_new)
        return all(n <= p.num_free - reserve for n, p in zip(need, self.pools))

    def needs_page_for_one(self, req) -> bool:
        """True if one more token of ``req`` starts a new page (in every group alike)."""
        return self._get(req).length % self.page_size == 0

    def append_one(self, req) -> None:
        """append(req, 1), for the decode loop."""
        h = self._get(req)
        if h.length % self.page_size == 0:
            self.append(req, 1)
        elif h.length + 1 > self.max_tokens_per_request:
            self.append(req, 1)          # raises the limit error
        else:
            h.length += 1

    def append(self, req, n_new: int) -> None:
        """Take the pages for tokens [length, length + n_new).  All groups or none."""
        h = self._get(req)
        if n_new < 0:
            raise ValueError("n_new must not be negative")
        if h.length + n_new > self.max_tokens_per_request:
            raise CacheError(f"request {req!r} would hold {h.length + n_new} tokens, more than "
                             f"max_tokens_per_request {self.max_tokens_per_request}")
        need = self.pages_needed(req, n_new)
        for g, n in enumerate(need):
            if n > self.pools[g].num_free:
                raise OutOfPages(f"group {g}: request {req!r} needs {n} more pages, "
                                 f"{self.pools[g].num_free} are free")
        for g, n in enumerate(need):
            if n > 0:
                pages = self.pools[g].take(n)
                start = len(h.tables[g])
                h.tables[g].extend(pages)
                self.mirror[g][h.slot, start:start + n] = pages
                self.table_version += 1
        h.length += n_new

    def release_passed(self, req) -> int:
        """Give back the pages of windowed groups that no later query can see; returns how many."""
        if not self._windowed:
            return 0
        h = self._get(req)
        released = 0
        for g in range(len(self.groups)):
            if self.groups[g].window is None:
                continue
            first = min(self._first_needed_page(g, h.length), len(h.tables[g]))
            if first > h.first_live[g]:
                pages = h.tables[g][h.first_live[g]:first]
                self.pools[g].give_back(pages)
                for i in range(h.first_live[g], first):
                    h.tables[g][i] = -1
                self.mirror[g][h.slot, h.first_live[g]:first] = -1
                self.table_version += 1
                released += len(pages)
                h.first_live[g] = first
        return released

    def free(self, req) -> None:
        """Give back everything ``req`` holds: pages of all groups and its slot."""
        h = self._get(req)
        for g, table in enumerate(h.tables):
            self.pools[g].give_back([p for p in table if p >= 0])
            self.mirror[g][h.slot, :] = -1
        self.table_version += 1
        self._free_slots.append(h.slot)
        del self._held[req]

    def block_table(self, req, group: int = 0) -> List[int]:
        return list(self._get(req).tables[group])

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
        for g, pool in enumerate(self.pools):
            held = [p for h in self._held.values() for p in h.tables[g] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g}: a page is held twice")
            if len(held) != pool.num_taken or any(not pool.is_taken(p) for p in held):
                raise CacheError(f"group {g}: {pool.num_taken} pages taken, {len(held)} held")
        slots = [h.slot for h in self._held.values()]
        if len(slots) != len(set(slots)) or len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("request slots are inconsistent")
