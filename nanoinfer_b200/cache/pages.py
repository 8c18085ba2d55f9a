"""Cache pages on the host side: the pool of page ids and the per-request block tables.

A page holds ``page_size`` consecutive positions of one request; one page id addresses the same
page in every layer of its cache group. Groups of layers with different needs (all keys; a window
of them) have pools and block tables of their own. Pages go back to the pool when a request
ends and when a window has passed them, and are handed out again.

Reference: cpp/src/paged.cpp:17-71 (free list as a stack handing out 0,1,2,...; reference counts;
allocate throws when empty; double free throws), cpp/src/paged.cpp:93-127 (block table grown
lazily, position p -> table[p / block_size], offset p % block_size). The reference has one group
and no windows (cpp/src/config.hpp:55-57 holds the fields unused).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


class OutOfPages(RuntimeError):
    """The pool of a cache group cannot cover what was asked for."""


class OutOfSlots(RuntimeError):
    """Every per-request state slot is taken."""


class PagePool:
    """Page ids ``0..num_pages-1`` of one cache group, with reference counts."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("num_pages must be > 0")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # pop() hands out 0, 1, 2, ...
        self._ref = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("page pool is empty")
        p = self._free.pop()
        self._ref[p] = 1
        return p

    def incref(self, page: int) -> None:
        self._check(page)
        if self._ref[page] <= 0:
            raise RuntimeError(f"incref of free page {page}")
        self._ref[page] += 1

    def free(self, page: int) -> None:
        self._check(page)
        if self._ref[page] <= 0:
            raise RuntimeError(f"page {page} freed twice")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        self._check(page)
        return self._ref[page]

    def _check(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise IndexError(f"page id {page} outside 0..{self.num_pages - 1}")


@dataclass(frozen=True)
class GroupSpec:
    """A cache group: schedule entries whose mixers keep the same kind of pages."""
    kv_heads: int
    head_dim: int
    window: int                      # 0: every key is kept; w: only the last w keys are ever read
    entries: Tuple[int, ...]         # schedule entries that own a cache in this group


class RequestCache:
    """What one live request holds: per group a block table (-1 = no page), and a state slot."""

    def __init__(self, request_id, slot: int, num_groups: int):
        self.request_id = request_id
        self.slot = slot
        self.length = 0                                   # positions committed
        self.tables: List[List[int]] = [[] for _ in range(num_groups)]
        self.first_live: List[int] = [0] * num_groups     # first logical page still held
        self.version = 0                                  # counts the changes of the block tables
        self.closed = False

    def pages_held(self, group: int) -> int:
        return sum(1 for p in self.tables[group] if p >= 0)


class CacheManager:
    """Pools, block tables and state slots for up to ``max_requests`` live requests."""

    def __init__(self, groups: Sequence[GroupSpec], num_pages: int, page_size: int, max_requests: int):
        if page_size <= 0:
            raise ValueError("page_size must be > 0")
        self.groups = list(groups)
        self.page_size = page_size
        self.num_pages = num_pages
        self.pools = [PagePool(num_pages) for _ in self.groups]
        self.max_requests = max_requests
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self.live: Dict[object, RequestCache] = {}
        self.fresh_slots: List[int] = []   # slots handed out since the storage last zeroed them

    # ---- requests -------------------------------------------------------------------------
    def open(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise KeyError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_requests} state slots are taken")
        rc = RequestCache(request_id, self._free_slots.pop(), len(self.groups))
        self.live[request_id] = rc
        self.fresh_slots.append(rc.slot)
        return rc

    def close(self, rc: RequestCache) -> None:
        """Give back every page and the state slot of a request."""
        if rc.closed:
            raise RuntimeError(f"request {rc.request_id!r} closed twice")
        for g, table in enumerate(rc.tables):
            for p in table:
                if p >= 0:
                    self.pools[g].free(p)
            table.clear()
        rc.closed = True
        self._free_slots.append(rc.slot)
        del self.live[rc.request_id]

    # ---- pages ----------------------------------------------------------------------------
    def _first_needed_page(self, group: int, length_before: int) -> int:
        """First logical page that queries at positions >= length_before can still read."""
        w = self.groups[group].window
        if not w:
            return 0
        return max(0, length_before - w + 1) // self.page_size

    def pages_needed(self, rc: RequestCache, n_new: int) -> List[int]:
        """New pages per group so that positions ``[length, length + n_new)`` have a page."""
        end_page = -(-(rc.length + n_new) // self.page_size)
        need = []
        for g, table in enumerate(rc.tables):
            have = len(table)
            need.append(max(0, end_page - max(have, 0)))
        return need

    def fits(self, demands: Sequence[Tuple[RequestCache, int]]) -> bool:
        total = [0] * len(self.groups)
        for rc, n in demands:
            for g, k in enumerate(self.pages_needed(rc, n)):
                total[g] += k
        return all(total[g] <= self.pools[g].num_free for g in range(len(self.groups)))

    def extend(self, rc: RequestCache, n_new: int) -> None:
        """Allocate the pages for the next ``n_new`` positions (all of them, or none and OutOfPages)."""
        need = self.pages_needed(rc, n_new)
        for g, k in enumerate(need):
            if k > self.pools[g].num_free:
                raise OutOfPages(
                    f"request {rc.request_id!r} needs {k} pages of group {g}, {self.pools[g].num_free} are free")
        for g, k in enumerate(need):
            for _ in range(k):
                rc.tables[g].append(self.pools[g].allocate())
            if k:
                rc.version += 1

    def commit(self, rc: RequestCache, n_new: int) -> None:
        """The step wrote ``n_new`` positions: advance, and return pages that a window has passed."""
        rc.length += n_new
        for table in rc.tables:
            if rc.length > len(table) * self.page_size:
                raise RuntimeError("commit beyond the pages held")
        for g in range(len(self.groups)):
            first = self._first_needed_page(g, rc.length)
            table = rc.tables[g]
            for lp in range(rc.first_live[g], min(first, len(table))):
                if table[lp] >= 0:
                    self.pools[g].free(table[lp])
                    table[lp] = -1
                    rc.version += 1
            rc.first_live[g] = max(rc.first_live[g], min(first, len(table)))

    # ---- views ----------------------------------------------------------------------------
    def capacity_tokens(self) -> int:
        """Positions that one request alone could hold (limited by the groups that keep every key)."""
        return self.num_pages * self.page_size

    def table_width(self, rcs: Sequence[RequestCache]) -> int:
        return max((len(t) for rc in rcs for t in rc.tables), default=0)

    def num_free(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def take_fresh_slots(self) -> List[int]:
        s, self.fresh_slots = self.fresh_slots, []
        return s

    def check(self) -> None:
        """Every page is either free or held exactly as often as its reference count says."""
        for g, pool in enumerate(self.pools):
            held: Dict[int, int] = {}
            for rc in self.live.values():
                for p in rc.tables[g]:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            free = set(pool._free)
            if len(free) != len(pool._free):
                raise AssertionError(f"group {g}: a page is on the free list twice")
            for p in range(pool.num_pages):
                n = held.get(p, 0)
                if n != pool.refcount(p):
                    raise AssertionError(f"group {g}: page {p} held {n} times, refcount {pool.refcount(p)}")
                if (n == 0) != (p in free):
                    raise AssertionError(f"group {g}: page {p} is lost or both free and held")
        slots = [rc.slot for rc in self.live.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise AssertionError("a state slot is lost")
