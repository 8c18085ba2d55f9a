"""Cache pages on the host side: the pool of page ids and the per-request block tables.

A page holds ``page_size`` consecutive positions of one request; one page id addresses the same
page in every layer of its cache group. Groups of layers with different needs (all keys; a window
of them) have pools and block tables of their own. Pages go back to the pool when a request
ends and when a window has passed them, and are handed out again. The pool's books (free stack,
reference counts) are kept in native code (``csrc/host/page_pool.cpp``); tables and slots here.

Reference: cpp/src/paged.cpp:17-71 (free list as a stack handing out 0,1,2,...; reference counts;
allocate throws when empty; double free throws), cpp/src/paged.cpp:93-127 (block table grown
lazily, position p -> table[p / block_size], offset p % block_size). The reference has one group
and no windows (cpp/src/config.hpp:55-57 holds the fields unused).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple


class OutOfPages(RuntimeError):
    """The pool of a cache group cannot cover what was asked for."""


class OutOfSlots(RuntimeError):
    """Every per-request state slot is taken."""


_host_lib = None


def _host():
    """The host runtime library (built with the host compiler at first use), with its signatures set."""
    global _host_lib
    if _host_lib is None:
        from ..csrc.build import build_host
        lib = ctypes.CDLL(build_host())
        i32, ptr, i32p = ctypes.c_int32, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)
        if lib.nibh_abi_version() != 1:
            raise RuntimeError("the host runtime library is of another version than this package")
        lib.nibh_pool_create.restype, lib.nibh_pool_create.argtypes = ptr, [i32]
        lib.nibh_pool_destroy.restype, lib.nibh_pool_destroy.argtypes = None, [ptr]
        lib.nibh_pool_num_free.restype, lib.nibh_pool_num_free.argtypes = i32, [ptr]
        lib.nibh_pool_allocate.restype, lib.nibh_pool_allocate.argtypes = i32, [ptr, i32, i32p]
        lib.nibh_pool_incref.restype, lib.nibh_pool_incref.argtypes = i32, [ptr, i32]
        lib.nibh_pool_free.restype, lib.nibh_pool_free.argtypes = i32, [ptr, i32p, i32, i32p]
        lib.nibh_pool_refcount.restype, lib.nibh_pool_refcount.argtypes = i32, [ptr, i32]
        lib.nibh_pool_free_list.restype, lib.nibh_pool_free_list.argtypes = i32, [ptr, i32p, i32]
        _host_lib = lib
    return _host_lib


_EMPTY, _BAD_PAGE, _NOT_HELD = -1, -2, -3


class PagePool:
    """Page ids ``0..num_pages-1`` of one cache group, with reference counts. The books are kept by the
    native allocator (``csrc/host/page_pool.cpp``); this class turns its status codes into exceptions."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("num_pages must be > 0")
        self.num_pages = num_pages
        self._lib = _host()
        self._pool = ctypes.c_void_p(self._lib.nibh_pool_create(num_pages))
        if not self._pool:
            raise MemoryError(f"no memory for a pool of {num_pages} pages")
        self._one = (ctypes.c_int32 * 1)()

    def __del__(self):
        pool, self._pool = getattr(self, "_pool", None), None
        if pool:
            try:
                self._lib.nibh_pool_destroy(pool)
            except Exception:       # the interpreter is shutting down and the library is gone already
                pass

    @property
    def num_free(self) -> int:
        return self._lib.nibh_pool_num_free(self._pool)

    def allocate(self) -> int:
        if self._lib.nibh_pool_allocate(self._pool, 1, self._one) != 0:
            raise OutOfPages("page pool is empty")
        return self._one[0]

    def allocate_many(self, n: int) -> List[int]:
        """``n`` pages, all of them or none (``OutOfPages``), in the order a loop of ``allocate`` gives."""
        out = (ctypes.c_int32 * max(n, 1))()
        if self._lib.nibh_pool_allocate(self._pool, n, out) != 0:
            raise OutOfPages(f"{n} pages asked for, {self.num_free} are free")
        return out[:n]

    def incref(self, page: int) -> None:
        self._raise(self._lib.nibh_pool_incref(self._pool, page), page, "incref of free page {}")

    def free(self, page: int) -> None:
        self._check(page)
        self._one[0] = page
        self._raise(self._lib.nibh_pool_free(self._pool, self._one, 1, None), page, "page {} freed twice")

    def free_many(self, pages: Sequence[int]) -> None:
        """Drops one reference of every page in ``pages``; entries below zero (no page) are skipped."""
        n = len(pages)
        arr = (ctypes.c_int32 * max(n, 1))(*pages)
        done = ctypes.c_int32(0)
        status = self._lib.nibh_pool_free(self._pool, arr, n, ctypes.byref(done))
        if status != 0:
            self._raise(status, pages[done.value], "page {} freed twice")

    def refcount(self, page: int) -> int:
        r = self._lib.nibh_pool_refcount(self._pool, page)
        if r < 0:
            self._raise(r, page, "")
        return r

    def free_pages(self) -> List[int]:
        """The free list, bottom of the stack first (the last one is handed out next)."""
        out = (ctypes.c_int32 * self.num_pages)()
        n = self._lib.nibh_pool_free_list(self._pool, out, self.num_pages)
        return out[:n]

    def _check(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise IndexError(f"page id {page} outside 0..{self.num_pages - 1}")

    def _raise(self, status: int, page: int, not_held: str) -> None:
        if status == 0:
            return
        if status == _BAD_PAGE:
            raise IndexError(f"page id {page} outside 0..{self.num_pages - 1}")
        if status == _NOT_HELD:
            raise RuntimeError(not_held.format(page))
        raise RuntimeError(f"page allocator: status {status}")


@dataclass(frozen=True)
class GroupSpec:
    """A cache group: schedule entries whose mixers keep the same kind of pages. The manager counts pages and
    positions only; what a page holds (``tensors``: name, heads, width, dtype of each tensor kept per token) matters
    to the storage alone."""
    window: int                      # 0: every key is kept; w: only the last w keys are ever read
    entries: Tuple[int, ...]         # schedule entries that own a cache in this group
    tensors: Tuple = ()              # the PagedTensor descriptions of the group's entries


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
        self._window_groups = [g for g, spec in enumerate(self.groups) if spec.window]   # the others never return pages early
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
            self.pools[g].free_many(table)
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
        return [max(0, end_page - len(table)) for table in rc.tables]

    def demand(self, demands: Sequence[Tuple[RequestCache, int]]) -> List[int]:
        """Pages per group that the given (request, new positions) pairs need together."""
        total = [0] * len(self.groups)
        ps = self.page_size
        for rc, n in demands:
            end_page = -(-(rc.length + n) // ps)
            for g, table in enumerate(rc.tables):
                if end_page > len(table):
                    total[g] += end_page - len(table)
        return total

    def fits(self, demands: Sequence[Tuple[RequestCache, int]]) -> bool:
        return all(k <= pool.num_free for k, pool in zip(self.demand(demands), self.pools))

    def extend(self, rc: RequestCache, n_new: int) -> None:
        """Allocate the pages for the next ``n_new`` positions (all of them, or none and OutOfPages)."""
        end = rc.length + n_new
        ps = self.page_size
        for table in rc.tables:
            if end > len(table) * ps:
                break
        else:
            return                      # the usual decode step: the last page still has room
        need = self.pages_needed(rc, n_new)
        for g, k in enumerate(need):
            if k > self.pools[g].num_free:
                raise OutOfPages(
                    f"request {rc.request_id!r} needs {k} pages of group {g}, {self.pools[g].num_free} are free")
        for g, k in enumerate(need):
            if k:
                rc.tables[g].extend(self.pools[g].allocate_many(k))
                rc.version += 1

    def commit(self, rc: RequestCache, n_new: int) -> None:
        """The step wrote ``n_new`` positions: advance, and return pages that a window has passed."""
        rc.length += n_new
        for table in rc.tables:
            if rc.length > len(table) * self.page_size:
                raise RuntimeError("commit beyond the pages held")
        for g in self._window_groups:
            first = self._first_needed_page(g, rc.length)
            table = rc.tables[g]
            for lp in range(rc.first_live[g], min(first, len(table))):
                if table[lp] >= 0:
                    self.pools[g].free(table[lp])
                    table[lp] = -1
                    rc.version += 1
            rc.first_live[g] = max(rc.first_live[g], min(first, len(table)))

    def truncate(self, rc: RequestCache, new_length: int) -> None:
        """Forget the positions from ``new_length`` on: what is fed next overwrites their keys and values. Pages
        that hold no position any more are returned. A group with a window cannot go back to a position whose
        window reaches into pages that it has already given back."""
        if rc.closed or not (0 <= new_length <= rc.length):
            raise ValueError(f"request {rc.request_id!r}: cannot truncate {rc.length} positions to {new_length}")
        for g in self._window_groups:
            if self._first_needed_page(g, new_length) < rc.first_live[g]:
                raise ValueError(f"request {rc.request_id!r}: the window's pages for position {new_length} were returned")
        keep = -(-new_length // self.page_size)
        for g, table in enumerate(rc.tables):
            if len(table) > keep:
                self.pools[g].free_many(table[keep:])
                del table[keep:]
                rc.version += 1
        rc.length = new_length

    # ---- views ----------------------------------------------------------------------------
    def capacity_tokens(self) -> int:
        """Positions that one request alone could hold (limited by the groups that keep every key)."""
        return self.num_pages * self.page_size

    def table_width(self, rcs: Sequence[RequestCache]) -> int:
        return max((len(t) for rc in rcs for t in rc.tables), default=0)

    def table_widths(self, positions: int) -> List[int]:
        """Per group, the block-table entries that address ``positions`` positions of a request. A captured step asks
        here for its tables' widths, so a group with pages of another size, or with a table of fixed width, answers
        for itself in this one place. (A windowed group keeps one entry per page of the whole sequence, the ones
        behind the window being -1, so today every group answers alike.)"""
        return [max(1, -(-positions // self.page_size)) for _ in self.groups]

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
            free_list = pool.free_pages()
            free = set(free_list)
            if len(free) != len(free_list):
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
