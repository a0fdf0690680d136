"""Cache manager: block tables per request and layer group, reclamation, state slots.

Layers whose mixers keep the same kind of cache (same kv heads, head size and window) form
a group.  A group has pages of its own: its own allocator, its own block table per request
and its own rule for giving pages back:

  * all-keys group: pages return when the request ends;
  * window-W group: after a step that brings a request to length L, every page whose last
    position is <= L - W can never be read again (the next query sits at p >= L and sees
    j > p - W) and returns at once; its block-table entry becomes -1.

Beside the pages each live request owns one slot index into fixed-size state arrays
(the reference keeps GatedDeltaNet state that way, crates/model/src/gdn_state.rs:64-116,
reset when a sequence starts at length 0, crates/model/src/cache.rs:612-617).

The bookkeeping itself is C++ (``csrc/host_cache.cpp``, part of the engine's shared library,
no CUDA in it); this module is its Python face.  The device arrays live in ``storage``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np


class OutOfPages(RuntimeError):
    """The pool of a group cannot supply the pages asked for.  Nothing was taken."""

    def __init__(self, group: int, wanted: int, free: int):
        super().__init__(f"cache group {group}: {wanted} pages wanted, {free} free")
        self.group, self.wanted, self.free = group, wanted, free


class OutOfSlots(RuntimeError):
    pass


@dataclass(frozen=True)
class GroupSpec:
    """What the bookkeeping needs to know of a group: its window (None = all keys)."""
    window: Optional[int] = None


def _lib():
    from ..kernels import lib
    L = lib()
    if not getattr(L, "_cache_api_ready", False):
        L.infero_cache_new.restype = ctypes.c_void_p
        L.infero_cache_mirror.restype = ctypes.POINTER(ctypes.c_int)
        L.infero_cache_counter.restype = ctypes.c_longlong
        L.infero_cache_error.restype = ctypes.c_char_p
        L.infero_step_layout.restype = ctypes.c_longlong
        L._cache_api_ready = True
    return L


class RequestCache:
    """One live request as the cache sees it (a view of the C++ record of its slot)."""
    __slots__ = ("rid", "slot", "_m")

    def __init__(self, rid: Hashable, slot: int, manager: "CacheManager"):
        self.rid, self.slot, self._m = rid, slot, manager

    @property
    def length(self) -> int:                     # tokens whose keys are in the cache
        return self._m._L.infero_cache_length(self._m._h, self.slot)

    @property
    def reserved(self) -> int:                   # tokens reserved by the running step, not yet committed
        return self._m._L.infero_cache_reserved(self._m._h, self.slot)

    @property
    def fresh(self) -> bool:                     # nothing committed yet: state slots still have to be zeroed
        return bool(self._m._L.infero_cache_fresh(self._m._h, self.slot))

    @property
    def tables(self) -> List[List[int]]:         # per group: logical page -> page id, -1 once given back
        m = self._m
        return [[int(p) for p in m._mirror(g)[self.slot, :m._L.infero_cache_table_len(m._h, g, self.slot)]]
                for g in range(len(m.groups))]

    def table_len(self, group: int) -> int:
        return self._m._L.infero_cache_table_len(self._m._h, group, self.slot)

    @property
    def first_live(self) -> List[int]:
        m = self._m
        return [m._L.infero_cache_first_live(m._h, g, self.slot) for g in range(len(m.groups))]


class _AllocatorView:
    """Read-only view of one group's page pool."""

    def __init__(self, manager: "CacheManager", group: int):
        self._m, self.group = manager, group
        self.num_pages = manager.pages_per_group[group]

    @property
    def num_free(self) -> int:
        return self._m._L.infero_cache_num_free(self._m._h, self.group)

    def held_pages(self) -> List[int]:
        buf = (ctypes.c_int * self.num_pages)()
        n = self._m._L.infero_cache_held(self._m._h, self.group, buf, self.num_pages)
        return [int(buf[i]) for i in range(n)]


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], num_pages, page_size: int, max_requests: int,
                 max_blocks: Optional[int] = None):
        """``num_pages``: the pool size of every group, or one size per group (each group has a pool of
        its own; a window group gets by with far fewer pages than a group that keeps every key)."""
        self.groups = list(groups)
        per_group = [int(num_pages)] * len(self.groups) if isinstance(num_pages, int) else [int(n) for n in num_pages]
        if len(per_group) != len(self.groups):
            raise ValueError(f"{len(per_group)} pool sizes for {len(self.groups)} groups")
        if any(n <= 0 for n in per_group) or (isinstance(num_pages, int) and num_pages <= 0):
            raise ValueError("a page pool needs at least one page")
        self.page_size = page_size
        self.pages_per_group = per_group
        self.num_pages = max(per_group, default=int(num_pages) if isinstance(num_pages, int) else 0)
        self.max_requests = max_requests
        self.max_blocks = max_blocks
        self._L = _lib()
        windows = (ctypes.c_int * max(1, len(self.groups)))(*[int(g.window or 0) for g in self.groups])
        pages = (ctypes.c_int * max(1, len(self.groups)))(*per_group)
        self._h = ctypes.c_void_p(self._L.infero_cache_new(len(self.groups), windows, pages, page_size,
                                                           max_requests, int(max_blocks or 0)))
        if not self._h:
            raise ValueError("bad cache geometry")
        self.allocators = [_AllocatorView(self, g) for g in range(len(self.groups))]
        self.requests: Dict[Hashable, RequestCache] = {}
        self._need = (ctypes.c_int * max(1, len(self.groups)))()
        self._info = (ctypes.c_int * 3)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._L.infero_cache_delete(h)

    def _mirror(self, group: int) -> np.ndarray:
        """[max_requests, width] int32 view of the C++ side's copy of every block table."""
        width = self._L.infero_cache_width(self._h)
        ptr = self._L.infero_cache_mirror(self._h, group)
        return np.ctypeslib.as_array(ptr, shape=(self.max_requests, width))

    @property
    def pages_reclaimed(self) -> int:             # window pages returned before their request ended
        return int(self._L.infero_cache_counter(self._h, 0))

    @property
    def pages_reused(self) -> int:                # allocations served by a page that was held before
        return int(self._L.infero_cache_counter(self._h, 1))

    # ---- requests ------------------------------------------------------------------------
    def open(self, rid: Hashable) -> RequestCache:
        if rid in self.requests:
            raise KeyError(f"request {rid!r} is already open")
        slot = self._L.infero_cache_open(self._h)
        if slot < 0:
            raise OutOfSlots(f"all {self.max_requests} request slots are in use")
        rc = RequestCache(rid, slot, self)
        self.requests[rid] = rc
        return rc

    def close(self, rid: Hashable) -> None:
        rc = self.requests.pop(rid)
        self._L.infero_cache_close(self._h, rc.slot)

    def adopt(self, rid: Hashable, slot: int) -> RequestCache:
        """A slot that native code (the scheduler) has opened for ``rid``."""
        if rid in self.requests:
            raise KeyError(f"request {rid!r} is already open")
        rc = RequestCache(rid, slot, self)
        self.requests[rid] = rc
        return rc

    def forget(self, rid: Hashable) -> None:
        """The slot of ``rid`` was closed by native code."""
        self.requests.pop(rid, None)

    def get(self, rid: Hashable) -> RequestCache:
        return self.requests[rid]

    # ---- pages ---------------------------------------------------------------------------
    def pages_needed(self, rc: RequestCache, n_new: int) -> List[int]:
        """New pages per group to hold n_new more tokens after what is held or reserved."""
        self._L.infero_cache_pages_needed(self._h, rc.slot, int(n_new), self._need)
        return [int(self._need[g]) for g in range(len(self.groups))]

    def free_pages(self, group: int = 0) -> int:
        return self._L.infero_cache_num_free(self._h, group)

    def reserve(self, rc: RequestCache, n_new: int) -> None:
        """Take the pages n_new more tokens need, in every group, or none at all."""
        if n_new <= 0:
            raise ValueError("reserve needs at least one token")
        rcode = self._L.infero_cache_reserve(self._h, rc.slot, int(n_new), self._info)
        if rcode:
            raise OutOfPages(int(self._info[0]), int(self._info[1]), int(self._info[2]))

    def commit(self, rc: RequestCache, n_new: int) -> None:
        """The step wrote n_new tokens: advance, and give back what a window has passed."""
        if self._L.infero_cache_commit(self._h, rc.slot, int(n_new)):
            raise ValueError("commit of more tokens than were reserved")

    def truncate(self, rc: RequestCache, length: int) -> None:
        """Forget the request's tokens from position ``length`` on; pages wholly behind the new end go
        back (the reference's ``KvPool::truncate``, crates/model/src/cache.rs:656-679).  A window group
        that has already given back keys a query at ``length`` would see cannot go back that far."""
        rcode = self._L.infero_cache_truncate(self._h, rc.slot, int(length))
        if rcode == 2:
            raise ValueError(f"request {rc.rid!r}: a window group no longer holds the keys position {length} sees")
        if rcode:
            raise ValueError(f"request {rc.rid!r} holds {rc.length} tokens (reserved {rc.reserved}); cannot cut to {length}")

    def abort_reservation(self, rc: RequestCache) -> None:
        """Drop pages reserved for a step that did not run."""
        self._L.infero_cache_abort(self._h, rc.slot)

    # ---- tables for the device -----------------------------------------------------------
    def step_layout(self, slots: np.ndarray, n_tokens: np.ndarray, tokens: np.ndarray, want_counts: np.ndarray,
                    wants: np.ndarray, table_width: int, out: np.ndarray, n_pad: int = 0, pad_slot: int = 0) -> List[int]:
        """Write a step's int32 arrays into ``out`` (see csrc/host_cache.cpp: token ids, positions,
        token -> entry, per entry first row / row count / cached length / slot, wanted rows, one
        block table per group) and return the section sizes.  All arguments are int32 arrays.
        ``n_pad`` entries of a request that does not exist follow the real ones (token 0 at position
        0, state slot ``pad_slot``, and in every group the single page past the group's pool)."""
        sizes = (ctypes.c_longlong * (8 + len(self.groups)))()
        as_p = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))     # noqa: E731
        total = self._L.infero_step_layout(self._h, int(slots.size), as_p(slots), as_p(n_tokens), as_p(tokens),
                                           as_p(want_counts), as_p(wants), int(table_width), as_p(out),
                                           ctypes.c_longlong(out.size), sizes, int(n_pad), int(pad_slot))
        if total < 0:
            raise ValueError("step layout does not fit its buffer, or a request holds more pages than the table is wide")
        return [int(v) for v in sizes]

    # ---- invariants (used by tests and debug runs) -----------------------------------------
    def check(self) -> None:
        if self._L.infero_cache_check(self._h):
            raise AssertionError(self._L.infero_cache_error(self._h).decode())
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots):
            raise AssertionError("a state slot is held twice")
