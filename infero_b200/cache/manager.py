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

This module is host-only bookkeeping; the device arrays live in ``storage``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from .pages import OutOfPages, PageAllocator


class OutOfSlots(RuntimeError):
    pass


@dataclass(frozen=True)
class GroupSpec:
    """What the bookkeeping needs to know of a group: its window (None = all keys)."""
    window: Optional[int] = None


@dataclass
class RequestCache:
    rid: Hashable
    slot: int
    length: int = 0                       # tokens whose keys are in the cache
    reserved: int = 0                     # tokens reserved by the running step, not yet committed
    tables: List[List[int]] = field(default_factory=list)   # per group: logical page -> page id / -1
    first_live: List[int] = field(default_factory=list)     # per group: first logical page still held
    fresh: bool = True                    # state slot still has to be zeroed


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], num_pages: int, page_size: int, max_requests: int,
                 max_blocks: Optional[int] = None):
        self.groups = list(groups)
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.max_blocks = max_blocks
        self.allocators = [PageAllocator(num_pages, g) for g in range(len(self.groups))]
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self.requests: Dict[Hashable, RequestCache] = {}
        # device-bound copy of every block table, one row per request slot, kept up to date as
        # pages come and go, so that a step gathers its rows instead of rebuilding them
        self._table_width = max_blocks if max_blocks is not None else 0
        self._table_np = [np.full((max_requests, max(1, self._table_width)), -1, dtype=np.int32)
                          for _ in self.groups]
        self.pages_reclaimed = 0          # window pages returned before their request ended
        self.pages_reused = 0             # allocations served by a page that was held before
        self._ever_held = [bytearray(num_pages) for _ in self.groups]

    # ---- requests ------------------------------------------------------------------------
    def open(self, rid: Hashable) -> RequestCache:
        if rid in self.requests:
            raise KeyError(f"request {rid!r} is already open")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_requests} request slots are in use")
        rc = RequestCache(rid=rid, slot=self._free_slots.pop(),
                          tables=[[] for _ in self.groups], first_live=[0 for _ in self.groups])
        self.requests[rid] = rc
        for t in self._table_np:
            t[rc.slot, :] = -1
        return rc

    def close(self, rid: Hashable) -> None:
        rc = self.requests.pop(rid)
        for g, table in enumerate(rc.tables):
            self.allocators[g].free([p for p in table if p >= 0])
        self._free_slots.append(rc.slot)

    def get(self, rid: Hashable) -> RequestCache:
        return self.requests[rid]

    # ---- pages ---------------------------------------------------------------------------
    def pages_needed(self, rc: RequestCache, n_new: int) -> List[int]:
        """New pages per group to hold n_new more tokens after what is held or reserved."""
        end = rc.length + rc.reserved + n_new
        want = -(-end // self.page_size)
        return [max(0, want - len(t)) for t in rc.tables]

    def can_reserve(self, items: Sequence[Tuple[RequestCache, int]]) -> bool:
        need = [0] * len(self.groups)
        for rc, n in items:
            for g, k in enumerate(self.pages_needed(rc, n)):
                need[g] += k
        return all(need[g] <= self.allocators[g].num_free for g in range(len(self.groups)))

    def free_pages(self, group: int = 0) -> int:
        return self.allocators[group].num_free

    def min_free_pages(self) -> int:
        return min((a.num_free for a in self.allocators), default=self.num_pages)

    def reserve(self, rc: RequestCache, n_new: int) -> None:
        """Take the pages n_new more tokens need, in every group, or none at all."""
        if n_new <= 0:
            raise ValueError("reserve needs at least one token")
        need = self.pages_needed(rc, n_new)
        if self.max_blocks is not None:
            want = -(-(rc.length + rc.reserved + n_new) // self.page_size)
            if want > self.max_blocks:
                raise OutOfPages(-1, want, self.max_blocks)
        for g, k in enumerate(need):
            if k > self.allocators[g].num_free:
                raise OutOfPages(g, k, self.allocators[g].num_free)
        for g, k in enumerate(need):
            pages = self.allocators[g].alloc(k)
            for p in pages:
                if self._ever_held[g][p]:
                    self.pages_reused += 1
                self._ever_held[g][p] = 1
            first = len(rc.tables[g])
            rc.tables[g].extend(pages)
            if pages:
                self._mirror(g, rc.slot, first, pages)
        rc.reserved += n_new

    def commit(self, rc: RequestCache, n_new: int) -> None:
        """The step wrote n_new tokens: advance, and give back what a window has passed."""
        if n_new > rc.reserved:
            raise ValueError("commit of more tokens than were reserved")
        rc.reserved -= n_new
        rc.length += n_new
        rc.fresh = False
        P = self.page_size
        for g, spec in enumerate(self.groups):
            if spec.window is None:
                continue
            # logical page k covers [kP, kP+P-1]; dead iff kP + P - 1 <= length - window
            dead_upto = (rc.length - spec.window + 1) // P if rc.length - spec.window + 1 > 0 else 0
            table = rc.tables[g]
            k = rc.first_live[g]
            freed = []
            while k < dead_upto and k < len(table):
                if table[k] >= 0:
                    freed.append(table[k])
                    table[k] = -1
                    if k < self._table_np[g].shape[1]:
                        self._table_np[g][rc.slot, k] = -1
                k += 1
            rc.first_live[g] = k
            if freed:
                self.allocators[g].free(freed)
                self.pages_reclaimed += len(freed)

    def abort_reservation(self, rc: RequestCache) -> None:
        """Drop pages reserved for a step that did not run."""
        if rc.reserved == 0:
            return
        keep = -(-rc.length // self.page_size)
        for g, table in enumerate(rc.tables):
            extra = [p for p in table[keep:] if p >= 0]
            del table[keep:]
            self.allocators[g].free(extra)
            self._table_np[g][rc.slot, keep:] = -1
        rc.reserved = 0

    # ---- tables for the device -----------------------------------------------------------
    def _mirror(self, group: int, slot: int, first: int, pages) -> None:
        t = self._table_np[group]
        end = first + len(pages)
        if end > t.shape[1]:                       # no fixed width was given: grow
            wider = np.full((t.shape[0], max(end, 2 * t.shape[1])), -1, dtype=np.int32)
            wider[:, :t.shape[1]] = t
            self._table_np[group] = t = wider
        t[slot, first:end] = pages

    def block_table_array(self, group: int, rcs: Sequence[RequestCache], width: int) -> np.ndarray:
        """[len(rcs), width] int32: logical page -> page id (-1 where none is held)."""
        t = self._table_np[group]
        if not rcs:
            return np.full((1, width), -1, dtype=np.int32)
        slots = np.fromiter((rc.slot for rc in rcs), dtype=np.intp, count=len(rcs))
        if width <= t.shape[1]:
            out = t[slots, :width]
        else:
            out = np.full((len(rcs), width), -1, dtype=np.int32)
            out[:, :t.shape[1]] = t[slots]
        for rc in rcs:
            if len(rc.tables[group]) > width:
                raise ValueError(f"request {rc.rid!r} holds {len(rc.tables[group])} pages, table width is {width}")
        return out

    # ---- invariants (used by tests and debug runs) -----------------------------------------
    def check(self) -> None:
        for g, alloc in enumerate(self.allocators):
            held = set()
            for rc in self.requests.values():
                for p in rc.tables[g]:
                    if p < 0:
                        continue
                    if p in held:
                        raise AssertionError(f"group {g}: page {p} is held twice")
                    held.add(p)
            if held != set(alloc.held_pages()):
                raise AssertionError(f"group {g}: pages lost or leaked "
                                     f"(tables {sorted(held)} vs allocator {alloc.held_pages()})")
            if len(held) + alloc.num_free != alloc.num_pages:
                raise AssertionError(f"group {g}: {len(held)} held + {alloc.num_free} free != {alloc.num_pages}")
            if len(set(alloc._free)) != len(alloc._free):
                raise AssertionError(f"group {g}: a page is on the free list twice")
        for g in range(len(self.groups)):
            for rc in self.requests.values():
                row = self._table_np[g][rc.slot]
                t = rc.tables[g]
                if list(row[:len(t)]) != list(t) or (row[len(t):] != -1).any():
                    raise AssertionError(f"group {g}: the table copy of request {rc.rid!r} is out of date")
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise AssertionError("a state slot was lost")
