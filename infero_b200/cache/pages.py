"""Page bookkeeping on the host: who holds which page of a group's pool.

The reference's pool hands out one-token "slots" from a stack and keeps per-sequence slot
lists with a device-side table (crates/model/src/cache.rs:100-249, :320-339, :567-594).
Here a page holds ``page_size`` consecutive tokens of one request in every layer of one
group; allocation is all-or-nothing per call and every page is either free or held by
exactly one request.
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """The pool of a group cannot supply the pages asked for.  Nothing was taken."""

    def __init__(self, group: int, wanted: int, free: int):
        super().__init__(f"cache group {group}: {wanted} pages wanted, {free} free")
        self.group, self.wanted, self.free = group, wanted, free


class PageAllocator:
    def __init__(self, num_pages: int, group: int = 0):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self.group = group
        # stack with the lowest page on top, so the first request gets page 0 upward
        # (the reference fills its free list the same way, cache.rs:193-195)
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = bytearray(num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("negative page count")
        if n > len(self._free):
            raise OutOfPages(self.group, n, len(self._free))
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._held[p]:
                raise AssertionError(f"page {p} handed out while held")
            self._held[p] = 1
        return out

    def free(self, pages) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages) or not self._held[p]:
                raise AssertionError(f"page {p} freed but not held (group {self.group})")
            self._held[p] = 0
            self._free.append(p)

    def held_pages(self) -> List[int]:
        return [p for p in range(self.num_pages) if self._held[p]]
