"""Host-side bookkeeping of cache pages: a pool with reference counts and a LIFO free list.

The behaviour follows the reference pool (src/model/kv_cache.cpp:10-69): a fixed number of pages,
page 0 handed out first, a freed page is the next one handed out (so stale contents are met early
in tests), and a page returns to the free list when its last reference is dropped. The memory
itself lives on the device and is owned by the engine; this class only counts.
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """No free page is left in a pool."""


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise ValueError("PagePool: n_pages must be >= 1")
        self.n_pages = n_pages
        self._refs: List[int] = [0] * n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))   # pop() gives page 0 first

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free cache page")
        p = self._free.pop()
        self._refs[p] = 1
        return p

    def retain(self, page: int) -> None:
        self._check_held(page, "retain")
        self._refs[page] += 1

    def release(self, page: int) -> None:
        self._check_held(page, "release")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def ref_count(self, page: int) -> int:
        if not (0 <= page < self.n_pages):
            raise IndexError(f"PagePool: bad page id {page}")
        return self._refs[page]

    def _check_held(self, page: int, what: str) -> None:
        if not (0 <= page < self.n_pages) or self._refs[page] < 1:
            raise RuntimeError(f"PagePool.{what}: page {page} is not allocated")

    def check_invariants(self) -> None:
        """Every page is either free exactly once or referenced; raises AssertionError otherwise."""
        assert len(set(self._free)) == len(self._free), "a page is on the free list twice"
        for p in range(self.n_pages):
            free = p in self._free_set()
            assert free == (self._refs[p] == 0), f"page {p}: refs {self._refs[p]} but free={free}"

    def _free_set(self):
        return set(self._free)
