"""Host bookkeeping of cache pages: a pool with a free list, and per-request block tables.

A page is ``page_size`` consecutive positions of every layer of one group.  The row of
position ``p`` is ``table[p // page_size] * page_size + p % page_size`` - nothing else
computes a cache row (crates/shiso-engine/src/kv.rs:10-16; crates/shiso-core/src/page.rs:60-65).
The pool hands out the page that has been free longest (a FIFO free list, as
crates/shiso-kvstore/src/pool.rs:93-184), counts holders per page so that sharing can
be added later, and treats giving back a page nobody holds as a bug.  A claim takes all
the pages it needs or none (crates/shiso-kvstore/src/page_table.rs:98-117).
"""

from __future__ import annotations

from collections import deque

import numpy as np


class OutOfPages(RuntimeError):
    """A claim needs more pages than the pool has free.  Nothing was taken."""

    def __init__(self, wanted: int, free: int, what: str = "pages"):
        self.wanted = wanted
        self.free = free
        super().__init__(f"cache pool: {wanted} {what} wanted, {free} free")


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free = deque(range(num_pages))
        self._holders = [0] * num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, count: int) -> list[int]:
        if count < 0:
            raise ValueError("cannot take a negative number of pages")
        if count > len(self._free):
            raise OutOfPages(count, len(self._free))
        pages = [self._free.popleft() for _ in range(count)]
        for p in pages:
            self._holders[p] = 1
        return pages

    def share(self, page: int) -> None:
        if self._holders[page] <= 0:
            raise RuntimeError(f"page {page} is free and cannot be shared")
        self._holders[page] += 1

    def give_back(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise RuntimeError(f"page {page} does not exist in a pool of {self.num_pages}")
        if self._holders[page] <= 0:
            raise RuntimeError(f"page {page} was given back twice")
        self._holders[page] -= 1
        if self._holders[page] == 0:
            self._free.append(page)

    def holders(self, page: int) -> int:
        return self._holders[page]

    def check(self) -> None:
        """Every page is either free exactly once or held; raises if one is lost."""
        free = list(self._free)
        if len(set(free)) != len(free):
            raise RuntimeError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (self._holders[p] == 0) != (p in self._free):
                raise RuntimeError(f"page {p}: {self._holders[p]} holders but free-list membership disagrees")


HOLE = -1  # a block-table entry whose page went back to the pool (the window passed it)


class BlockTable:
    """One request's pages in one group, in position order."""

    def __init__(self, page_size: int, window: int | None = None):
        self.page_size = page_size
        self.window = window
        self.pages: list[int] = []
        self.first_live = 0  # entries below this index are holes
        self._array = np.empty(16, dtype=np.int32)  # the same entries, ready to be copied into a step's table

    def pages_for(self, length: int) -> int:
        return -(-length // self.page_size)

    def missing_for(self, length: int) -> int:
        return max(0, self.pages_for(length) - len(self.pages))

    def grow(self, pool: PagePool, length: int) -> None:
        need = self.missing_for(length)
        if need:
            have = len(self.pages)
            self.pages.extend(pool.take(need))
            if len(self.pages) > len(self._array):
                bigger = np.empty(max(2 * len(self._array), len(self.pages)), dtype=np.int32)
                bigger[:have] = self._array[:have]
                self._array = bigger
            self._array[have : len(self.pages)] = self.pages[have:]

    def shrink(self, pool: PagePool, length: int) -> None:
        """Gives back the pages beyond those ``length`` positions need (a claim that was not used)."""
        keep = max(self.pages_for(length), self.first_live)
        while len(self.pages) > keep:
            pool.give_back(self.pages.pop())

    def release_passed(self, pool: PagePool, length: int) -> int:
        """Gives back pages that no later position can read: with a window ``w`` the
        query at position ``length`` (the next one) reads positions ``> length - w``."""
        if self.window is None:
            return 0
        first_needed = max(0, length + 1 - self.window)
        keep_from = first_needed // self.page_size
        released = 0
        while self.first_live < min(keep_from, len(self.pages)):
            pool.give_back(self.pages[self.first_live])
            self.pages[self.first_live] = HOLE
            self._array[self.first_live] = HOLE
            self.first_live += 1
            released += 1
        return released

    def release_all(self, pool: PagePool) -> None:
        for p in self.pages[self.first_live :]:
            pool.give_back(p)
        self.pages = []
        self.first_live = 0

    def as_array(self) -> np.ndarray:
        """The entries as int32 (a view; valid until the table grows)."""
        return self._array[: len(self.pages)]

    def live_pages(self) -> list[int]:
        return self.pages[self.first_live :]
