"""A pool of fixed-size cache pages.

The reference's ``PageManager`` (DELTA/Engine/DELTA/scheduler.py:8-40) keeps a
shuffled free list, pops from its tail, reshuffles on every free and silently
ignores a page that is freed twice.  This pool hands pages out last-in
first-out (a page given back is the next one used again, which is what the
tests of page reuse want; pages given back together come out again in their
old order), can start from a seeded shuffle to scatter pages as
the reference does, and treats a double free or a foreign page as an error.
"""
from __future__ import annotations

import random
from typing import List, Optional


class OutOfPages(RuntimeError):
    """The pool cannot give as many pages as were asked for."""


class PagePool:
    def __init__(self, num_pages: int, shuffle_seed: Optional[int] = None):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        order = list(range(self.num_pages - 1, -1, -1))  # page 0 is handed out first
        self.shuffled = shuffle_seed is not None            # pages of a request lie scattered over the pool
        if shuffle_seed is not None:
            random.Random(shuffle_seed).shuffle(order)
        self._free: List[int] = order
        self._held = [False] * self.num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def held_pages(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> List[int]:
        """n pages, or ``OutOfPages`` with nothing taken."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"out of cache pages: {n} asked for, {len(self._free)} of {self.num_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def free(self, pages) -> None:
        """Gives pages back.  They go on the stack in reverse, so that pages freed together are
        handed out again in the order they had: a request's pages that followed one another in the
        pool still do for the next request, and the prefill kernel fetches such a run with one copy."""
        pages = list(pages)
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise ValueError(f"page {p} does not belong to this pool of {self.num_pages}")
            if not self._held[p]:
                raise ValueError(f"page {p} is freed twice (or was never handed out)")
            self._held[p] = False
        for p in reversed(pages):
            self._free.append(p)

    def check(self) -> None:
        """No page lost, none both free and held, none free twice."""
        if len(set(self._free)) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        for p in self._free:
            if self._held[p]:
                raise AssertionError(f"page {p} is free and held at once")
        if sum(self._held) + len(self._free) != self.num_pages:
            raise AssertionError("pages were lost")
