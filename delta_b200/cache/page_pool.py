"""A pool of fixed-size cache pages that hands them out in runs.

The reference's ``PageManager`` (DELTA/Engine/DELTA/scheduler.py:8-40) keeps a
shuffled free list, pops from its tail, reshuffles on every free and silently
ignores a page that is freed twice.  Here the order in which pages go out is
chosen for the attention kernels, which fetch pages that follow one another in
the pool with one copy: the pool is cut into aligned runs of ``run_pages``
pages, and a request that says which page it took last (``after``) gets

1. the page behind it, while that is in the same run and free;
2. else the first page of a run that is wholly free (the run given back last
   comes first, its pages in their order);
3. else, when no run is wholly free, a free page of a run that others have
   begun (the lowest one of the run that changed last).

So requests that grow by a page now and then, in turns, still hold runs, and a
request that takes many pages at once takes them in order.  Nothing is set
aside: a request holds the pages it asked for and no more, and every free page
can be had by whoever asks.  With ``run_pages = 1`` this is a last-in
first-out stack of pages.  A seeded shuffle scatters pages as the reference
does (then ``after`` is ignored).  A double free or a foreign page is an error.
"""
from __future__ import annotations

import random
from typing import Dict, List, Optional


class OutOfPages(RuntimeError):
    """The pool cannot give as many pages as were asked for."""


class PagePool:
    def __init__(self, num_pages: int, shuffle_seed: Optional[int] = None, run_pages: int = 1):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        if run_pages < 1:
            raise ValueError("a run has at least one page")
        self.num_pages = int(num_pages)
        self.shuffled = shuffle_seed is not None            # pages of a request lie scattered over the pool
        self.run_pages = 1 if self.shuffled else int(run_pages)
        self._held = [False] * self.num_pages
        self._n_free = self.num_pages
        n_runs = -(-self.num_pages // self.run_pages)
        self._free_in_run = [self._run_size(r) for r in range(n_runs)]
        order = list(range(n_runs - 1, -1, -1))             # run 0 is handed out first
        if shuffle_seed is not None:
            random.Random(shuffle_seed).shuffle(order)
        self._whole: List[int] = order                      # wholly free runs, a stack
        self._begun: Dict[int, None] = {}                   # runs with some pages out and some free, in order of their last change

    def _run_size(self, r: int) -> int:
        return min(self.run_pages, self.num_pages - r * self.run_pages)

    @property
    def free_pages(self) -> int:
        return self._n_free

    @property
    def held_pages(self) -> int:
        return self.num_pages - self._n_free

    def _take(self, p: int) -> None:
        r = p // self.run_pages
        self._held[p] = True
        self._n_free -= 1
        self._free_in_run[r] -= 1
        self._begun.pop(r, None)
        if self._free_in_run[r] > 0:
            self._begun[r] = None

    def alloc(self, n: int, after: Optional[int] = None) -> List[int]:
        """n pages, or ``OutOfPages`` with nothing taken.  ``after``: the page the asking
        request took last, so that the new ones continue its run where they can."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > self._n_free:
            raise OutOfPages(f"out of cache pages: {n} asked for, {self._n_free} of {self.num_pages} free")
        out: List[int] = []
        R = self.run_pages
        last = after if (after is not None and not self.shuffled and 0 <= after < self.num_pages) else None
        for _ in range(n):
            nxt = last + 1 if last is not None else None
            if nxt is not None and nxt % R != 0 and nxt < self.num_pages and not self._held[nxt]:
                p = nxt
            elif self._whole:
                p = self._whole.pop() * R
            else:
                r = next(reversed(self._begun))
                p = next(q for q in range(r * R, r * R + self._run_size(r)) if not self._held[q])
            self._take(p)
            out.append(p)
            last = p
        return out

    def free(self, pages) -> None:
        """Gives pages back.  Runs that become wholly free go on the stack in reverse, so that
        runs freed together are handed out again in the order they had."""
        pages = list(pages)
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise ValueError(f"page {p} does not belong to this pool of {self.num_pages}")
            if not self._held[p]:
                raise ValueError(f"page {p} is freed twice (or was never handed out)")
            self._held[p] = False
        self._n_free += len(pages)
        whole = []
        for p in reversed(pages):
            r = p // self.run_pages
            self._free_in_run[r] += 1
            self._begun.pop(r, None)
            if self._free_in_run[r] == self._run_size(r):
                whole.append(r)
            else:
                self._begun[r] = None
        self._whole.extend(whole)

    def check(self) -> None:
        """No page lost, none both free and held, no run listed twice or in the wrong list."""
        if len(set(self._whole)) != len(self._whole):
            raise AssertionError("a run is on the free stack twice")
        if set(self._whole) & set(self._begun):
            raise AssertionError("a run is wholly free and begun at once")
        free = 0
        whole = set(self._whole)
        for r in range(len(self._free_in_run)):
            n = sum(1 for q in range(r * self.run_pages, r * self.run_pages + self._run_size(r)) if not self._held[q])
            free += n
            if n != self._free_in_run[r]:
                raise AssertionError(f"run {r}: {n} pages are free, the count says {self._free_in_run[r]}")
            if (n == self._run_size(r)) != (r in whole):
                raise AssertionError(f"run {r} with {n} free pages is {'not ' if r not in whole else ''}on the free stack")
            if (0 < n < self._run_size(r)) != (r in self._begun):
                raise AssertionError(f"run {r} with {n} free pages is {'not ' if r not in self._begun else ''}among the begun runs")
        if free != self._n_free or sum(self._held) + free != self.num_pages:
            raise AssertionError("pages were lost")
