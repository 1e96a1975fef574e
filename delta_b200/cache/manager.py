"""The cache manager: pages of keys and values with a block table per request,
in groups, and slots of fixed-size state per request.

Reference counterparts: ``KVCache`` (one buffer [pages, 2, 16, heads, head_dim] per
layer, DELTA/Engine/DELTA/model.py:99-127), ``PageManager`` and
``Request.plan/initialize_pages`` (scheduler.py:8-40, 60-74), the slot block table
(backend.py:1835-1848) and the slot-indexed arrays ``cachelens`` and the selected
pages (backend.py:263, page_selector_v2.py:62-63).

What differs, on purpose:
  * Layers are sorted into groups by what they keep per token (the layout of a
    page, which the mixer declares, and the window).  A group has a pool and block tables of its own; all layers
    of a group share a request's page ids.  A group with a window gives pages back
    as soon as the window has passed them; the others when the request ends.
  * A request holds ceil(len / page_size) pages: no empty page in advance
    (the reference allocates one whenever the length reaches a page's end,
    scheduler.py:60-66).
  * Growing a request is all or nothing over the groups; ``OutOfPages`` leaves
    everything as it was, and the scheduler decides what happens then.
  * What a page holds is the mixer's business: the manager allocates
    [layers of the group][page][*layout] from the layout the mixer declares.  The
    attention part keeps [K|V][kv head][offset][head_dim], so that the keys of one
    (page, head) are one contiguous tile.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from ..parts.base import CacheSpec, StateSpec
from .page_pool import OutOfPages, PagePool


@dataclass
class LayerCacheView:
    """What a mixer gets for one run: its layer's pages and the block table of its group
    for the rows of this step."""
    pages: torch.Tensor         # [num_pages, *page layout]: the pages of this layer
    block_table: torch.Tensor   # [rows, max_pages] int32 (device), -1 where no page is held
    page_size: int
    writes: bool
    window: Optional[int]
    group: str


class CacheGroup:
    def __init__(self, name: str, spec: CacheSpec, cache_ids: List[int], num_pages: int, page_size: int,
                 max_slots: int, max_pages_per_request: int, dtype, device, shuffle_seed=None, page_runs=True):
        self.name, self.spec, self.cache_ids = name, spec, list(cache_ids)
        self.page_size = page_size
        self.pool = PagePool(num_pages, shuffle_seed, run_pages=max(1, spec.run_tokens // page_size) if page_runs else 1)
        self.index_of = {cid: i for i, cid in enumerate(self.cache_ids)}
        # one page more than the pool hands out: the spare page that the padding slot points at
        self.pages = torch.zeros((len(self.cache_ids), num_pages + 1, *spec.page_shape(page_size)), dtype=dtype, device=device)
        self.spare_page = num_pages
        # host block tables; -1 = no page.  first_page[slot]: pages below it were given back.
        # Row max_slots is the padding slot: one logical page, the spare one, for ever.
        self.table = np.full((max_slots + 1, max_pages_per_request), -1, dtype=np.int32)
        self.first_page = np.zeros(max_slots + 1, dtype=np.int64)
        self.num_logical = np.zeros(max_slots + 1, dtype=np.int64)  # logical pages ever reached
        self.table[max_slots, 0] = self.spare_page
        self.num_logical[max_slots] = 1

    def pages_needed(self, slot: int, new_len: int) -> int:
        want = (new_len + self.page_size - 1) // self.page_size
        return max(0, want - int(self.num_logical[slot]))

    def held(self, slot: int) -> List[int]:
        row = self.table[slot, int(self.first_page[slot]):int(self.num_logical[slot])]
        return [int(p) for p in row if p >= 0]


class CacheManager:
    """Owns every cache group and every state slot.  ``device`` may be "cpu" for tests of
    the bookkeeping; kernels only ever see CUDA tensors.

    Beside the ``max_slots`` slots that requests get there is one padding slot
    (``padding_slot``), which no request ever holds: it has a row in every block table
    with one page, a spare page outside the pool, and a row in every state.  A decode step
    captured for a rounded-up batch size points its spare rows at it (position 0), so that
    they read and write nothing that belongs to a request."""

    def __init__(self, cache_specs: Dict[int, CacheSpec], state_specs: Dict[str, StateSpec], *, max_slots: int,
                 max_seq_len: int, page_size: int, num_pages, dtype=torch.bfloat16, device="cuda", shuffle_seed=None,
                 page_runs: bool = True):
        self.max_slots, self.max_seq_len, self.page_size = int(max_slots), int(max_seq_len), int(page_size)
        self.max_pages_per_request = (self.max_seq_len + page_size - 1) // page_size
        self.device = device
        by_spec: Dict[CacheSpec, List[int]] = {}
        for cid, spec in sorted(cache_specs.items()):
            by_spec.setdefault(spec, []).append(cid)
        self.groups: Dict[str, CacheGroup] = {}
        self.group_of_cache: Dict[int, CacheGroup] = {}
        for spec, cids in by_spec.items():
            name = spec.describe()
            n = num_pages[name] if isinstance(num_pages, dict) else int(num_pages)
            g = CacheGroup(name, spec, cids, n, page_size, self.max_slots, self.max_pages_per_request, dtype, device, shuffle_seed,
                           page_runs)
            self.groups[name] = g
            for cid in cids:
                self.group_of_cache[cid] = g
        self.state_specs = dict(state_specs)
        self.states: Dict[str, torch.Tensor] = {
            k: torch.full((self.max_slots + 1, *s.shape), s.fill, dtype=s.dtype, device=device) for k, s in state_specs.items()}
        self.padding_slot = self.max_slots
        self.seq_len = np.zeros(self.max_slots, dtype=np.int64)
        self._free_slots = list(range(self.max_slots - 1, -1, -1))
        self._live = [False] * self.max_slots

    # ---- slots -------------------------------------------------------------
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def acquire_slot(self) -> int:
        """A free request slot with empty block tables and its state reset."""
        if not self._free_slots:
            raise RuntimeError("no free request slot")
        slot = self._free_slots.pop()
        self._live[slot] = True
        self.seq_len[slot] = 0
        for g in self.groups.values():
            g.table[slot].fill(-1)
            g.first_page[slot] = 0
            g.num_logical[slot] = 0
        for k, s in self.state_specs.items():
            self.states[k][slot] = s.fill
        return slot

    def release_slot(self, slot: int) -> None:
        """Gives back every page the request holds, and the slot."""
        if not self._live[slot]:
            raise ValueError(f"slot {slot} is released twice (or was never acquired)")
        for g in self.groups.values():
            g.pool.free(g.held(slot))
            g.table[slot].fill(-1)
            g.first_page[slot] = 0
            g.num_logical[slot] = 0
        self.seq_len[slot] = 0
        self._live[slot] = False
        self._free_slots.append(slot)

    def is_live(self, slot: int) -> bool:
        return self._live[slot]

    # ---- pages ---------------------------------------------------------------
    def pages_needed(self, slot: int, new_len: int) -> Dict[str, int]:
        return {n: g.pages_needed(slot, new_len) for n, g in self.groups.items()}

    def can_grow(self, slot: int, new_len: int, reserve: Optional[Dict[str, int]] = None) -> bool:
        """True when every group can give the pages that ``new_len`` tokens need, on top of
        ``reserve`` pages per group that are already spoken for in this step."""
        if new_len > self.max_seq_len:
            return False
        for n, g in self.groups.items():
            if g.pages_needed(slot, new_len) + (reserve or {}).get(n, 0) > g.pool.free_pages:
                return False
        return True

    def grow(self, slot: int, new_len: int) -> None:
        """Makes room for the request to hold ``new_len`` tokens.  All groups or none."""
        if not self._live[slot]:
            raise ValueError(f"slot {slot} is not live")
        if new_len > self.max_seq_len:
            raise OutOfPages(f"a request of {new_len} tokens is above the limit of {self.max_seq_len}")
        need = self.pages_needed(slot, new_len)
        for n, g in self.groups.items():
            if need[n] > g.pool.free_pages:
                raise OutOfPages(f"out of cache pages in group {n}: {need[n]} needed, {g.pool.free_pages} free")
        for n, g in self.groups.items():
            if need[n]:
                a = int(g.num_logical[slot])
                last = int(g.table[slot, a - 1]) if a > 0 else -1
                pages = g.pool.alloc(need[n], after=last if last >= 0 else None)
                g.table[slot, a:a + need[n]] = pages
                g.num_logical[slot] = a + need[n]

    def advance(self, slot: int, new_len: int) -> None:
        """Records that the request now holds ``new_len`` tokens, and gives back the pages
        that every later query's window has passed."""
        self.seq_len[slot] = new_len
        for g in self.groups.values():
            w = g.spec.window
            if not w:
                continue
            # the next query sits at position >= new_len and reads keys > new_len - w
            first_needed = max(0, new_len - w + 1) // g.page_size
            a = int(g.first_page[slot])
            if first_needed > a:
                row = g.table[slot, a:first_needed]
                g.pool.free([int(p) for p in row if p >= 0])
                g.table[slot, a:first_needed] = -1
                g.first_page[slot] = first_needed

    # ---- views for a step ------------------------------------------------------
    def layer_pages(self, cache_id: int) -> torch.Tensor:
        g = self.group_of_cache[cache_id]
        return g.pages[g.index_of[cache_id]]

    def check(self) -> None:
        """Bookkeeping invariants: every held page belongs to exactly one live request."""
        for g in self.groups.values():
            g.pool.check()
            seen = set()
            for slot in range(self.max_slots):
                pages = g.held(slot)
                if pages and not self._live[slot]:
                    raise AssertionError(f"slot {slot} is free but holds pages in group {g.name}")
                for p in pages:
                    if p in seen:
                        raise AssertionError(f"page {p} of group {g.name} is held twice")
                    seen.add(p)
            if len(seen) != g.pool.held_pages:
                raise AssertionError(f"group {g.name}: {g.pool.held_pages} pages are out, requests hold {len(seen)}")

    def pages_in_use(self) -> Dict[str, int]:
        return {n: g.pool.held_pages for n, g in self.groups.items()}
