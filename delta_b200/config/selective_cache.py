"""DELTA's selective cache as an option of the Yi model specification.

The reference's scripts put these on ``model.config`` (tests/reasoni.py:327-335); the
names are its command-line names (tests/reasoni.py:251-262).  The generic engine does
not know them: they travel in ``EngineConfig.options["selective_cache"]`` to the
function that builds the model specification, which gives every attention layer its role.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SelectiveCacheConfig:
    """DELTA: which layers read the whole cache and how many pages the others read.

    ``full_cache_layers`` are layer indices (tests/reasoni.py:251).  A full
    layer followed by a non-full layer scores the pages and chooses
    ``subset_cache_size`` of them for the layers after it
    (DELTA/Engine/DELTA/model.py:177-194).  The last ``L`` pages are always
    chosen (page_selector_v2.py:120-123); ``L`` is clamped to
    ``subset_cache_size``.  A request uses the subset once
    pages / min(pages, subset_cache_size) > ``compression_ratio``
    (backend.py:1893-1897, decided per request here, per batch there).
    """
    full_cache_layers: tuple = ()
    subset_cache_size: int = 1024
    compression_ratio: float = 1.0
    L: int = 8
    position_bias: float = 1e-7
    # The reference takes a request's next page as soon as the newest is exactly full
    # (DELTA/Engine/DELTA/scheduler.py:60-74), so at one position in ``page size`` its selection counts
    # an empty page, which is always among the newest ``L`` and so takes one place of the subset.
    # False: a request has the pages that hold its tokens.  True: counted as the reference counts
    # them, for outputs that follow the reference's position by position.
    count_page_ahead: bool = False

    def __post_init__(self):
        object.__setattr__(self, "full_cache_layers", tuple(sorted(set(int(i) for i in self.full_cache_layers))))
        if self.subset_cache_size < 1:
            raise ValueError("subset_cache_size must be at least 1")
        if self.L < 1:
            raise ValueError("L must be at least 1: the page that holds the newest token is always read")
        if self.compression_ratio < 1.0:
            raise ValueError("compression_ratio must be at least 1")
        if self.count_page_ahead and min(self.L, self.subset_cache_size) < 2:
            raise ValueError("count_page_ahead needs L >= 2 and subset_cache_size >= 2: the empty page takes one place")

    @property
    def keep_last(self) -> int:
        return min(self.L, self.subset_cache_size)

    def role(self, layer: int, num_layers: int) -> str:
        """'full', 'planner' (full, and it chooses pages for what follows) or 'subset'."""
        if not self.full_cache_layers:
            return "full"
        if layer in self.full_cache_layers:
            next_full = (layer + 1) in self.full_cache_layers if layer + 1 < num_layers else True
            return "full" if next_full else "planner"
        return "subset"
