"""Engine options: cache sizing, precision, DELTA's selective cache.

The reference passes these as keyword arguments of ``LMBackend``
(DELTA/Engine/DELTA/backend.py:29-48) and as attributes put on
``model.config`` by its scripts (tests/reasoni.py:327-335).  The names of the
selective-cache options are the reference's command-line names
(tests/reasoni.py:251-262).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


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

    def __post_init__(self):
        object.__setattr__(self, "full_cache_layers", tuple(sorted(set(int(i) for i in self.full_cache_layers))))
        if self.subset_cache_size < 1:
            raise ValueError("subset_cache_size must be at least 1")
        if self.L < 1:
            raise ValueError("L must be at least 1: the page that holds the newest token is always read")
        if self.compression_ratio < 1.0:
            raise ValueError("compression_ratio must be at least 1")

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


@dataclass(frozen=True)
class EngineConfig:
    """What the engine is built with.

    ``max_batch`` is the number of request slots (``--B``), ``max_seq_len`` the
    most tokens one request may hold (``--max_len``).  ``num_pages`` sizes the
    pool of every cache group; by default every slot can reach ``max_seq_len``
    (the reference's sizing, backend.py:253-254).
    """
    max_batch: int = 16
    max_seq_len: int = 2048
    page_size: int = 16
    num_pages: Optional[int] = None
    dtype: str = "bfloat16"            # "bfloat16" | "float32"
    max_tokens_per_step: int = 2048
    cuda_graph_decode: bool = False
    selective: Optional[SelectiveCacheConfig] = None
    rope_interleaved: bool = False
    seed: int = 123
    check_kernel_errors: bool = True   # read the kernels' error flag after every step
    shuffle_pages: Optional[int] = None  # seed: hand pages out in a shuffled order

    def __post_init__(self):
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got '{self.dtype}'")
        if self.page_size < 1 or self.page_size > 128 or (self.page_size & (self.page_size - 1)):
            raise ValueError(f"page_size must be a power of two of at most 128, got {self.page_size}")
        if self.max_batch < 1 or self.max_seq_len < 1 or self.max_tokens_per_step < 1:
            raise ValueError("max_batch, max_seq_len and max_tokens_per_step must be positive")

    @property
    def pages_per_request(self) -> int:
        return (self.max_seq_len + self.page_size - 1) // self.page_size

    @property
    def pool_pages(self) -> int:
        return self.num_pages if self.num_pages is not None else self.pages_per_request * self.max_batch
