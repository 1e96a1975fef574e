"""Engine options: cache sizing, precision, limits of a step.

The reference passes these as keyword arguments of ``LMBackend``
(DELTA/Engine/DELTA/backend.py:29-48) and ``setup_caches`` (backend.py:247-256).
What belongs to one architecture (DELTA's selective cache, the pairing of rotary
positions) is not known here: it travels in ``options`` to the function that
builds that architecture's model specification.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional


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
    check_kernel_errors: bool = True   # read the kernels' error record with every step's result
    shuffle_pages: Optional[int] = None  # seed: hand pages out in a shuffled order
    page_runs: bool = True               # hand pages out in the runs a mixer asks for (False: one page at a time, last in first out)
    options: Mapping[str, Any] = field(default_factory=dict)   # for the architecture's specification builder

    def __post_init__(self):
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got '{self.dtype}'")
        if self.page_size < 1 or self.page_size > 128 or (self.page_size & (self.page_size - 1)):
            raise ValueError(f"page_size must be a power of two of at most 128, got {self.page_size}")
        if self.max_batch < 1 or self.max_seq_len < 1 or self.max_tokens_per_step < 1:
            raise ValueError("max_batch, max_seq_len and max_tokens_per_step must be positive")

    def option(self, name: str, default=None):
        """An architecture-specific option (None or ``default`` when it was not given)."""
        v = self.options.get(name)
        return default if v is None else v

    @property
    def pages_per_request(self) -> int:
        return (self.max_seq_len + self.page_size - 1) // self.page_size

    @property
    def pool_pages(self) -> int:
        return self.num_pages if self.num_pages is not None else self.pages_per_request * self.max_batch
