"""What the parts see of one step: the batch on the device, the cache views and
the per-request state."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.manager import CacheManager, LayerCacheView


_SM_COUNT = {}     # device -> number of SMs (asked once)


class StepContext:
    """One batch of (request, its next tokens).

    Device tensors (int32): ``tokens`` [T]; ``tok_row`` [T] batch row of each token;
    ``tok_pos`` [T] position in its request; per batch row ``row_slot`` (request
    slot), ``row_flags`` (bits that parts interpret, ``parts.base.ROW_DECODE`` and
    whatever else a caller sets), ``row_q_start`` (first token of the row),
    ``row_q_len``, ``row_pos_start`` (tokens cached before this step); ``logit_rows``
    [R] token rows whose logits are wanted.  ``host`` holds the same as Python lists
    for parts that plan on the host.

    ``replayable``: the step is recorded once and replayed for later batches of the
    same number of rows, with only the contents of the device tensors above
    renewed.  A part must then choose nothing from the step's host data: no kernel,
    grid or buffer size may depend on ``host``; the bounds are the engine's limits
    (``cache.max_seq_len``, the full block-table width ``max_pages``).

    ``max_rows`` and ``max_step_tokens`` are the engine's limits on a step (rows of a
    batch, tokens of a scheduled step), for parts that size working memory once.

    ``plain_kernels``: names of kernel families ("products", "attention") for which
    the slow plain kernels are to be taken, for comparisons.
    """

    def __init__(self, *, device, dtype, cache: CacheManager, sections: Dict[str, torch.Tensor], block_tables,
                 host: dict, err: torch.Tensor, scratch_pool: dict, plain_kernels=frozenset(), replayable: bool = False,
                 capture: Optional[dict] = None, max_rows: int = 0, max_step_tokens: int = 0):
        self.device, self.dtype, self.cache = device, dtype, cache
        self.tokens = sections["tokens"]
        self.tok_row = sections["tok_row"]
        self.tok_pos = sections["tok_pos"]
        self.row_slot = sections["row_slot"]
        self.row_flags = sections["row_flags"]
        self.row_q_start = sections["row_q_start"]
        self.row_q_len = sections["row_q_len"]
        self.row_pos_start = sections["row_pos_start"]
        self.logit_rows = sections["logit_rows"]
        self.sampling_sections = {k: v for k, v in sections.items() if k.startswith("samp_")}
        self.block_tables = block_tables
        self.host = host
        self.num_tokens = int(self.tokens.shape[0])
        self.num_rows = int(self.row_slot.shape[0])
        self.max_pages = int(host["max_pages"])
        self.page_size = cache.page_size
        self.replayable = bool(replayable)
        self.max_rows = max(int(max_rows), self.num_rows)
        self.max_step_tokens = max(int(max_step_tokens), self.num_tokens)
        self.decode_only = bool(host["decode_only"])
        self.max_q_len = int(host["max_q_len"])
        self.max_seq_len = int(host["max_seq_len"])
        self.err = err
        self.plain_kernels = frozenset(plain_kernels)
        self.capture = capture
        self._scratch_pool = scratch_pool
        self._once = set()
        self._memo = {}

    def memo(self, key, make):
        """``make()`` the first time it is asked with this key in a step, its value from then on: for what every
        layer of a step would otherwise work out again from the same rows."""
        if key not in self._memo:
            self._memo[key] = make()
        return self._memo[key]

    def once(self, key: str) -> bool:
        """True the first time it is asked with this key in a step."""
        if key in self._once:
            return False
        self._once.add(key)
        return True

    def state(self, key: str) -> torch.Tensor:
        """The per-request state tensor [slots, ...] of this key."""
        return self.cache.states[key]

    def cache_view(self, cache_id: int, writes: bool) -> LayerCacheView:
        g = self.cache.group_of_cache[cache_id]
        return LayerCacheView(pages=self.cache.layer_pages(cache_id), block_table=self.block_tables[g.name],
                              page_size=g.page_size, writes=writes, window=g.spec.window, group=g.name)

    def any_row_flag(self, bit: int) -> bool:
        """True when some row of the step has this flag set; in a replayable step always
        (the rows of a later replay may have it, the kernels look at ``row_flags``)."""
        return self.replayable or self.memo(("row flag", bit), lambda: any(r.flags & bit for r in self.host["rows"]))

    @property
    def sm_count(self) -> int:
        n = _SM_COUNT.get(self.device)
        if n is None:
            n = _SM_COUNT[self.device] = torch.cuda.get_device_properties(self.device).multi_processor_count
        return n

    def scratch(self, key: str, shape, dtype, bound=None) -> torch.Tensor:
        """Working memory that lives across steps.  ``bound`` is the largest shape the part
        will ever ask for under the engine's limits; the buffer is made that large at once, so
        that its address never changes (a recorded step keeps raw addresses).  If a larger one
        is asked for all the same, the old buffer is kept alive beside the new one."""
        def count(sh):
            n = 1
            for s in sh:
                n *= int(s)
            return n
        n = count(shape)
        buf = self._scratch_pool.get(key)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            if buf is not None:
                self._scratch_pool.setdefault("__retired__", []).append(buf)
            buf = torch.empty(max(n, count(bound) if bound is not None else 0, 1), dtype=dtype, device=self.device)
            self._scratch_pool[key] = buf
        return buf[:n].view(*shape)
