"""What the parts see of one step: the batch on the device, the cache views and
the per-request state."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.manager import CacheManager, LayerCacheView
from ..kernels import ops


class StepContext:
    """One batch of (request, its next tokens).

    Device tensors (int32): ``tokens`` [T]; ``tok_row`` [T] batch row of each token;
    ``tok_pos`` [T] position in its request; per batch row ``row_slot`` (request
    slot), ``row_flags`` (bit 0: a decode row that page selection applies to),
    ``row_q_start`` (first token of the row), ``row_q_len``, ``row_pos_start``
    (tokens cached before this step); ``logit_rows`` [R] token rows whose logits are
    wanted.  ``host`` holds the same as Python lists for parts that plan on the host.
    """

    def __init__(self, *, device, dtype, cache: CacheManager, sections: Dict[str, torch.Tensor], block_tables,
                 host: dict, err: torch.Tensor, scratch_pool: dict, plain_products=False, plain_attention=False,
                 capture: Optional[dict] = None):
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
        self.any_selective = bool(host["any_selective"])
        self.decode_only = bool(host["decode_only"])
        self.max_q_len = int(host["max_q_len"])
        self.max_seq_len = int(host["max_seq_len"])
        self.err = err
        self.plain_products = plain_products
        self.plain_attention = plain_attention
        self.capture = capture
        self.fixed_decode_splits = 0   # set by the decode graph: a captured launch keeps its grid
        self._scratch_pool = scratch_pool
        self._once = set()

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
        return LayerCacheView(kv=self.cache.layer_kv(cache_id), block_table=self.block_tables[g.name],
                              page_size=g.page_size, writes=writes, window=g.spec.window, group=g.name)

    def scratch(self, key: str, shape, dtype) -> torch.Tensor:
        """Working memory that lives across steps (so its address is stable) and grows on demand."""
        n = 1
        for s in shape:
            n *= int(s)
        buf = self._scratch_pool.get(key)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._scratch_pool[key] = buf
        return buf[:n].view(*shape)

    def can_fuse_rope_append(self, H, KV, hd, ps, interleaved) -> bool:
        from . import attention_dispatch
        return attention_dispatch.can_fuse_rope_append(self, H, KV, hd, ps, interleaved)

    def attention(self, params) -> None:
        """Runs paged attention with the kernel that fits the batch."""
        from . import attention_dispatch
        attention_dispatch.run(self, params)
