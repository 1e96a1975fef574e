"""Chooses the attention kernel for a batch.

Steps in which every row brings one token go to the split-key decode kernel when it
takes the sizes (bfloat16, head size 64 or 128, at most 16 query heads per key-value
head); everything else goes to the plain kernel, which takes every size.
"""
from __future__ import annotations

import torch

from ..kernels import ops

SM_COUNT = 148
DECODE_TILE = 64
MAX_SPLITS = 64
BLOCKS_PER_SM = 2     # the decode kernel's registers and shared memory let two blocks share an SM


def decode_splits(rows: int, kv_heads: int, max_keys: int) -> int:
    """Blocks per (row, key-value head): as many as run at once (a second, partly filled
    wave would double the time), no more than there are 64-key tiles."""
    want = (BLOCKS_PER_SM * SM_COUNT) // max(1, rows * kv_heads)
    tiles = max(1, -(-max_keys // DECODE_TILE))
    return max(1, min(want, tiles, MAX_SPLITS))


def run(ctx, params) -> None:
    if (ctx.decode_only and not ctx.plain_attention
            and ops.attention_decode_supported(ctx.dtype, params.H, params.KV, params.hd, params.ps)):
        max_keys = ctx.max_seq_len if not params.window else min(ctx.max_seq_len, params.window + params.ps)
        if params.sel_pages is not None and not params.dump:
            pass  # chosen pages bound the keys too, but rows that read everything may share the step
        splits = ctx.fixed_decode_splits or decode_splits(ctx.num_rows, params.KV, max_keys)
        params.splits = splits
        if splits > 1:
            n = ops.attention_decode_scratch_floats(ctx.num_rows, params.H, params.hd, splits)
            scratch = ctx.scratch("attention.decode_partials", (n,), torch.float32)
            params.scratch = scratch.data_ptr()
        ops.attention_decode(params)
        return
    ops.attention_plain(params)
