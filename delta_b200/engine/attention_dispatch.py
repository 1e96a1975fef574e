"""Chooses the attention kernels for a batch.

bfloat16 with head size 64 or 128: rows that bring one token go to the split-key decode
kernel (at most 16 query heads per key-value head), rows that bring more go to a tiled
prefill kernel (tcgen05 with 128-query tiles when a row brings at least 32 tokens, else
warp-level MMA with 64-query tiles); a mixed step launches both, each skipping the other's
rows.  Everything else (32 bit, other head sizes) goes to the plain kernel, which takes
every size.
"""
from __future__ import annotations

import os

import torch

from ..kernels import ops

_NO_RUNS = os.environ.get("DELTA_B200_DECODE_NO_TMA") == "1"   # for measurements: never look for runs of pages
SM_COUNT = 148
DECODE_TILE = 64
MAX_SPLITS = 64
TMA_MIN_TILES = int(os.environ.get("DELTA_B200_TMA_MIN_TILES", "16"))    # tiles a block must walk for the decode kernel's TMA variant to be taken
BLOCKS_PER_SM = 2     # the decode kernel's registers and shared memory let two blocks share an SM


def decode_splits(rows: int, kv_heads: int, max_keys: int) -> int:
    """Blocks per (row, key-value head): as many as run at once (a second, partly filled
    wave would double the time), no more than there are 64-key tiles."""
    want = (BLOCKS_PER_SM * SM_COUNT) // max(1, rows * kv_heads)
    tiles = max(1, -(-max_keys // DECODE_TILE))
    return max(1, min(want, tiles, MAX_SPLITS))


def can_fuse_rope_append(ctx, H: int, KV: int, hd: int, ps: int, interleaved: bool) -> bool:
    """True when the step goes to the decode kernel, which can then rotate q and k and append the
    new token's k and v itself; the separate rotary/append kernel is left out."""
    return (ctx.decode_only and not ctx.plain_attention and ctx.dtype == torch.bfloat16 and not interleaved
            and ops.attention_decode_supported(ctx.dtype, H, KV, hd, ps))


def _pages_scattered(ctx, params) -> bool:
    """True when fewer than half of the rows' pages follow their predecessor in the pool: the decode
    kernel then does not look for runs of pages to fetch with one copy."""
    import numpy as np
    for g in ctx.cache.groups.values():
        if g.page_size != params.ps:
            continue
        slots = [r.slot for r in ctx.host["rows"]]
        t = g.table[slots]
        held = t[:, 1:] >= 0
        n = int(held.sum())
        return n > 0 and int(((t[:, 1:] - t[:, :-1] == 1) & held).sum()) * 2 < n
    return False


def _decode(ctx, params, row_filter: int) -> None:
    max_keys = ctx.max_seq_len if not params.window else min(ctx.max_seq_len, params.window + params.ps)
    splits = ctx.fixed_decode_splits or decode_splits(ctx.num_rows, params.KV, max_keys)
    params.splits = splits
    params.row_filter = row_filter
    # The variant that fetches runs of pages by TMA pays for finding the runs at the start of a block:
    # it wins when a block walks many tiles (batch 64 at 4,096 keys: 111 -> 85 us) and loses a little
    # when it walks few (batch 8 at 4,096 keys with 9 splits, 7 tiles a block: +1.6 % on the step).
    long_blocks = -(-max_keys // (DECODE_TILE * splits)) >= TMA_MIN_TILES
    params.reserved = 0 if (long_blocks and not _NO_RUNS and not _pages_scattered(ctx, params)) else 1
    if splits > 1:
        n = ops.attention_decode_scratch_floats(ctx.num_rows, params.H, params.hd, splits)
        params.scratch = ctx.scratch("attention.decode_partials", (n,), torch.float32).data_ptr()
    ops.attention_decode(params)


TC_PREFILL_MIN_TOKENS = 32   # below this a 128-query tile of the tcgen05 kernel is mostly padding


def _prefill_kernel(ctx, params):
    """The kernel for rows that bring several tokens: tcgen05 when some row brings enough of them
    and the sizes fit it, else warp-level MMA; None when neither takes the sizes."""
    tc = ops.attention_prefill_tc_supported(ctx.dtype, params.H, params.KV, params.hd, params.ps, params.q_stride)
    mma = ops.attention_prefill_supported(ctx.dtype, params.H, params.KV, params.hd, params.ps)
    if tc and (ctx.max_q_len >= TC_PREFILL_MIN_TOKENS or not mma):
        return ops.attention_prefill_tc
    return ops.attention_prefill if mma else None


def run(ctx, params) -> None:
    if ctx.plain_attention or ctx.dtype != torch.bfloat16:
        ops.attention_plain(params)
        return
    dec_ok = ops.attention_decode_supported(ctx.dtype, params.H, params.KV, params.hd, params.ps)
    prefill = _prefill_kernel(ctx, params)
    if ctx.decode_only:
        if dec_ok:
            _decode(ctx, params, 0)
        else:
            ops.attention_plain(params)
        return
    if prefill is None:
        ops.attention_plain(params)
        return
    singles = any(n == 1 for n in ctx.host["q_lens"])
    if not singles:
        params.row_filter = 0
        prefill(params, ctx.max_q_len)
    elif dec_ok:
        _decode(ctx, params, 1)
        params.row_filter = 2
        prefill(params, ctx.max_q_len)
    elif params.sel_pages is None and params.dump is None:
        params.row_filter = 0
        prefill(params, ctx.max_q_len)
    else:
        ops.attention_plain(params)
