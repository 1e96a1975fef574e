"""The attention part's choice of kernels for a batch.

bfloat16 with head size 64 or 128: rows that bring one token go to the split-key decode
kernel (at most 16 query heads per key-value head), rows that bring more go to a tiled
prefill kernel (tcgen05 with 128-query tiles when a row brings at least 32 tokens, else
warp-level MMA with 64-query tiles); a mixed step launches both, each skipping the other's
rows.  Everything else (32 bit, other head sizes) goes to the plain kernel, which takes
every size.

In a replayable step (``ctx.replayable``) nothing is chosen from the step's host data: the
grid is the one for the longest request the engine allows, and whether pages are looked for
in runs follows from how the pool hands pages out, not from this step's block tables.
"""
from __future__ import annotations

import functools
import os

import torch

from ..kernels import ops

_NO_RUNS = os.environ.get("DELTA_B200_DECODE_NO_TMA") == "1"   # for measurements: never look for runs of pages
_NO_CLUSTER = os.environ.get("DELTA_B200_DECODE_NO_CLUSTER") == "1"   # for measurements: splits always merged by the second kernel
# The most splits of a (row, key-value head) that are launched as one thread-block cluster, which merges them itself.
# Measured on the decode step (Yi-6B shape, context 4,096): 4 splits (batch 16) 3.89 -> 3.78 ms, 2 splits (batch 32)
# 4.34 -> 4.30 ms, 5 splits (batch 14) 3.76 -> 3.72 ms; 8 splits (batch 8) no gain, and 6 to 8 splits at batches 9 to
# 12 lose half a millisecond, because fewer of the larger clusters fit on the device at once than blocks do.
CLUSTER_SPLITS = int(os.environ.get("DELTA_B200_CLUSTER_SPLITS", "5"))
DECODE_TILE = 64
MAX_SPLITS = int(os.environ.get("DELTA_B200_MAX_SPLITS", "64"))
TMA_MIN_TILES = int(os.environ.get("DELTA_B200_TMA_MIN_TILES", "16"))    # tiles a block must walk for the decode kernel's TMA variant to be taken
TC_PREFILL_MIN_TOKENS = 32   # below this a 128-query tile of the tcgen05 kernel is mostly padding
PARTIALS = "attention.decode_partials"


def decode_splits(rows: int, kv_heads: int, max_keys: int, sm_count: int, blocks_per_sm: int) -> int:
    """Blocks per (row, key-value head): as many as run at once (a second, partly filled
    wave would double the time), and so few that a block has two 64-key tiles at the longest context (one
    request at 4,096 keys: 64 blocks of one tile each 2.914 ms a step, 32 blocks of two 2.877 ms; at
    32,768 keys 64 blocks of eight tiles beat 32 of sixteen, 3.276 against 3.345 ms)."""
    want = (max(1, blocks_per_sm) * sm_count) // max(1, rows * kv_heads)
    tiles = max(1, -(-max_keys // DECODE_TILE))
    return max(1, min(want, max(1, tiles // 2), MAX_SPLITS))


@functools.lru_cache(maxsize=None)
def _partials_bound(max_rows: int, H: int, KV: int, hd: int, max_keys: int, sm_count: int, per_sm: int) -> int:
    """The most floats of split partials any decode step of up to ``max_rows`` rows can ask for."""
    return max(ops.attention_decode_scratch_floats(b, H, hd, decode_splits(b, KV, max_keys, sm_count, per_sm))
               for b in range(1, max_rows + 1))


def plain(ctx) -> bool:
    return "attention" in ctx.plain_kernels or ctx.dtype != torch.bfloat16


def can_fuse_rope_append(ctx, H: int, KV: int, hd: int, ps: int, interleaved: bool) -> bool:
    """True when the step goes to the decode kernel, which can then rotate q and k and append the
    new token's k and v itself; the separate rotary/append kernel is left out."""
    return (ctx.decode_only and not plain(ctx) and not interleaved and ops.attention_decode_supported(ctx.dtype, H, KV, hd, ps))


def _pages_scattered(ctx, group: str) -> bool:
    """True when fewer than half of the rows' pages follow their predecessor in the pool: the decode
    kernel then does not look for runs of pages to fetch with one copy.  A replayable step asks how
    the pool hands pages out instead of looking at this step's tables."""
    g = ctx.cache.groups[group]
    if ctx.replayable:
        return g.pool.shuffled

    def look():
        t = g.table[[r.slot for r in ctx.host["rows"]]]
        held = t[:, 1:] >= 0
        n = int(held.sum())
        return n > 0 and int(((t[:, 1:] - t[:, :-1] == 1) & held).sum()) * 2 < n
    return ctx.memo(("pages scattered", group), look)     # the same for every layer of the group in this step


def _decode(ctx, params, row_filter: int, group: str) -> None:
    longest = ctx.cache.max_seq_len if ctx.replayable else ctx.max_seq_len
    max_keys = longest if not params.window else min(longest, params.window + params.ps)
    rows = ctx.num_rows
    # blocks per SM depend on the page ids a block keeps in shared memory, which depend on the splits:
    # ask for the occupancy without them, split, and ask again with what a block then holds
    per_sm = ops.attention_decode_blocks_per_sm(params.H, params.KV, params.hd, 0)
    splits = decode_splits(rows, params.KV, max_keys, ctx.sm_count, per_sm)
    tile_pages = max(1, DECODE_TILE // params.ps)           # a block's share is a whole number of tiles
    held = ops.attention_decode_blocks_per_sm(params.H, params.KV, params.hd, -(-(-(-params.max_pages // splits)) // tile_pages) * tile_pages)
    if held < per_sm:
        per_sm = held
        splits = decode_splits(rows, params.KV, max_keys, ctx.sm_count, per_sm)
    # A few splits are launched as one cluster that merges them over distributed shared memory: no partial
    # results in global memory, no second kernel.
    cluster = 2 <= splits <= CLUSTER_SPLITS and not _NO_CLUSTER
    if cluster:    # only when all clusters run at once: a second wave would cost more than the merge kernel
        entries = -(-(-(-params.max_pages // splits)) // tile_pages) * tile_pages
        cluster = rows * params.KV <= ops.attention_decode_max_clusters(params.H, params.KV, params.hd, entries, splits)
    params.splits = splits
    params.row_filter = row_filter
    # The variant that fetches runs of pages by TMA pays for finding the runs at the start of a block:
    # it wins when a block walks many tiles (batch 64 at 4,096 keys: 111 -> 85 us) and loses a little
    # when it walks few (batch 8 at 4,096 keys with 9 splits, 7 tiles a block: +1.6 % on the step).
    long_blocks = -(-max_keys // (DECODE_TILE * splits)) >= TMA_MIN_TILES
    params.reserved = (0 if (long_blocks and not _NO_RUNS and not _pages_scattered(ctx, group)) else 1) | (2 if cluster else 0)
    if splits > 1 and not cluster:
        n = ops.attention_decode_scratch_floats(rows, params.H, params.hd, splits)
        bound = _partials_bound(max(ctx.max_rows, rows), params.H, params.KV, params.hd, ctx.cache.max_seq_len, ctx.sm_count, per_sm)
        params.scratch = ctx.scratch(PARTIALS, (n,), torch.float32, bound=(bound,)).data_ptr()
    ops.attention_decode(params)


def _prefill_kernel(ctx, params):
    """The kernel for rows that bring several tokens: tcgen05 when some row brings enough of them
    and the sizes fit it, else warp-level MMA; None when neither takes the sizes."""
    tc = ops.attention_prefill_tc_supported(ctx.dtype, params.H, params.KV, params.hd, params.ps, params.q_stride)
    mma = ops.attention_prefill_supported(ctx.dtype, params.H, params.KV, params.hd, params.ps)
    if tc and (ctx.max_q_len >= TC_PREFILL_MIN_TOKENS or not mma):
        return ops.attention_prefill_tc
    return ops.attention_prefill if mma else None


def run(ctx, params, group: str) -> None:
    """Runs paged attention with the kernels that fit the batch.  ``group`` names the cache group
    of the layer (its block tables tell whether pages lie in runs)."""
    if plain(ctx):
        ops.attention_plain(params)
        return
    dec_ok = ops.attention_decode_supported(ctx.dtype, params.H, params.KV, params.hd, params.ps)
    prefill = _prefill_kernel(ctx, params)
    if ctx.decode_only:
        if dec_ok:
            _decode(ctx, params, 0, group)
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
        _decode(ctx, params, 1, group)
        params.row_filter = 2
        prefill(params, ctx.max_q_len)
    elif params.sel_pages is None and params.dump is None:
        params.row_filter = 0
        prefill(params, ctx.max_q_len)
    else:
        ops.attention_plain(params)
