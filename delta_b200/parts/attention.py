"""Grouped-query attention over the paged cache, with DELTA's three layer roles.

One projection gives q, k and v (rows of q_proj, k_proj, v_proj stacked, as the
reference's ``load_hook`` does, DELTA/Engine/DELTA/model.py:394-399); q and k
get their position encoding, k and v are appended to the layer's pages, and
every new token attends causally to the keys of its request
(model.py:437-492; backend.py:461-484).

``role`` (model.py:177-194):
  "full"     reads every key (or the last ``window`` of them);
  "planner"  as "full", and for decode rows it also scores the request's pages
             from this layer's attention and chooses ``subset_cache_size`` of them
             (backend.py:518-581, 787-853, 887-904; page_selector_v2.py:113-150);
  "subset"   decode rows read only the chosen pages (backend.py:486-516); before a
             planner has run in a step these are the most recent pages
             (backend.py:1871-1873).
``count_page_ahead`` counts a request's pages as the reference's scheduler does (one more, empty, once
the newest is exactly full); without it a request has the pages that hold its tokens.
Rows of a prompt always read everything; the planner and subset roles apply to rows
flagged ``ROW_DECODE`` (a single token at or after the prompt's end) of requests that hold
more pages than the subset.  Which kernels run is chosen in ``attention_kernels``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from . import attention_kernels, linear
from .base import MIXERS, PAGE, POSITION_ENCODINGS, ROW_DECODE, CacheSpec, Mixer, PartSpec, StateSpec, TensorSpec

SELECTED_PAGES = "delta.selected_pages"
SELECTED_COUNT = "delta.selected_count"


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
    def __init__(self, prefix: str, width: int, heads: int, kv_heads: int, head_dim: int,
                 position: Optional[PartSpec] = None, window: Optional[int] = None, role: str = "full",
                 subset_cache_size: int = 0, keep_last: int = 1, compression_ratio: float = 1.0,
                 position_bias: float = 1e-7, count_page_ahead: bool = False, scale: Optional[float] = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are no multiple of {kv_heads} key-value heads")
        if role not in ("full", "planner", "subset"):
            raise ValueError(f"unknown attention role '{role}'")
        if role != "full" and subset_cache_size < 1:
            raise ValueError("a planner or subset layer needs subset_cache_size >= 1")
        if role != "full" and window:
            raise ValueError("a windowed layer reads a bounded number of keys already; it takes no page selection")
        self.prefix = prefix
        self.width, self.heads, self.kv_heads, self.head_dim = int(width), int(heads), int(kv_heads), int(head_dim)
        self.window = int(window) if window else None
        self.role = role
        self.k = int(subset_cache_size)
        self.keep_last = int(keep_last)
        self.ratio = float(compression_ratio)
        self.bias = float(position_bias)
        # the reference's count of a request's pages: one more, empty, once the newest is exactly full
        # (DELTA/Engine/DELTA/scheduler.py:60-74); it takes a place among the chosen and is not read
        self.page_ahead = bool(count_page_ahead)
        if self.page_ahead and role != "full" and min(self.k, self.keep_last) < 2:
            raise ValueError("with count_page_ahead the empty page takes one of the newest L places: L and subset_cache_size "
                             "must be at least 2, or the page of the newest token would not be read")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = position.build(POSITION_ENCODINGS) if position is not None else None
        self.w_qkv = None
        self.w_o = None

    # ---- what it needs ---------------------------------------------------
    def tensor_specs(self):
        p, d, hd = self.prefix, self.width, self.head_dim
        return [TensorSpec(p + "q_proj.weight", (self.heads * hd, d)), TensorSpec(p + "k_proj.weight", (self.kv_heads * hd, d)),
                TensorSpec(p + "v_proj.weight", (self.kv_heads * hd, d)), TensorSpec(p + "o_proj.weight", (d, self.heads * hd))]

    def bind(self, tensors):
        p = self.prefix
        self.w_qkv = torch.cat([tensors[p + "q_proj.weight"], tensors[p + "k_proj.weight"], tensors[p + "v_proj.weight"]],
                               dim=0).contiguous()
        self.w_o = tensors[p + "o_proj.weight"]

    def cache_spec(self):
        # a page of a layer: [K|V][kv head][offset in the page][head_dim]
        # (the kernels fetch a tile of keys whose pages follow one another with one copy; the widest tile has 128 keys)
        return CacheSpec((2, self.kv_heads, PAGE, self.head_dim), self.window, run_tokens=128)

    def decode_rows_differ(self):
        return self.role != "full"

    def state_specs(self):
        if self.role == "full":
            return {}
        return {SELECTED_PAGES: StateSpec((self.k,), torch.int32, 0), SELECTED_COUNT: StateSpec((), torch.int32, -1)}

    # ---- a step ------------------------------------------------------------
    def begin_step(self, ctx):
        if self.role == "full" or not ctx.any_row_flag(ROW_DECODE) or not ctx.once("delta.recent_pages"):
            return
        ops.recent_pages(ctx.row_slot, ctx.row_flags, ctx.row_pos_start, ctx.row_q_len,
                         ctx.state(SELECTED_PAGES), ctx.state(SELECTED_COUNT), ctx.page_size, self.ratio, self.page_ahead)

    def forward(self, ctx, x, cache):
        H, KV, hd = self.heads, self.kv_heads, self.head_dim
        T = x.shape[0]
        qkv = linear.linear(ctx, x, self.w_qkv)
        table = self.position.table(x.device) if self.position is not None else None
        interleaved = bool(getattr(self.position, "interleaved", False))
        fuse = attention_kernels.can_fuse_rope_append(ctx, H, KV, hd, cache.page_size, interleaved)
        if not fuse:
            ops.rope_append(qkv, ctx.tok_pos, ctx.tok_row, cache.block_table, cache.pages if cache.writes else None, table,
                            H, KV, hd, cache.page_size, interleaved, err=ctx.err)
        out = torch.empty((T, H * hd), dtype=x.dtype, device=x.device)
        selective = self.role != "full" and ctx.any_row_flag(ROW_DECODE)
        dump = lse = None
        widest = ctx.cache.max_pages_per_request
        if self.role == "planner" and selective:
            dump = ctx.scratch("delta.dump", (ctx.num_rows, H, ctx.max_pages * cache.page_size), torch.float32,
                               bound=(ctx.max_rows, H, widest * cache.page_size))
            lse = ctx.scratch("delta.lse", (T, H), torch.float32, bound=(ctx.max_step_tokens, H))
        step = ctx.memo("attention.step_params", lambda: ops.attn_step_params(
            tok_row=ctx.tok_row, tok_pos=ctx.tok_pos, row_slot=ctx.row_slot, row_flags=ctx.row_flags, row_q_start=ctx.row_q_start,
            row_q_len=ctx.row_q_len, row_pos_start=ctx.row_pos_start, err=ctx.err))
        params = ops.make_attn_params(
            step=step, q=qkv, q_stride=qkv.shape[1], out=out, kv=cache.pages, block_table=cache.block_table,
            H=H, KV=KV, hd=hd, ps=cache.page_size, scale=self.scale,
            sel_pages=ctx.state(SELECTED_PAGES) if (self.role == "subset" and selective) else None,
            sel_count=ctx.state(SELECTED_COUNT) if (self.role == "subset" and selective) else None,
            dump=dump, lse=lse, window=self.window or 0,
            fuse=(2 if cache.writes else 1) if fuse else 0, rope_table=table if fuse else None)
        attention_kernels.run(ctx, params, cache.group)
        if self.role == "planner" and selective:
            scores = ctx.scratch("delta.page_scores", (ctx.num_rows, ctx.max_pages), torch.float32, bound=(ctx.max_rows, widest))
            ops.page_scores(dump, lse, ctx.row_flags, ctx.row_q_start, ctx.row_pos_start, ctx.row_q_len, scores,
                            cache.page_size, self.k, self.ratio, self.page_ahead)
            ops.select_pages(scores, ctx.row_slot, ctx.row_flags, ctx.row_pos_start, ctx.row_q_len,
                             ctx.state(SELECTED_PAGES), ctx.state(SELECTED_COUNT), self.keep_last, cache.page_size,
                             self.bias, self.ratio, self.page_ahead)
            if ctx.capture is not None:
                # for tests: what this planner chose, per (part, request slot, position)
                pages, counts = ctx.state(SELECTED_PAGES).cpu(), ctx.state(SELECTED_COUNT).cpu()
                planned = ctx.capture.setdefault("planned", {})
                for r in ctx.host["rows"]:
                    if (r.flags & ROW_DECODE) and int(counts[r.slot]) >= 0:
                        planned[(self.prefix, r.slot, r.start_pos)] = pages[r.slot, :int(counts[r.slot])].tolist()
        return linear.linear(ctx, out, self.w_o)
