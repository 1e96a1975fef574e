"""Tensor-level entry points of the CUDA kernels.

Each function checks that its tensors are CUDA tensors of the expected type and
layout, and launches on torch's current stream.  Sizes that a kernel does not
take are refused with an error by the launcher itself; nothing is computed on
the CPU and no library model code is called.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import lib as _l
from .lib import AttnParams, KernelError

F32, BF16 = 0, 1


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"the kernels take float32 and bfloat16, not {dt}")


def _ptr(t: Optional[torch.Tensor], name: str, dtype=None):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{name} is on '{t.device}': the kernels run on CUDA tensors only and there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t.data_ptr()


def _stream():
    """The current stream's handle.  (``torch.cuda.current_stream().cuda_stream`` makes a Python object and looks up
    the device three times over: 15 us a launch, the largest part of the host's time in a step that is not replayed.)"""
    return _raw_stream(_current_device())


def _device_index() -> int:
    return _current_device() if _current_device is not None else torch.cuda.current_device()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)
if _raw_stream is None or _current_device is None:      # a torch without these entry points: the public, slower way
    def _stream():  # noqa: F811
        return torch.cuda.current_stream().cuda_stream


def launch_count() -> int:
    """Kernels launched through this module so far (library products included)."""
    return _l.LAUNCHES[0]


def count_launch(n: int = 1) -> None:
    _l.LAUNCHES[0] += n


def new_error_record(device) -> torch.Tensor:
    """Four ints the kernels write {code, a, b, c} into when they meet a bad index."""
    return torch.zeros(4, dtype=torch.int32, device=device)


_ERR_TEXT = {1: "page id out of range (token {0}, logical page {1}, page id {2})",
             2: "token id out of range (row {0}: id {1}, vocabulary {2})",
             3: "position out of range (token {0}: position {1}, limit {2})",
             4: "a wait inside a kernel ran out (block {0}, part {1}, {2} steps); its result was not stored"}


def error_text(code: int, a: int, b: int, c: int) -> str:
    return "a kernel met a bad index and skipped it: " + _ERR_TEXT.get(code, "code {3}").format(a, b, c, code)


def raise_if_error(err: torch.Tensor) -> None:
    """Reads the record (this waits for the device), clears it and raises when it is set."""
    code, a, b, c = err.tolist()
    if code != 0:
        err.zero_()
        raise KernelError(error_text(code, a, b, c))


def wait_check(err: torch.Tensor, limit_ms: float = 1.0) -> None:
    """Launches a kernel whose only wait, bounded by ``limit_ms`` (at most 10), can never be satisfied:
    it gives up, records it in ``err`` and returns.  For checking that path; nothing else uses it."""
    _l.check(_l.load().dk_wait_check(_ptr(err, "err", torch.int32), int(limit_ms * 1e6), _stream()), "wait_check")


# ---------------------------------------------------------------------------

def embedding(tokens, table, out, err=None):
    T, d = out.shape
    _l.check(_l.load().dk_embedding(_ptr(tokens, "tokens", torch.int32), _ptr(table, "table"), _ptr(out, "out", table.dtype),
                                    T, d, table.shape[0], dtype_code(table.dtype), _ptr(err, "err", torch.int32), _stream()),
             "embedding")
    return out


def rms_norm(x, weight, eps, out, add=None, rows=None, cast_first=False):
    """out[r] = rmsnorm(x[s]) * weight with s = rows[r] (or r); when ``add`` is
    given, x[s] += add[s] first, in place.  ``rows`` must not name a row twice
    together with ``add``."""
    n_rows = out.shape[0]
    d = x.shape[-1]
    if add is not None and add.dtype != x.dtype:
        raise KernelError("rms_norm: add and x differ in dtype")
    _l.check(_l.load().dk_rms_norm(_ptr(x, "x"), _ptr(add, "add"), _ptr(weight, "weight"), _ptr(out, "out", x.dtype),
                                   _ptr(rows, "rows", torch.int32), n_rows, d, float(eps), dtype_code(x.dtype),
                                   dtype_code(weight.dtype), int(bool(cast_first)), _stream()), "rms_norm")
    return out


def silu_mul(gate_up, out):
    T, I2 = gate_up.shape
    _l.check(_l.load().dk_silu_mul(_ptr(gate_up, "gate_up"), _ptr(out, "out", gate_up.dtype), T, I2 // 2,
                                   dtype_code(gate_up.dtype), _stream()), "silu_mul")
    return out


def rope_append(qkv, tok_pos, tok_row, block_table, kv, table, H, KV, hd, ps, interleaved, err=None):
    """Rotates q and k inside ``qkv`` [T, (H+2KV)*hd] and appends k, v to the pages
    of ``kv`` [pages, 2, KV, ps, hd].  ``table`` [positions, hd/2, 2] float holds
    cos and sin; None leaves q and k unrotated.  ``kv`` None appends nothing."""
    T = qkv.shape[0]
    if qkv.shape[1] != (H + 2 * KV) * hd:
        raise KernelError(f"rope_append: qkv has width {qkv.shape[1]}, expected {(H + 2 * KV) * hd}")
    if kv is not None and (tuple(kv.shape[1:]) != (2, KV, ps, hd) or kv.dtype != qkv.dtype):
        raise KernelError(f"rope_append: cache has shape {tuple(kv.shape)} / {kv.dtype}, expected [pages, 2, {KV}, {ps}, {hd}] of {qkv.dtype}")
    if table is not None and (table.dim() != 3 or table.shape[1] != hd // 2 or table.shape[2] != 2):
        raise KernelError(f"rope_append: table has shape {tuple(table.shape)}, expected [positions, {hd // 2}, 2]")
    _l.check(_l.load().dk_rope_append(
        _ptr(qkv, "qkv"), _ptr(tok_pos, "tok_pos", torch.int32), _ptr(tok_row, "tok_row", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1] if block_table is not None else 0,
        _ptr(kv, "kv"), kv.shape[0] if kv is not None else 0, _ptr(table, "table", torch.float32),
        table.shape[0] if table is not None else 0, T, H, KV, hd, ps, int(bool(interleaved)), dtype_code(qkv.dtype),
        _ptr(err, "err", torch.int32), _stream()), "rope_append")


def gemm_nt_plain(a, w, out):
    """out[M,N] = a[M,K] @ w[N,K]^T on the FMA units with float accumulation."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N) or a.dtype != w.dtype:
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} or dtypes do not fit")
    _l.check(_l.load().dk_gemm_nt_plain(_ptr(a, "a"), _ptr(w, "w"), _ptr(out, "out"), M, N, K, K, K, N,
                                        dtype_code(a.dtype), dtype_code(out.dtype), _stream()), "gemm_nt_plain")
    return out


def attn_step_params(*, tok_row, tok_pos, row_slot=None, row_flags=None, row_q_start=None, row_q_len=None, row_pos_start=None,
                     err=None) -> AttnParams:
    """The part of the attention kernels' parameters that is the same for every layer of a step (the step's
    tokens and rows): made once per step and handed to ``make_attn_params`` as ``step``."""
    p = AttnParams()
    i32 = torch.int32
    p.tok_row = _ptr(tok_row, "tok_row", i32)
    p.tok_pos = _ptr(tok_pos, "tok_pos", i32)
    p.row_slot = _ptr(row_slot, "row_slot", i32)
    p.row_flags = _ptr(row_flags, "row_flags", i32)
    p.row_q_start = _ptr(row_q_start, "row_q_start", i32)
    p.row_q_len = _ptr(row_q_len, "row_q_len", i32)
    p.row_pos_start = _ptr(row_pos_start, "row_pos_start", i32)
    p.err = _ptr(err, "err", i32)
    p.T = tok_row.shape[0]
    return p


def make_attn_params(*, q, q_stride, out, kv, block_table, tok_row=None, tok_pos=None, H, KV, hd, ps, scale, row_slot=None,
                     row_flags=None, row_q_start=None, row_q_len=None, row_pos_start=None, sel_pages=None,
                     sel_count=None, dump=None, lse=None, scratch=None, err=None, window=0, splits=0, row_filter=0,
                     fuse=0, rope_table=None, step: Optional[AttnParams] = None) -> AttnParams:
    i32 = torch.int32
    if step is not None:
        p = AttnParams.from_buffer_copy(step)
    else:
        p = AttnParams()
        p.tok_row = _ptr(tok_row, "tok_row", i32)
        p.tok_pos = _ptr(tok_pos, "tok_pos", i32)
        p.row_slot = _ptr(row_slot, "row_slot", i32)
        p.row_flags = _ptr(row_flags, "row_flags", i32)
        p.row_q_start = _ptr(row_q_start, "row_q_start", i32)
        p.row_q_len = _ptr(row_q_len, "row_q_len", i32)
        p.row_pos_start = _ptr(row_pos_start, "row_pos_start", i32)
        p.err = _ptr(err, "err", i32)
        p.T = tok_row.shape[0]
    p.q = _ptr(q, "q")
    p.out = _ptr(out, "out", q.dtype)
    p.kv = _ptr(kv, "kv", q.dtype)
    if tuple(kv.shape[1:]) != (2, KV, ps, hd):
        raise KernelError(f"attention: cache has shape {tuple(kv.shape)}, expected [pages, 2, {KV}, {ps}, {hd}]")
    p.block_table = _ptr(block_table, "block_table", i32)
    p.sel_pages = _ptr(sel_pages, "sel_pages", i32)
    p.sel_count = _ptr(sel_count, "sel_count", i32)
    p.dump = _ptr(dump, "dump", torch.float32)
    p.lse = _ptr(lse, "lse", torch.float32)
    p.scratch = _ptr(scratch, "scratch")
    p.rows = block_table.shape[0]
    p.H, p.KV, p.hd, p.ps = H, KV, hd, ps
    p.max_pages = block_table.shape[1]
    p.num_pages = kv.shape[0]
    p.q_stride = q_stride
    p.window = int(window or 0)
    p.sel_stride = sel_pages.shape[1] if sel_pages is not None else 0
    p.dump_stride = dump.shape[-1] if dump is not None else 0
    p.dtype = dtype_code(q.dtype)
    p.splits = splits
    p.row_filter = row_filter
    p.fuse = fuse
    p.rope_table = _ptr(rope_table, "rope_table", torch.float32)
    p.rope_positions = rope_table.shape[0] if rope_table is not None else 0
    p.scale = float(scale)
    return p


def attention_plain(params: AttnParams):
    _l.check(_l.load().dk_attention_plain(C.byref(params), _stream()), "attention_plain")


def attention_decode_supported(dtype, H, KV, hd, ps) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(_l.load().dk_attention_decode_supported(BF16, H, KV, hd, ps))


_decode_occupancy = {}


def attention_decode_blocks_per_sm(H, KV, hd, block_entries) -> int:
    """Blocks of the decode kernel one SM of the current device holds at once (asked of the runtime once)."""
    key = (_device_index(), H, KV, hd, block_entries)
    if key not in _decode_occupancy:
        n = int(_l.load().dk_attention_decode_blocks_per_sm(H, KV, hd, block_entries))
        if n < 1:
            raise KernelError("attention_decode: " + _l.load().dk_last_error().decode("utf-8", "replace"))
        _decode_occupancy[key] = n
    return _decode_occupancy[key]


def attention_decode_max_clusters(H, KV, hd, block_entries, splits) -> int:
    """Clusters of ``splits`` blocks of the decode kernel that the current device holds at once (asked of the runtime once)."""
    key = (_device_index(), H, KV, hd, block_entries, splits)
    if key not in _decode_occupancy:
        n = int(_l.load().dk_attention_decode_max_clusters(H, KV, hd, block_entries, splits))
        if n < 1:
            raise KernelError("attention_decode: " + _l.load().dk_last_error().decode("utf-8", "replace"))
        _decode_occupancy[key] = n
    return _decode_occupancy[key]


def attention_decode_scratch_floats(rows, H, hd, splits) -> int:
    return int(_l.load().dk_attention_decode_scratch_floats(rows, H, hd, splits))


def attention_decode(params: AttnParams):
    """One new token per row; ``params.splits`` blocks share a request's keys and, when there
    is more than one, ``params.scratch`` holds their partial results."""
    _l.check(_l.load().dk_attention_decode(C.byref(params), _stream()), "attention_decode", 2 if params.splits > 1 else 1)


def attention_prefill_supported(dtype, H, KV, hd, ps) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(_l.load().dk_attention_prefill_supported(BF16, H, KV, hd, ps))


def attention_prefill(params: AttnParams, max_q_len: int):
    """Rows that bring several tokens (``params.row_filter`` 2 leaves single tokens to the
    decode kernel); ``max_q_len`` is the most tokens any row brings."""
    _l.check(_l.load().dk_attention_prefill(C.byref(params), int(max_q_len), _stream()), "attention_prefill")


def attention_prefill_tc_supported(dtype, H, KV, hd, ps, q_stride) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(_l.load().dk_attention_prefill_tc_supported(BF16, H, KV, hd, ps, int(q_stride)))


def attention_prefill_tc(params: AttnParams, max_q_len: int):
    """The same rows as ``attention_prefill`` on the tcgen05 tensor cores: 128 queries a block,
    accumulators in tensor memory, pages fetched by TMA."""
    _l.check(_l.load().dk_attention_prefill_tc(C.byref(params), int(max_q_len), _stream()), "attention_prefill_tc")


def gemm_small_m_supported(M, N, K, swiglu=False) -> bool:
    return bool(_l.load().dk_gemm_small_m_supported(M, N, K, int(swiglu)))


def gemm_small_m(x, w, out, swiglu=False):
    """out = x @ w^T for up to 64 rows of bfloat16 x, streaming w once.  ``swiglu``: w holds
    gate rows then up rows, and out [M, N/2] = silu(x gate^T) * (x up^T)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_small_m: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} or dtypes do not fit")
    _l.check(_l.load().dk_gemm_small_m(_ptr(x, "x"), _ptr(w, "w"), _ptr(out, "out"), M, N, K, x.stride(0), w.stride(0),
                                       out.stride(0), dtype_code(out.dtype), int(swiglu), _stream()), "gemm_small_m")
    return out


def gemm_tc_supported(M, N, K, swiglu=False) -> bool:
    return bool(_l.load().dk_gemm_tc_supported(M, N, K, int(swiglu)))


def gemm_tc_many_rows_supported(M, N, K, swiglu=False) -> bool:
    return bool(_l.load().dk_gemm_tc_many_rows_supported(M, N, K, int(swiglu)))


def gemm_tc(x, w, out, swiglu=False, splits=1, err=None, per_sm=1):
    """out = x @ w^T for up to 128 rows of bfloat16 x on the tcgen05 tensor cores; the weights
    stream through shared memory by TMA.  ``splits`` blocks (1, 2, 4, 8) share K as a cluster.
    ``swiglu``: w holds gate rows then up rows, out [M, N/2] = silu(x gate^T) * (x up^T).
    ``per_sm`` 2: shorter stages, so that two blocks fit on an SM.
    More than 128 rows are taken in chunks of up to 256 (``splits`` and ``per_sm`` 1)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} or dtypes do not fit")
    _l.check(_l.load().dk_gemm_tc(_ptr(x, "x"), _ptr(w, "w"), _ptr(out, "out"), M, N, K, x.stride(0), w.stride(0),
                                  out.stride(0), dtype_code(out.dtype), int(swiglu), int(splits), int(per_sm),
                                  _ptr(err, "err", torch.int32), _stream()), "gemm_tc")
    return out


def gemm_stream_k_supported(M, N, K, swiglu=False) -> bool:
    return bool(_l.load().dk_gemm_stream_k_supported(M, N, K, int(swiglu)))


_stream_k_workspace = {}


def gemm_stream_k(x, w, out, swiglu=False, err=None):
    """out = x @ w^T for up to 128 rows of bfloat16 x as one persistent tcgen05 kernel: the
    (tile, K step) sequence is cut into one equal piece per SM, tiles that two pieces share are
    summed through a workspace in block order.  The workspace (partials and flags, zero at first)
    belongs to the device and is used by one stream at a time.
    ``swiglu``: w holds gate rows then up rows, out [M, N/2] = silu(x gate^T) * (x up^T)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_stream_k: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} or dtypes do not fit")
    ws = _stream_k_workspace.get(x.device)
    if ws is None:
        ws = torch.zeros(int(_l.load().dk_gemm_stream_k_workspace_bytes(128)), dtype=torch.uint8, device=x.device)
        _stream_k_workspace[x.device] = ws
    _l.check(_l.load().dk_gemm_stream_k(_ptr(x, "x"), _ptr(w, "w"), _ptr(out, "out"), M, N, K, x.stride(0), w.stride(0),
                                        out.stride(0), dtype_code(out.dtype), int(swiglu), _ptr(ws, "workspace", torch.uint8),
                                        _ptr(err, "err", torch.int32), _stream()), "gemm_stream_k")
    return out


def recent_pages(row_slot, row_flags, row_pos_start, row_q_len, sel_pages, sel_count, ps, ratio, page_ahead=False):
    """``page_ahead``: a request whose newest page is exactly full counts one more, empty page (see delta_select.cu)."""
    i32 = torch.int32
    _l.check(_l.load().dk_recent_pages(_ptr(row_slot, "row_slot", i32), _ptr(row_flags, "row_flags", i32),
                                       _ptr(row_pos_start, "row_pos_start", i32), _ptr(row_q_len, "row_q_len", i32),
                                       _ptr(sel_pages, "sel_pages", i32), _ptr(sel_count, "sel_count", i32),
                                       row_slot.shape[0], sel_pages.shape[1], ps, float(ratio), int(page_ahead), _stream()), "recent_pages")


def page_scores(dump, lse, row_flags, row_q_start, row_pos_start, row_q_len, scores, ps, k, ratio, page_ahead=False):
    rows, H, stride = dump.shape
    i32 = torch.int32
    _l.check(_l.load().dk_page_scores(_ptr(dump, "dump", torch.float32), _ptr(lse, "lse", torch.float32),
                                      _ptr(row_flags, "row_flags", i32), _ptr(row_q_start, "row_q_start", i32),
                                      _ptr(row_pos_start, "row_pos_start", i32), _ptr(row_q_len, "row_q_len", i32),
                                      _ptr(scores, "scores", torch.float32), rows, H, ps, stride, scores.shape[1], k,
                                      float(ratio), int(page_ahead), _stream()), "page_scores")


def select_pages(scores, row_slot, row_flags, row_pos_start, row_q_len, sel_pages, sel_count, keep_last, ps, bias, ratio,
                 page_ahead=False):
    i32 = torch.int32
    _l.check(_l.load().dk_select_pages(_ptr(scores, "scores", torch.float32), _ptr(row_slot, "row_slot", i32),
                                       _ptr(row_flags, "row_flags", i32), _ptr(row_pos_start, "row_pos_start", i32),
                                       _ptr(row_q_len, "row_q_len", i32), _ptr(sel_pages, "sel_pages", i32),
                                       _ptr(sel_count, "sel_count", i32), scores.shape[0], scores.shape[1],
                                       sel_pages.shape[1], keep_last, ps, float(bias), float(ratio), int(page_ahead),
                                       _stream()), "select_pages")


def sample(logits, out, temperature=None, top_p=None, seeds=None, positions=None, err=None):
    """One token per row of float ``logits`` [R, V]: greedy where temperature is 0
    (or not given), else a draw from softmax(logits / temperature).  With ``err`` (the kernels'
    error record) ``out`` has four more ints than rows, and the record is copied behind the tokens."""
    R, V = logits.shape
    if err is not None:
        if out.shape[0] != R + 4:
            raise KernelError(f"sample: with an error record the output holds rows + 4 ints, got {out.shape[0]} for {R} rows")
        if R == 0:
            out.copy_(err)
            return out
    _l.check(_l.load().dk_sample(_ptr(logits, "logits", torch.float32), logits.stride(0) if R else V, R, V,
                                 _ptr(temperature, "temperature", torch.float32), _ptr(top_p, "top_p", torch.float32),
                                 _ptr(seeds, "seeds", torch.int64), _ptr(positions, "positions", torch.int32),
                                 _ptr(out, "out", torch.int32), _ptr(err, "err", torch.int32), _stream()), "sample")
    return out
