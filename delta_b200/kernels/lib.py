"""Loads the CUDA library and declares the C signature of every launcher.

There is one code path: the hand-written kernels.  If the library cannot be
built or loaded, or a tensor handed to a kernel is not on a CUDA device, the
call raises; nothing falls back to the CPU or to library model code.
"""
from __future__ import annotations

import ctypes as C
import threading

from .build import build

_lock = threading.Lock()
_lib = None

P = C.c_void_p
I = C.c_int
F = C.c_float
D = C.c_double


class KernelError(RuntimeError):
    """A launcher refused its arguments or the launch failed."""


class AttnParams(C.Structure):
    """Mirror of ``DkAttnParams`` in csrc/attention_params.h."""
    _fields_ = [
        ("q", P), ("out", P), ("kv", P), ("block_table", P), ("tok_row", P), ("tok_pos", P),
        ("row_slot", P), ("row_flags", P), ("row_q_start", P), ("row_q_len", P), ("row_pos_start", P),
        ("sel_pages", P), ("sel_count", P), ("dump", P), ("lse", P), ("scratch", P), ("err", P), ("rope_table", P),
        ("T", I), ("rows", I), ("H", I), ("KV", I), ("hd", I), ("ps", I), ("max_pages", I), ("num_pages", I),
        ("q_stride", I), ("window", I), ("sel_stride", I), ("dump_stride", I), ("dtype", I), ("splits", I),
        ("scale", F), ("block_entries", I), ("row_filter", I), ("fuse", I), ("rope_positions", I), ("reserved", I),
    ]


_SIGNATURES = {
    "dk_embedding": [P, P, P, I, I, I, I, P, P],
    "dk_rms_norm": [P, P, P, P, P, I, I, F, I, I, I, P],
    "dk_silu_mul": [P, P, I, I, I, P],
    "dk_rope_append": [P, P, P, P, I, P, I, P, I, I, I, I, I, I, I, I, P, P],
    "dk_gemm_nt_plain": [P, P, P, I, I, I, I, I, I, I, I, P],
    "dk_attention_plain": [C.POINTER(AttnParams), P],
    "dk_recent_pages": [P, P, P, P, P, P, I, I, I, D, I, P],
    "dk_page_scores": [P, P, P, P, P, P, P, I, I, I, I, I, I, D, I, P],
    "dk_select_pages": [P, P, P, P, P, P, P, I, I, I, I, I, F, D, I, P],
    "dk_sample": [P, I, I, I, P, P, P, P, P, P, P],
    "dk_attention_decode": [C.POINTER(AttnParams), P],
    "dk_attention_decode_supported": [I, I, I, I, I],
    "dk_attention_decode_blocks_per_sm": [I, I, I, I],
    "dk_attention_decode_max_clusters": [I, I, I, I, I],
    "dk_attention_prefill": [C.POINTER(AttnParams), I, P],
    "dk_attention_prefill_supported": [I, I, I, I, I],
    "dk_attention_prefill_tc": [C.POINTER(AttnParams), I, P],
    "dk_attention_prefill_tc_supported": [I, I, I, I, I, I],
    "dk_gemm_small_m": [P, P, P, I, I, I, I, I, I, I, I, P],
    "dk_gemm_small_m_supported": [I, I, I, I],
    "dk_gemm_tc": [P, P, P, I, I, I, I, I, I, I, I, I, I, P, P],
    "dk_gemm_tc_supported": [I, I, I, I],
    "dk_gemm_tc_many_rows_supported": [I, I, I, I],
    "dk_gemm_stream_k_supported": [I, I, I, I],
    "dk_gemm_stream_k": [P, P, P, I, I, I, I, I, I, I, I, P, P, P],
    "dk_wait_check": [P, C.c_longlong, P],
}


def load():
    """The loaded library (built at the first call)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = build()
        lib = C.CDLL(str(path))
        lib.dk_last_error.restype = C.c_char_p
        lib.dk_last_error.argtypes = []
        lib.dk_sizeof_attn_params.restype = I
        lib.dk_attention_decode_scratch_floats.restype = C.c_longlong
        lib.dk_attention_decode_scratch_floats.argtypes = [I, I, I, I]
        lib.dk_gemm_stream_k_workspace_bytes.restype = C.c_longlong
        lib.dk_gemm_stream_k_workspace_bytes.argtypes = [I]
        if lib.dk_sizeof_attn_params() != C.sizeof(AttnParams):
            raise KernelError(f"AttnParams is {C.sizeof(AttnParams)} bytes in Python and "
                              f"{lib.dk_sizeof_attn_params()} in the library: the two declarations differ")
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = I
            fn.argtypes = args
        _lib = lib
    return _lib


def declare(name: str, argtypes: list) -> None:
    """Adds a launcher's signature (used by kernel files that come later)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = I
        fn.argtypes = argtypes


LAUNCHES = [0]


def check(code: int, what: str, kernels: int = 1) -> None:
    """Raises when a launcher returned an error; counts the kernels it launched."""
    LAUNCHES[0] += kernels
    if code != 0:
        msg = load().dk_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what}: {msg} (code {code})")
