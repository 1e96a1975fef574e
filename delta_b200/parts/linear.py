"""Matrix products  y = x W^T  of the parts.

32-bit activations go through the plain FMA kernel (true 32 bit: no
reduced-precision matrix mode, no split over K).  bfloat16 activations go
through the tensor cores: the library product that the reference uses for its
``nn.Linear`` layers (DELTA/Engine/DELTA/model.py:369-370, 498-500), or the
hand-written kernels where they are faster.
"""
from __future__ import annotations

import torch

from ..kernels import ops


SMALL_M = 64   # up to this many rows the product streams the weights once (decode steps)


def swiglu_linear(ctx, x: torch.Tensor, w_gate_up: torch.Tensor):
    """silu(x gate^T) * (x up^T) in one kernel when the batch is small enough; else None."""
    T, N, K = x.shape[0], w_gate_up.shape[0], x.shape[1]
    if x.dtype != torch.bfloat16 or ctx.plain_products or not (0 < T <= SMALL_M):
        return None
    if not ops.gemm_small_m_supported(T, N, K, swiglu=True):
        return None
    out = torch.empty((T, N // 2), dtype=x.dtype, device=x.device)
    return ops.gemm_small_m(x, w_gate_up, out, swiglu=True)


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """x [T, K], w [N, K] -> [T, N] in ``out_dtype`` (the type of x by default)."""
    out_dtype = out_dtype or x.dtype
    T, N = x.shape[0], w.shape[0]
    if x.dtype == torch.float32 or ctx.plain_products:
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
        if T:
            ops.gemm_nt_plain(x, w, out)
        return out
    if 0 < T <= SMALL_M and ops.gemm_small_m_supported(T, N, x.shape[1]):
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
        return ops.gemm_small_m(x, w, out)
    if out_dtype == x.dtype:
        ops.count_launch()
        return torch.mm(x, w.t())
    out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    if T:
        ops.gemm_nt_plain(x, w, out)
    return out
