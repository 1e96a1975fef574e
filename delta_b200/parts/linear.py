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


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """x [T, K], w [N, K] -> [T, N] in ``out_dtype`` (the type of x by default)."""
    out_dtype = out_dtype or x.dtype
    T, N = x.shape[0], w.shape[0]
    if x.dtype == torch.float32 or ctx.plain_products:
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
        if T:
            ops.gemm_nt_plain(x, w, out)
        return out
    if out_dtype == x.dtype:
        ops.count_launch()
        return torch.mm(x, w.t())
    out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    if T:
        ops.gemm_nt_plain(x, w, out)
    return out
