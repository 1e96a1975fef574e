"""RMSNorm: x * rsqrt(mean(x^2) + eps) * weight, the statistics in 32 bit
(reference: DELTA/Engine/DELTA/model.py:521-532)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import NORMS, Norm, TensorSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    """``width`` and ``eps`` are parameters.  ``cast_before_weight`` keeps the order of
    the reference in reduced precision: the normalised value is rounded to the
    activation type before it is multiplied by the weight (model.py:531-532)."""

    def __init__(self, name: str, width: int, eps: float, cast_before_weight: bool = True):
        self.name = name
        self.width = int(width)
        self.eps = float(eps)
        self.cast_before_weight = bool(cast_before_weight)
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width,), kind="vector", init="norm")]

    def bind(self, tensors):
        self.weight = tensors[self.name]

    def forward(self, ctx, x, add=None, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=x.dtype, device=x.device)
        cast_first = self.cast_before_weight and x.dtype != torch.float32
        return ops.rms_norm(x, self.weight, self.eps, out, add=add, rows=rows, cast_first=cast_first)
