"""SwiGLU feed-forward:  down( silu(gate x) * (up x) )
(reference: DELTA/Engine/DELTA/model.py:495-518, ``w2(silu(w1 x) * w3 x)``)."""
from __future__ import annotations

import torch

from ..kernels import ops
from . import linear
from .base import FEED_FORWARDS, FeedForward, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """``width`` d and ``intermediate`` I are parameters.  gate_proj and up_proj
    are stacked into one [2I, d] matrix so that one product feeds the gate kernel."""

    def __init__(self, prefix: str, width: int, intermediate: int):
        self.prefix = prefix
        self.width = int(width)
        self.intermediate = int(intermediate)
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        p, d, i = self.prefix, self.width, self.intermediate
        return [TensorSpec(p + "gate_proj.weight", (i, d)), TensorSpec(p + "up_proj.weight", (i, d)),
                TensorSpec(p + "down_proj.weight", (d, i))]

    def bind(self, tensors):
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"]

    def forward(self, ctx, x):
        act = linear.swiglu_linear(ctx, x, self.w_gate_up)
        if act is None:
            gu = linear.linear(ctx, x, self.w_gate_up)
            act = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
            ops.silu_mul(gu, act)
        return linear.linear(ctx, act, self.w_down)
