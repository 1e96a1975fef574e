"""Arrangement of a layer: the pre-norm residual block
    h = x + mixer(norm1(x));  out = h + feed_forward(norm2(h))
(reference: DELTA/Engine/DELTA/model.py:338-341).

The residual sum is not a kernel of its own: a block hands its last update on as
``pending`` and the next norm adds it while it reads the stream, so the stream is
read and written once per norm."""
from __future__ import annotations

from .base import BLOCKS, Block


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    roles = ("norm1", "mixer", "norm2", "feed_forward")

    def forward(self, ctx, x, pending, cache):
        a = self.norm1.forward(ctx, x, add=pending)
        y = self.mixer.forward(ctx, a, cache)
        f = self.norm2.forward(ctx, x, add=y)
        m = self.feed_forward.forward(ctx, f)
        return x, m
