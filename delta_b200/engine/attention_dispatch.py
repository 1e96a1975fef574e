"""Chooses the attention kernel for a batch."""
from __future__ import annotations

from ..kernels import ops


def run(ctx, params) -> None:
    ops.attention_plain(params)
