"""Rotary position encoding.

Pair j of a head is rotated by the angle  position / (scale * theta^(2j/head_dim))
(reference: DELTA/Engine/DELTA/model.py:165-175, ``apply_rope`` with
``rope_scale`` and ``rope_theta``).  The reference pairs neighbouring elements
(2j, 2j+1) because it runs checkpoints whose q and k rows were permuted by a
converter; on the rows of an unconverted model folder the same function pairs
(j, j + head_dim/2), which is the default here.  ``interleaved=True`` gives the
reference's pairing.

Cos and sin are tabulated once per (head_dim, theta, scale) in 64 bit and
rounded to 32 bit, so the kernels do no trigonometry and the angles carry no
32-bit rounding of a large position times a small frequency.
"""
from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, PositionEncoding

_TABLES: dict = {}


@POSITION_ENCODINGS.register("rotary")
class RotaryPositions(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int, interleaved: bool = False, scale: float = 1.0):
        if head_dim % 2:
            raise ValueError(f"rotary positions need an even head size, got {head_dim}")
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self.interleaved = bool(interleaved)
        self.scale = float(scale)

    def table_cpu(self) -> torch.Tensor:
        """[max_positions, head_dim/2, 2] float32: cos and sin of every angle."""
        half = self.head_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        inv = 1.0 / (self.scale * self.theta ** (2.0 * j / self.head_dim))
        ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).contiguous()

    def table(self, device) -> torch.Tensor:
        key = (self.head_dim, self.theta, self.scale, self.max_positions, str(device))
        if key not in _TABLES:
            _TABLES[key] = self.table_cpu().to(device)
        return _TABLES[key]
