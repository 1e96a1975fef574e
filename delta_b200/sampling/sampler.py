"""Greedy and temperature sampling.

The reference's live path is greedy: ``torch.argmax`` inside the model
(DELTA/Engine/DELTA/model.py:323).  Its helpers for temperature and top-p
sampling (DELTA/Engine/utils.py:81-111: the top-p filter on sorted cumulative
probabilities, then ``softmax(logits / T)`` and one multinomial draw) give the
meaning of the other two options here.  The draw uses a counter-based generator
keyed by (seed of the request, position of the new token), so what a request
samples depends neither on its batch nor on how its prompt was cut into steps.
The kernel (csrc/sampling.cu) is launched by the step function with the rows'
parameters from the step's staging block.
"""
from __future__ import annotations

from dataclasses import dataclass

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0   # 0: greedy
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if not (0 < self.top_p <= 1):
            raise ValueError("top_p must lie in (0, 1]")


def uniform_of(seed: int, position: int) -> float:
    """The uniform number in (0, 1) that the kernel uses for this (seed, position)."""
    x = (seed + (position + 1) * 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return ((z >> 40) + 0.5) / 16777216.0
