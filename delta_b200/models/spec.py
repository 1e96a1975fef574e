"""A model as data: layers made of named parts, and the order in which they run."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional

from ..parts.base import PartSpec, TensorSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the parts it is built from, by the role each
    plays in that block (the pre-norm block: norm1, mixer, norm2, feed_forward).  Every
    ``PartSpec`` names its registry in ``category``."""
    parts: Mapping[str, PartSpec]
    block: str = "pre_norm"


@dataclass(frozen=True)
class RunEntry:
    """One run of a layer.  ``cache`` names the cache the run uses (an index of its
    own by default); ``writes_cache`` False makes the run read a cache that another
    run filled instead of appending its own keys and values."""
    layer: int
    cache: Optional[int] = None
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """Everything the generic model needs: sizes of the token interface, the layers,
    the run order (a layer may be named twice), the last norm and the names of the
    embedding table and of the output matrix."""
    vocab_size: int
    width: int
    layers: tuple
    order: tuple
    final_norm: PartSpec
    embedding: TensorSpec
    lm_head: TensorSpec
    max_positions: int = 0
    ignorable_tensors: tuple = ()   # shell patterns of tensor names a model folder may hold beside the ones asked for

    def __post_init__(self):
        for e in self.order:
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"run order names layer {e.layer}, the model has {len(self.layers)}")
