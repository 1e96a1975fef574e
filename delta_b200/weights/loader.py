"""Loads the tensors a model names from the safetensors files of a model folder.

The reference loads a pickled state dict strictly (DELTA/Engine/utils.py:209-231)
and casts everything to bfloat16 (line 230).  Here tensors are looked up by their
names in the model folder; every problem (missing names, names nobody asked for,
wrong shapes) is collected and raised as one error.  An architecture may name
patterns of tensors that a folder is allowed to hold although the model does not
read them (stored ``rotary_emb.inv_freq`` buffers of older exports, for one).

Types: operands of matrix products and the embedding table are kept in the
compute type (bfloat16, or float32 on the 32-bit path); integer tables become
int32; any other tensor that the file stores in 32 bit stays in 32 bit.
"""
from __future__ import annotations

from fnmatch import fnmatchcase
from pathlib import Path
from typing import Dict, List, Sequence

import torch

from ..parts.base import TensorSpec
from .safetensors_io import open_model_files


class WeightError(ValueError):
    """The model folder does not hold what the model needs; lists every problem."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_type=()):
        self.missing, self.unexpected, self.wrong_shape, self.wrong_type = list(missing), list(unexpected), list(wrong_shape), list(wrong_type)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_type:
            lines.append(f"  wrong type: {name} is {got}")
        super().__init__("\n".join(lines))


def target_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.kind == "int":
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if spec.kind in ("matrix", "table"):
        return compute
    return torch.float32 if stored in (torch.float32, torch.float64) else compute


def load_tensors(folder, specs: List[TensorSpec], compute: torch.dtype, device, ignorable: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """``ignorable``: shell patterns of names that may be in the folder without being asked for."""
    files = open_model_files(folder)
    where = {}
    for f in files:
        for n in f.names():
            where[n] = f
    wanted = {s.name: s for s in specs}
    missing = [n for n in wanted if n not in where]
    unexpected = sorted(n for n in where if n not in wanted and not any(fnmatchcase(n, pat) for pat in ignorable))
    wrong_shape, wrong_type = [], []
    for n, s in wanted.items():
        if n in where:
            shape, dt = where[n].info(n)
            if tuple(shape) != tuple(s.shape):
                wrong_shape.append((n, tuple(s.shape), tuple(shape)))
            if s.kind == "int" and dt.is_floating_point or s.kind != "int" and not dt.is_floating_point:
                wrong_type.append((n, str(dt)))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(folder, missing, unexpected, wrong_shape, wrong_type)
    out = {}
    for n, s in wanted.items():
        t = where[n].tensor(n)
        out[n] = t.to(device=device, dtype=target_dtype(s, t.dtype, compute)).contiguous()
    for f in files:
        f.close()
    return out
