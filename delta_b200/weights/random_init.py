"""Random weights from a configuration and a seed.

``write_random_model`` writes a model folder (config.json, model.safetensors):
matrices and the embedding table N(0, 0.02), norm weights 1 + U(-0.1, 0.1), drawn
on the CPU from one seeded generator in the order of the model's tensor list, so
that anything reading the folder sees the same values.  ``random_tensors`` draws
the same kinds of values straight on a device for models too large to be worth
writing (benchmarks).  The reference has no such mode: it builds its model on the
meta device and needs a real checkpoint (DELTA/Engine/utils.py:211-223).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List

import torch

from ..parts.base import TensorSpec
from .safetensors_io import write_safetensors


def _draw(spec: TensorSpec, gen: torch.Generator, device) -> torch.Tensor:
    if spec.init == "normal":
        return torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32) * 0.02
    if spec.init == "norm":
        return 1.0 + (torch.rand(spec.shape, generator=gen, device=device, dtype=torch.float32) * 0.2 - 0.1)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, device=device, dtype=torch.float32)
    raise ValueError(f"unknown init '{spec.init}' of tensor {spec.name}")


def random_tensors(specs: List[TensorSpec], seed: int, compute: torch.dtype, device) -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for s in specs:
        if s.kind == "int":
            out[s.name] = torch.zeros(s.shape, dtype=torch.int32, device=device)
        else:
            out[s.name] = _draw(s, gen, device).to(compute)
    return out


def write_random_model(folder, config_json: dict, seed: int, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Writes ``folder/config.json`` and ``folder/model.safetensors`` for the
    architecture that ``config_json`` names, with every float tensor stored in ``dtype``."""
    from ..config.registry import architecture_of
    from ..models.model import Model
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch = architecture_of(config_json)
    cfg = arch.config_from_dict(config_json)
    model = Model(arch.build_spec(cfg, None))
    tensors = random_tensors(model.tensor_specs(), seed, dtype, "cpu")
    (folder / "config.json").write_text(json.dumps(config_json, indent=1))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder
