"""One registry from the architecture name in config.json to its configuration
class and to the function that turns a configuration into a model.

The reference picks sizes by matching the checkpoint's directory name against a
table (DELTA/Engine/DELTA/model.py:57-69) and always builds its one
``Transformer``; here the name in ``architectures`` decides, and an unknown name
is an error that lists the known ones.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable  # dict of config.json -> typed configuration
    build_spec: Callable        # (configuration, EngineConfig) -> ModelSpec


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict: Callable, build_spec: Callable) -> None:
    ARCHITECTURES[name] = Architecture(name, config_from_dict, build_spec)


def unregister_architecture(name: str) -> None:
    ARCHITECTURES.pop(name, None)


def architecture_of(config_json: dict) -> Architecture:
    archs = config_json.get("architectures") or []
    if not archs:
        raise ConfigError("config.json has no 'architectures'")
    name = archs[0]
    if name not in ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}'; known: {', '.join(sorted(ARCHITECTURES))}")
    return ARCHITECTURES[name]


def read_config(folder):
    """(architecture, typed configuration) of a model folder."""
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {folder}")
    raw = json.loads(path.read_text())
    arch = architecture_of(raw)
    return arch, arch.config_from_dict(raw)
