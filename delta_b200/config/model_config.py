"""Typed model configuration, read from the keys of the architecture's config.json.

The reference has no config.json reader: it keeps a table of sizes keyed by
directory name (DELTA/Engine/DELTA/model.py:57-97, ``ModelArgs`` at 20-55).
Here every size and constant comes from the model folder, and nothing that
config.json gives is repeated in code.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Optional


class ConfigError(ValueError):
    """config.json is missing a key, or asks for something this engine does not do."""


_FULL = "full_attention"
_SLIDING = "sliding_attention"


@dataclass(frozen=True)
class YiConfig:
    """Sizes and constants of a Yi model (Llama-layout dense decoder).

    Field names are the config.json keys.  ``head_dim`` is optional in the file
    (``hidden_size // num_attention_heads`` then; the reference always uses that
    quotient, model.py:51).  ``layer_types`` and ``sliding_window`` are optional:
    a layer listed as ``sliding_attention`` attends to the last
    ``sliding_window`` tokens only and keeps its keys in a cache group of its own.
    """
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    sliding_window: Optional[int] = None
    layer_types: tuple = ()
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    # ---- reading -------------------------------------------------------
    @staticmethod
    def from_dict(c: dict) -> "YiConfig":
        def need(key):
            if key not in c or c[key] is None:
                raise ConfigError(f"config.json has no '{key}'")
            return c[key]

        archs = c.get("architectures") or []
        if not archs:
            raise ConfigError("config.json has no 'architectures'")
        hidden = int(need("hidden_size"))
        heads = int(need("num_attention_heads"))
        kv = int(c.get("num_key_value_heads") or heads)
        head_dim = c.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"hidden_size {hidden} is no multiple of num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        layers = int(need("num_hidden_layers"))
        if c.get("tie_word_embeddings"):
            raise ConfigError("tie_word_embeddings=true: Yi has an lm_head of its own")
        if c.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act '{c['hidden_act']}' is not supported (silu only)")
        if c.get("attention_bias") or c.get("mlp_bias"):
            raise ConfigError("attention_bias / mlp_bias are not supported")
        if c.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is not supported")
        if heads % kv:
            raise ConfigError(f"num_attention_heads {heads} is no multiple of num_key_value_heads {kv}")
        window = c.get("sliding_window")
        lt = tuple(c.get("layer_types") or ())
        if lt:
            if len(lt) != layers:
                raise ConfigError(f"layer_types has {len(lt)} entries for {layers} layers")
            for t in lt:
                if t not in (_FULL, _SLIDING):
                    raise ConfigError(f"unknown layer type '{t}'")
            if _SLIDING in lt and not window:
                raise ConfigError("layer_types names sliding_attention but sliding_window is not set")
        eos = c.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        cfg = YiConfig(
            architecture=str(archs[0]), hidden_size=hidden, num_hidden_layers=layers,
            num_attention_heads=heads, num_key_value_heads=kv, head_dim=int(head_dim),
            intermediate_size=int(need("intermediate_size")), vocab_size=int(need("vocab_size")),
            rms_norm_eps=float(need("rms_norm_eps")), rope_theta=float(c.get("rope_theta", 10000.0)),
            max_position_embeddings=int(need("max_position_embeddings")),
            sliding_window=int(window) if window else None, layer_types=lt,
            bos_token_id=c.get("bos_token_id"), eos_token_id=eos,
            torch_dtype=str(c.get("torch_dtype") or c.get("dtype") or "bfloat16"))
        cfg.validate()
        return cfg

    @staticmethod
    def from_folder(folder) -> "YiConfig":
        path = Path(folder) / "config.json"
        if not path.is_file():
            raise ConfigError(f"no config.json in {folder}")
        return YiConfig.from_dict(json.loads(path.read_text()))

    def validate(self) -> None:
        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                     "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} is odd: rotary positions need pairs")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be positive")
        if not (self.rope_theta > 0):
            raise ConfigError("rope_theta must be positive")

    # ---- writing -------------------------------------------------------
    def to_dict(self) -> dict:
        d = asdict(self)
        arch = d.pop("architecture")
        d["architectures"] = [arch]
        d["layer_types"] = list(self.layer_types) or None
        d["hidden_act"] = "silu"
        d["tie_word_embeddings"] = False
        d["attention_bias"] = False
        d["mlp_bias"] = False
        d["rope_scaling"] = None
        d["model_type"] = "llama"
        return {k: v for k, v in d.items() if v is not None or k in ("rope_scaling",)}

    def window_of_layer(self, layer: int) -> Optional[int]:
        if self.layer_types and self.layer_types[layer] == _SLIDING:
            return self.sliding_window
        return None
