"""Interfaces of the parts a layer is put together from, and their registries.

A model is data: a list of layers, each naming a block arrangement, two norms, a
mixer and a feed-forward by their registry names with their parameters, and a
list that says in which order layers run and which cache each run uses.  The
parts know their own sizes and constants and nothing about the model they sit
in.  A new part is a class registered under a new name; nothing else changes.

The reference builds one fixed module tree (DELTA/Engine/DELTA/model.py:130-137,
330-336) whose sizes come through ``ModelArgs``; the parts below are the same
units (RMSNorm 521-532, Attention 362-492, FeedForward 495-518,
TransformerBlock 330-341) made exchangeable.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional

import torch


# ---------------------------------------------------------------- tensors

@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part needs from the model folder.

    ``kind``: "matrix" (operand of a matrix product, kept in the compute type),
    "vector" (norm weights and the like; a tensor stored in 32 bit stays so),
    "table" (embedding rows, kept in the compute type), "int" (integer tables,
    kept as int32).  ``init`` names how random weights are drawn: "normal"
    N(0, 0.02), "norm" 1 + U(-0.1, 0.1), "zeros".
    """
    name: str
    shape: tuple
    kind: str = "matrix"
    init: str = "normal"


PAGE = "page"     # the axis of a page layout that counts the tokens of the page


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps per token, and how far back it reads.

    ``layout`` is the shape of one page of one layer with the token axis written
    as ``PAGE``: keys and values per head are ``(2, kv_heads, PAGE, head_dim)``, one
    latent vector per token is ``(PAGE, width)``, keys and values of different
    widths can be packed as ``(kv_heads, PAGE, k_width + v_width)``.  The cache
    manager allocates ``[layers of the group, pages, *layout]`` with the page size
    in place of ``PAGE`` and knows nothing else about the contents.  Mixers with
    equal specs share a cache group (one pool of pages, one block table per
    request); ``window`` None means every token is kept.  ``run_tokens``: the mixer reads
    a request's pages fastest when the pages of this many consecutive tokens follow one another
    in the pool; the pool then hands pages out in aligned runs of that length where it can
    (0: any order is as good)."""
    layout: tuple
    window: Optional[int] = None
    run_tokens: int = 0

    def __post_init__(self):
        if tuple(self.layout).count(PAGE) != 1:
            raise ValueError(f"a page layout names the token axis once, as PAGE: {self.layout}")
        object.__setattr__(self, "layout", tuple(self.layout))

    def page_shape(self, page_size: int) -> tuple:
        return tuple(page_size if a == PAGE else int(a) for a in self.layout)

    def describe(self) -> str:
        return "x".join("P" if a == PAGE else str(a) for a in self.layout) + (f"w{self.window}" if self.window else "")


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, one slot per request slot.  Parts that name
    the same key share the tensor.  ``fill`` is the value a slot is reset to when a
    request is admitted."""
    shape: tuple
    dtype: torch.dtype = torch.float32
    fill: float = 0.0


# ------------------------------------------------------------------ parts

class Part:
    """Anything with weights.  ``prefix`` is the tensor-name prefix in the model folder."""

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Takes the tensors named by ``tensor_specs`` (on the device, already in
        the type their kind asks for)."""

    def state_specs(self) -> Dict[str, StateSpec]:
        return {}

    def begin_step(self, ctx) -> None:
        """Called once per step before any layer runs."""

    def decode_rows_differ(self) -> bool:
        """True when the part treats a row flagged ``ROW_DECODE`` otherwise than the same
        token inside a prompt portion.  The scheduler then never folds generated tokens
        into a prompt portion: a request that is recomputed feeds them one per step."""
        return False


class Norm(Part):
    """``forward(ctx, x, out=None, add=None, rows=None)``: normalises rows of x [T, d].
    With ``add`` the sum x + add is written back to x first (the residual sum,
    fused); with ``rows`` only those rows are read and the output has len(rows) rows."""

    def forward(self, ctx, x, add=None, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    """Position information a mixer applies to its queries and keys.  ``table(device)``
    returns what the mixer's kernel needs (for rotary positions: cos and sin)."""

    def table(self, device):
        raise NotImplementedError


class Mixer(Part):
    """The part of a layer that mixes tokens.  ``cache_spec()`` says what it keeps per
    token (None: nothing); ``forward(ctx, x, cache)`` maps normalised rows x [T, d]
    to [T, d], appending to ``cache`` when ``cache.writes`` and reading from it."""

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def forward(self, ctx, x, cache):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(ctx, x)``: rows [T, d] to rows [T, d], token by token."""

    def forward(self, ctx, x):
        raise NotImplementedError


class Block(Part):
    """Arrangement of parts around the residual stream.  A block is built from a dict
    of parts, ``{role: part}``; which roles it needs is the block's own business (the
    pre-norm block: norm1, mixer, norm2, feed_forward; another block may take more
    norms, no feed-forward, two mixers).  ``forward(ctx, x, pending, cache)`` takes the
    stream x [T, d] and a not yet added update ``pending`` (or None) and returns the
    same pair."""

    roles: tuple = ()

    def __init__(self, parts: Dict[str, Part]):
        missing = [r for r in self.roles if r not in parts]
        extra = [r for r in parts if r not in self.roles]
        if missing or extra:
            raise ValueError(f"{type(self).__name__} takes the parts {list(self.roles)}; missing {missing}, not taken {extra}")
        self._parts = dict(parts)
        for role, part in parts.items():
            setattr(self, role, part)

    def parts(self) -> list:
        return list(self._parts.values())

    def cache_spec(self) -> Optional[CacheSpec]:
        """What a run of this block appends to its cache: that of its first part that keeps one."""
        for p in self._parts.values():
            cs = p.cache_spec() if hasattr(p, "cache_spec") else None
            if cs is not None:
                return cs
        return None

    def forward(self, ctx, x, pending, cache):
        raise NotImplementedError


# Flags of a row of a step (``RowInput.flags``, ``ctx.row_flags``), for parts to interpret.
ROW_DECODE = 1      # a single token at or after the end of the request's prompt


# -------------------------------------------------------------- registries

class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Callable[..., Any]] = {}

    def register(self, name: str):
        def deco(cls):
            if name in self._items and self._items[name] is not cls:
                raise ValueError(f"{self.what} '{name}' is registered already")
            self._items[name] = cls
            return cls
        return deco

    def unregister(self, name: str) -> None:
        self._items.pop(name, None)

    def create(self, kind: str, /, **params):
        if kind not in self._items:
            raise KeyError(f"unknown {self.what} '{kind}'; known: {', '.join(sorted(self._items)) or 'none'}")
        return self._items[kind](**params)

    def names(self) -> list[str]:
        return sorted(self._items)

    def __contains__(self, name: str) -> bool:
        return name in self._items


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")


REGISTRIES = {"norm": NORMS, "position": POSITION_ENCODINGS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS,
              "block": BLOCKS}


@dataclass(frozen=True)
class PartSpec:
    """Registry name of a part, its parameters, and the registry it is looked up in
    ("norm", "position", "mixer", "feed_forward", "block")."""
    kind: str
    params: dict = field(default_factory=dict)
    category: str = ""

    def build(self, registry: Optional[Registry] = None, **extra):
        if registry is None:
            if self.category not in REGISTRIES:
                raise KeyError(f"part '{self.kind}' names no registry (category '{self.category}'); known: {', '.join(REGISTRIES)}")
            registry = REGISTRIES[self.category]
        return registry.create(self.kind, **{**self.params, **extra})
