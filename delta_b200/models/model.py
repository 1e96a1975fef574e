"""The generic model: parts built from a ``ModelSpec`` and run in its order.

Reference counterpart: ``Transformer.forward`` (DELTA/Engine/DELTA/model.py:198-206):
embedding, the blocks, the last norm and the output product.  Differences that are
meant: logits are made only for the rows that are asked for and are returned (the
reference makes them for every row and returns their argmax, model.py:205, 323),
and the run order is a list, not the layer index.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..parts import linear
from ..parts.base import BLOCKS, NORMS, CacheSpec, StateSpec, TensorSpec
from .spec import ModelSpec, RunEntry


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.blocks = []
        for ls in spec.layers:
            self.blocks.append(BLOCKS.create(ls.block, parts={role: ps.build() for role, ps in ls.parts.items()}))
        self.final_norm = spec.final_norm.build(NORMS)
        self.embed_table = None
        self.lm_head = None
        # run order with every entry's cache index resolved
        self.order: List[RunEntry] = []
        for n, e in enumerate(spec.order):
            self.order.append(RunEntry(e.layer, e.cache if e.cache is not None else n, e.writes_cache))
        writers = {e.cache for e in self.order if e.writes_cache}
        for e in self.order:
            if not e.writes_cache and e.cache not in writers:
                raise ValueError(f"a run of layer {e.layer} reads cache {e.cache}, which no run writes")

    # ---- what the model needs ---------------------------------------------
    def parts(self):
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [self.spec.embedding]
        for p in self.parts():
            specs.extend(p.tensor_specs())
        specs.append(self.spec.lm_head)
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.embed_table = tensors[self.spec.embedding.name]
        self.lm_head = tensors[self.spec.lm_head.name]
        for p in self.parts():
            p.bind(tensors)

    def cache_specs(self) -> Dict[int, CacheSpec]:
        """cache index -> what its writer keeps per token (runs without a cache are left out)."""
        out = {}
        for e in self.order:
            cs = self.blocks[e.layer].cache_spec()
            if cs is None:
                continue
            if e.writes_cache:
                out[e.cache] = cs
        for e in self.order:
            cs = self.blocks[e.layer].cache_spec()
            if cs is not None and not e.writes_cache and out[e.cache].layout != cs.layout:
                raise ValueError(f"layer {e.layer} reads cache {e.cache} whose page layout differs from its own")
        return out

    def decode_rows_differ(self) -> bool:
        """True when some part treats decode rows otherwise than the same tokens in a prompt portion."""
        return any(p.decode_rows_differ() for p in self.parts())

    def state_specs(self) -> Dict[str, StateSpec]:
        out: Dict[str, StateSpec] = {}
        for p in self.parts():
            for k, s in p.state_specs().items():
                if k in out and out[k] != s:
                    raise ValueError(f"two parts declare the state '{k}' with different layouts")
                out[k] = s
        return out

    # ---- a step -------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        """Runs the tokens of ``ctx`` and returns float32 logits [len(ctx.logit_rows), vocab]."""
        T = ctx.num_tokens
        x = torch.empty((T, self.spec.width), dtype=ctx.dtype, device=ctx.device)
        ops.embedding(ctx.tokens, self.embed_table, x, err=ctx.err)
        for p in self.parts():
            p.begin_step(ctx)
        pending = None
        for e in self.order:
            block = self.blocks[e.layer]
            cache = ctx.cache_view(e.cache, e.writes_cache) if block.cache_spec() is not None else None
            x, pending = block.forward(ctx, x, pending, cache)
        R = ctx.logit_rows.shape[0]
        if R == 0:      # nothing reads the stream after the last layer
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=ctx.device)
        h = self.final_norm.forward(ctx, x, add=pending, rows=ctx.logit_rows)
        return linear.linear(ctx, h, self.lm_head, out_dtype=torch.float32)
