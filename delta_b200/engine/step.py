"""The step function: one batch of (request, its next tokens) in, logits out.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.
Only the tokens it brings are run, as one batch, against the cache that earlier
steps left; logits are made for the rows that are asked for.

Reference counterpart: ``LMBackend._forward`` (DELTA/Engine/DELTA/backend.py:1641-1792)
with its batch builders (1850-1936, 2040-2172) and ``Transformer.forward``
(model.py:198-206).  The reference builds CSR page lists and calls a planning
routine of its attention library every step; here the kernels read the block table
rows directly, so the host work of a step is filling one staging buffer and one
copy to the device.
"""
from __future__ import annotations

import gc
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..config.registry import architecture_of, read_config
from ..kernels import ops
from ..models.model import Model
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors
from .context import StepContext


@dataclass
class RowInput:
    """One request's share of a step: its next tokens, the position of the first of
    them, and the places among them whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    start_pos: int
    want: Sequence[int] = ()
    flags: int = 0            # bits for the parts to interpret (parts.base.ROW_DECODE: a single token at or after the prompt's end)
    sampling: Optional[object] = None   # SamplingParams for the tokens sampled at ``want`` (None: greedy)


@dataclass
class StepResult:
    """What a sampled step leaves for the host: ``tensor`` [rows + 4] int32 on the device holds the
    new tokens (the first ``n_tokens`` belong to requests) and, from ``status_at`` on, the four
    ints of the kernels' error record as the step's last kernel saw them."""
    tensor: torch.Tensor
    n_tokens: int
    status_at: int


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


def _require_cuda(device: torch.device) -> None:
    if device.type != "cuda":
        raise RuntimeError("delta_b200 runs on a CUDA device only; there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; delta_b200 has no CPU path")
    torch.cuda.set_device(device)


def _alloc_pinned(n: int) -> torch.Tensor:
    return torch.empty(n, dtype=torch.int32, pin_memory=True)


def _record_event():
    ev = torch.cuda.Event()
    ev.record()
    return ev


class ModelRunner:
    """Owns the model, its weights, the cache manager and the step function."""

    def __init__(self, model_dir=None, *, engine_config: Optional[EngineConfig] = None, config_json: Optional[dict] = None,
                 seed: Optional[int] = None, device="cuda:0"):
        self.cfg = engine_config or EngineConfig()
        self.device = torch.device(device)
        _require_cuda(self.device)
        self.dtype = torch.bfloat16 if self.cfg.dtype == "bfloat16" else torch.float32
        if model_dir is not None:
            arch, self.model_config = read_config(model_dir)
        elif config_json is not None:
            arch = architecture_of(config_json)
            self.model_config = arch.config_from_dict(config_json)
        else:
            raise ValueError("give a model folder, or config_json with a seed for random weights")
        self.architecture = arch
        self.spec = arch.build_spec(self.model_config, self.cfg)
        self.model = Model(self.spec)
        specs = self.model.tensor_specs()
        if model_dir is not None:
            tensors = load_tensors(model_dir, specs, self.dtype, self.device, ignorable=self.spec.ignorable_tensors)
        else:
            tensors = random_tensors(specs, 0 if seed is None else seed, self.dtype, self.device)
        self.model.bind(tensors)
        self.cache = CacheManager(self.model.cache_specs(), self.model.state_specs(), max_slots=self.cfg.max_batch,
                                  max_seq_len=self.cfg.max_seq_len, page_size=self.cfg.page_size,
                                  num_pages=self.cfg.pool_pages, dtype=self.dtype, device=self.device,
                                  shuffle_seed=self.cfg.shuffle_pages, page_runs=self.cfg.page_runs)
        self.vocab_size = self.spec.vocab_size
        self.err = ops.new_error_record(self.device)
        self._scratch: Dict[str, torch.Tensor] = {}
        self._staging = []      # ring of (pinned buffer, event)
        self.on_device_work = None   # called once per step right before its first device operation (for timing)
        self._staging_next = 0
        self.plain_kernels = set()   # "products", "attention": take the slow plain kernels (for comparisons)
        self.capture: Optional[dict] = None
        self.steps_run = 0
        self.last_staging_bytes = 0
        self._graphs: Dict[int, dict] = {}
        self.graph_captures = 0
        self.graph_replays = 0
        self.graph_fallbacks: Dict[str, int] = {}     # why decode steps ran eagerly although graphs are on: reason -> count
        self.step_result: Optional[StepResult] = None

    # ---- staging ---------------------------------------------------------------
    def _pinned(self, n: int):
        if len(self._staging) < 4:
            self._staging.append([_alloc_pinned(max(n, 1 << 14)), None])
        i = self._staging_next % len(self._staging)
        self._staging_next += 1
        buf, ev = self._staging[i]
        if ev is not None:
            ev.synchronize()
        if buf.numel() < n:
            buf = _alloc_pinned(n * 2)
            self._staging[i][0] = buf
        return i, buf

    def _layout(self, B: int, T: int, R: int, max_pages: int):
        """Where each section of a step's metadata lies in the staging buffer (in ints)."""
        layout = {}
        pos = 0
        for key, n in (("tokens", T), ("tok_row", T), ("tok_pos", T), ("row_slot", B), ("row_flags", B), ("row_q_start", B),
                       ("row_q_len", B), ("row_pos_start", B), ("logit_rows", R), ("samp_temp", R), ("samp_top_p", R),
                       ("samp_pos", R), ("samp_seed", 2 * R)):
            layout[key] = (pos, n)
            pos = _align(pos + n)
        for g in self.cache.groups:
            layout["bt:" + g] = (pos, B * max_pages)
            pos = _align(pos + B * max_pages)
        return layout, pos

    def _check_rows(self, rows: List[RowInput]):
        q_lens = [len(r.tokens) for r in rows]
        wants, q_start, off, max_seq = [], [], 0, 0
        for r, n in zip(rows, q_lens):
            if n < 1:
                raise ValueError("a row of a step needs at least one token")
            if not self.cache.is_live(r.slot):
                raise ValueError(f"slot {r.slot} is not live")
            for w in r.want:
                if not (0 <= w < n):
                    raise ValueError(f"wanted place {w} lies outside the row's {n} tokens")
                wants.append(off + w)
            q_start.append(off)
            off += n
            end = r.start_pos + n
            max_seq = max(max_seq, end)
            for g in self.cache.groups.values():
                if int(g.num_logical[r.slot]) * g.page_size < end:
                    raise ValueError(f"slot {r.slot} has no pages for {end} tokens; grow it before the step")
        if len(set(r.slot for r in rows)) != len(rows):
            raise ValueError("a request appears twice in one step")
        return q_lens, q_start, wants, max_seq

    def _fill(self, host: np.ndarray, layout: dict, rows: List[RowInput], q_lens, q_start, wants, max_pages: int) -> None:
        B = len(rows)

        def put(key, values):
            a, n = layout[key]
            host[a:a + n] = values

        put("tokens", np.concatenate([np.asarray(r.tokens, dtype=np.int32) for r in rows]))
        put("tok_row", np.repeat(np.arange(B, dtype=np.int32), q_lens))
        put("tok_pos", np.concatenate([np.arange(r.start_pos, r.start_pos + n, dtype=np.int32) for r, n in zip(rows, q_lens)]))
        put("row_slot", [r.slot for r in rows])
        put("row_flags", [int(r.flags) for r in rows])
        put("row_q_start", q_start)
        put("row_q_len", q_lens)
        put("row_pos_start", [r.start_pos for r in rows])
        put("logit_rows", wants)
        if wants:
            temp, top_p, pos, seed = [], [], [], []
            for r in rows:
                sp = r.sampling
                for w in r.want:
                    temp.append(sp.temperature if sp else 0.0)
                    top_p.append(sp.top_p if sp else 1.0)
                    seed.append((sp.seed if sp else 0) & 0xFFFFFFFFFFFFFFFF)
                    pos.append(r.start_pos + w + 1)     # the position the new token will take
            put("samp_temp", np.asarray(temp, dtype=np.float32).view(np.int32))
            put("samp_top_p", np.asarray(top_p, dtype=np.float32).view(np.int32))
            put("samp_pos", pos)
            put("samp_seed", np.asarray(seed, dtype=np.uint64).view(np.int32))
        slots = [r.slot for r in rows]
        for g in self.cache.groups:
            a, n = layout["bt:" + g]
            host[a:a + n] = self.cache.groups[g].table[slots, :max_pages].reshape(-1)

    def _context(self, dev: torch.Tensor, layout: dict, rows, q_lens, q_start, wants, max_pages, max_seq,
                 replayable: bool = False) -> StepContext:
        B = len(rows)
        sections = {k: dev[a:a + n] for k, (a, n) in layout.items() if not k.startswith("bt:")}
        block_tables = {g: dev[layout["bt:" + g][0]:layout["bt:" + g][0] + B * max_pages].view(B, max_pages)
                        for g in self.cache.groups}
        info = dict(max_pages=max_pages, decode_only=all(n == 1 for n in q_lens), max_q_len=max(q_lens) if q_lens else 0, max_seq_len=max_seq,
                    rows=rows, q_lens=q_lens, q_start=q_start, wants=wants)
        return StepContext(device=self.device, dtype=self.dtype, cache=self.cache, sections=sections,
                           block_tables=block_tables, host=info, err=self.err, scratch_pool=self._scratch,
                           plain_kernels=self.plain_kernels, replayable=replayable, capture=None if replayable else self.capture,
                           max_rows=self.cfg.max_batch, max_step_tokens=self.cfg.max_tokens_per_step)

    def build_context(self, rows: List[RowInput]) -> StepContext:
        """Fills the staging buffer for these rows and copies it to the device."""
        q_lens, q_start, wants, max_seq = self._check_rows(rows)
        ps = self.cache.page_size
        max_pages = min(max(1, _align((max_seq + ps - 1) // ps)), max(1, self.cache.max_pages_per_request))
        layout, size = self._layout(len(rows), sum(q_lens), len(wants), max_pages)
        idx, pinned = self._pinned(size)
        self._fill(pinned.numpy(), layout, rows, q_lens, q_start, wants, max_pages)
        self.last_staging_bytes = size * 4
        dev = torch.empty(size, dtype=torch.int32, device=self.device)
        if self.on_device_work is not None:
            self.on_device_work()
        dev.copy_(pinned[:size], non_blocking=True)
        self._staging[idx][1] = _record_event()
        return self._context(dev, layout, rows, q_lens, q_start, wants, max_pages, max_seq)

    # ---- the step ----------------------------------------------------------------
    def step(self, rows: List[RowInput]) -> torch.Tensor:
        """Runs one batch.  Pages for the new tokens must be held already
        (``cache.grow``); afterwards the caller records the new lengths
        (``cache.advance``).  Returns float32 logits [wanted places, vocab] on the
        device, in the order of the rows and of their ``want`` lists."""
        if not rows:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        ctx = self.build_context(rows)
        logits = self.model.forward(ctx)
        self.steps_run += 1
        if self.cfg.check_kernel_errors:
            ops.raise_if_error(self.err)
        return logits

    def _sample(self, ctx: StepContext, logits: torch.Tensor) -> torch.Tensor:
        """One token per wanted place, and after them the four ints of the kernels' error
        record as the step's last kernel saw them: [R + 4] int32.  Whoever reads the tokens
        on the host gets the step's status with them, without a synchronisation of its own."""
        R = logits.shape[0]
        out = torch.empty(R + 4, dtype=torch.int32, device=self.device)
        s = ctx.sampling_sections
        ops.sample(logits, out, temperature=s["samp_temp"].view(torch.float32), top_p=s["samp_top_p"].view(torch.float32),
                   seeds=s["samp_seed"].view(torch.int64), positions=s["samp_pos"], err=self.err)
        return out

    def graph_batch(self, batch: int) -> int:
        """The batch size a decode step of ``batch`` rows is captured for: up to 8 as it is, above
        that the next of 12, 16, 24, 32, 48, 64, 96, ... (at most half as many rows again), never
        above the engine's largest batch.  So a batch that shrinks request by request, as the end
        of a wave of requests does, replays a dozen graphs instead of meeting a new size, with its
        eager runs and its capture, at every step."""
        if batch <= 8:
            return batch
        size = 8
        while size < batch:
            size = size * 3 // 2 if (size & (size - 1)) == 0 else size * 4 // 3
        return max(batch, min(size, self.cfg.max_batch))

    def decode_graph_ready(self, batch: int) -> bool:
        """True when decode steps of this many rows are replayed from a captured graph already."""
        g = self._graphs.get(self.graph_batch(batch))
        return bool(self.cfg.cuda_graph_decode and g is not None and g["graph"] is not None)

    def step_and_sample(self, rows: List[RowInput], tokens_from: Optional[torch.Tensor] = None):
        """One batch, and one new token for every wanted place (greedy, or as the row's
        ``sampling`` says).  Returns (logits, tokens), both on the device; ``step_result`` holds
        the tokens followed by the kernels' error record for a single read by the host
        (``StepResult``), and nothing here waits for the device.  A step in which
        every row brings one token is replayed from a CUDA graph when the engine was set up
        with ``cuda_graph_decode``.  ``tokens_from``: a device tensor with one token per row that
        takes the place of the rows' own tokens (the tokens the step before sampled, which the
        host has not read yet); only for steps that ``decode_graph_ready`` says are replayed."""
        if not rows:
            self.step_result = None
            return (torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device),
                    torch.empty(0, dtype=torch.int32, device=self.device))
        if self.cfg.cuda_graph_decode and all(len(r.tokens) == 1 and list(r.want) == [0] for r in rows):
            return self._graph_step(rows, tokens_from)
        if tokens_from is not None:
            raise ValueError("tokens from the device are taken by captured decode steps only")
        ctx = self.build_context(rows)
        logits = self.model.forward(ctx)
        out = self._sample(ctx, logits)
        R = logits.shape[0]
        self.step_result = StepResult(out, R, R)
        self.steps_run += 1
        return logits, out[:R]

    def check_errors(self) -> None:
        """Reads the kernels' error record (waits for the device) and raises if it is set."""
        ops.raise_if_error(self.err)

    # ---- decode steps from a CUDA graph ---------------------------------------------
    def _graph_step(self, rows: List[RowInput], tokens_from: Optional[torch.Tensor] = None):
        """Replays the recorded decode step for this batch size.  All metadata lives in one
        device buffer of fixed layout that a single copy refreshes before the replay; block
        tables have their full width and the parts are told that the step is replayable, so
        nothing in the graph depends on the step.  When recording fails, this batch size runs
        eagerly from then on and the reason is counted in ``graph_fallbacks``.
        Reference: backend.py:974-1001 (when a graph is used), 1119-1162 (two warm-up runs,
        then capture), 1138-1150 and 1174-1181 (failure: eager, with counted reasons)."""
        n_real = len(rows)
        self._check_rows(rows)
        # The step is captured for a rounded-up batch size; the spare rows decode position 0 of
        # the cache's padding slot, which belongs to no request, and their tokens are dropped.
        B = self.graph_batch(n_real)
        rows = list(rows) + [RowInput(self.cache.padding_slot, [0], 0, [0])] * (B - n_real)
        q_lens, q_start, wants = [1] * B, list(range(B)), list(range(B))
        max_pages = self.cache.max_pages_per_request
        g = self._graphs.get(B)
        if g is None:
            layout, size = self._layout(B, B, B, max_pages)
            g = dict(layout=layout, size=size, dev=torch.zeros(size, dtype=torch.int32, device=self.device), graph=None,
                     warm=0, failed=None)
            self._graphs[B] = g
        layout, size, dev = g["layout"], g["size"], g["dev"]
        idx, pinned = self._pinned(size)
        self._fill(pinned.numpy(), layout, rows, q_lens, q_start, wants, max_pages)
        self.last_staging_bytes = size * 4
        if self.on_device_work is not None:
            self.on_device_work()
        dev.copy_(pinned[:size], non_blocking=True)
        self._staging[idx][1] = _record_event()
        if tokens_from is not None:
            if g["graph"] is None:
                raise ValueError("tokens from the device are taken by captured decode steps only")
            a, _ = layout["tokens"]
            dev[a:a + n_real].copy_(tokens_from[:n_real])      # device to device, in stream order before the replay

        def run():
            ctx = self._context(dev, layout, rows, q_lens, q_start, wants, max_pages, self.cache.max_seq_len, replayable=True)
            logits = self.model.forward(ctx)
            return logits, self._sample(ctx, logits)

        if g["graph"] is None and not g["failed"] and g["warm"] >= 2:
            # two eager runs have sized the working buffers; now record the same launches
            torch.cuda.synchronize()
            l0 = ops.launch_count()
            # No garbage collection while the stream records: a collected object that frees something of
            # CUDA's (the graphs of an engine that is no longer used, say) makes calls that are not allowed
            # during a recording and would spoil it.  What is garbage now is collected before.
            gc_was_on = gc.isenabled()
            gc.collect()
            gc.disable()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    g["out"] = run()
                g["graph"] = graph
                g["launches"] = ops.launch_count() - l0     # kernels recorded, not run
                self.graph_captures += 1
            except Exception as e:  # noqa: BLE001  (whatever stops the recording: this size stays eager)
                first = (str(e).strip().splitlines() or [""])[0][:160]
                g["failed"] = f"capture failed: {type(e).__name__}: {first}"
                g["error"] = str(e)
                torch.cuda.synchronize()
            finally:
                if gc_was_on:
                    gc.enable()
            ops.count_launch(l0 - ops.launch_count())
        if g["graph"] is None:
            g["warm"] += 1
            if g["failed"]:
                self.graph_fallbacks[g["failed"]] = self.graph_fallbacks.get(g["failed"], 0) + 1
            logits, out = run()
            self.steps_run += 1
            self.step_result = StepResult(out, n_real, B)
            return logits[:n_real], out[:n_real]
        g["graph"].replay()
        ops.count_launch(g["launches"])
        self.steps_run += 1
        self.graph_replays += 1
        logits, out = g["out"]
        self.step_result = StepResult(out, n_real, B)
        return logits[:n_real], out[:n_real]

    # ---- convenience used by replay and tests --------------------------------------
    def run_rows(self, rows: List[RowInput]) -> torch.Tensor:
        """grow, step, advance for every row."""
        for r in rows:
            self.cache.grow(r.slot, r.start_pos + len(r.tokens))
        logits = self.step(rows)
        for r in rows:
            self.cache.advance(r.slot, r.start_pos + len(r.tokens))
        return logits
