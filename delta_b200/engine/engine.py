"""The Python entry point, in the manner of the reference's ``LMBackend``.

The reference is used like this (tests/reasoni.py:320-342, 449-455):

    e = LMBackend(dtype=torch.bfloat16, device="cuda:0", cuda_graph_decode=...)
    e.load_model(path)
    e.model.config.enable_selective_cache = ...   # and full_cache_layers, subset_cache_size, ...
    e.setup_caches(max_batch_size=B, max_seq_length=max_len)
    e.add_requests(list_of_id_tensors, max_lengths, eot_token_ids)
    results = e.run_scheduler_loop()

The same calls work here.  ``load_model`` takes a model folder (config.json and
safetensors) instead of a converted ``model.pth``; the selective-cache options are
arguments of ``setup_caches`` (or attributes of ``options`` set before it).
Results have the reference's keys (scheduler.py:166-182) plus the generated ids.
"""
from __future__ import annotations

import json
import time
from pathlib import Path
from types import SimpleNamespace
from typing import List, Optional, Sequence

import torch

from ..config.engine_config import EngineConfig
from ..config.selective_cache import SelectiveCacheConfig
from ..kernels import ops
from ..parts.base import ROW_DECODE
from ..sampling.sampler import SamplingParams
from .scheduler import PlannedRow, Scheduler
from .step import ModelRunner, RowInput, StepResult


class LMBackend:
    def __init__(self, dtype=torch.bfloat16, device: str = "cuda:0", cuda_graph_decode: bool = False, **unused):
        if dtype in (torch.bfloat16, "bfloat16", "bf16"):
            self.dtype = "bfloat16"
        elif dtype in (torch.float32, "float32", "fp32"):
            self.dtype = "float32"
        else:
            raise ValueError(f"dtype {dtype} is not supported: bfloat16 or float32")
        self.device = device
        self.cuda_graph_decode = bool(cuda_graph_decode)
        # the reference's scripts set these on model.config; here they are plain options
        self.options = SimpleNamespace(enable_selective_cache=False, full_cache_layers=None, subset_cache_size=1024,
                                       compression_ratio=1.0, L=8, count_page_ahead=False)
        self._model_dir = None
        self._config_json = None
        self._seed = None
        self.runner: Optional[ModelRunner] = None
        self.scheduler: Optional[Scheduler] = None
        self.tokenizer = None
        self.step_timings: List[dict] = []
        self.throughput_mode = False
        self._host_tokens = [None, None]
        self._read_turn = 0
        self.record_timings = False
        # Decode steps are launched one step ahead of the host: while the host waits for the tokens
        # of step N, step N + 1 already runs with those tokens taken on the device.  See _run_ahead.
        self.run_ahead = True
        self._ahead = None
        # called as on_step_logits(plan, logits) after every step, with the float32 logits [sampled rows, vocab]
        # on the device in the order of the plan's sampling rows; while it is set no step is launched ahead
        self.on_step_logits = None

    # ---- set-up -------------------------------------------------------------
    def load_model(self, model_dir=None, *, config_json: Optional[dict] = None, seed: Optional[int] = None, **unused):
        """Names the model: a folder, or a config.json dict with a seed for random weights.
        The weights are read when the caches are set up."""
        if model_dir is None and config_json is None:
            raise ValueError("give a model folder or config_json with a seed")
        self._model_dir, self._config_json, self._seed = model_dir, config_json, seed

    def set_tokenizer(self, tokenizer):
        self.tokenizer = tokenizer

    def setup_caches(self, max_batch_size: int = 1, max_seq_length: int = 2048, *, page_size: int = 16,
                     num_pages: Optional[int] = None, max_tokens_per_step: int = 2048,
                     enable_selective_cache: Optional[bool] = None, full_cache_layers=None,
                     subset_cache_size: Optional[int] = None, compression_ratio: Optional[float] = None,
                     L: Optional[int] = None, count_page_ahead: Optional[bool] = None, check_kernel_errors: bool = True, rope_interleaved: bool = False,
                     shuffle_pages: Optional[int] = None, page_runs: bool = True):
        """``check_kernel_errors``: the kernels' error record (a bad page id, token id or position
        that a kernel skipped, a wait inside a kernel that ran out) travels to the host with every
        step's tokens and raises there; this costs no synchronisation."""
        o = self.options
        if enable_selective_cache is not None:
            o.enable_selective_cache = enable_selective_cache
        if full_cache_layers is not None:
            o.full_cache_layers = full_cache_layers
        if subset_cache_size is not None:
            o.subset_cache_size = subset_cache_size
        if compression_ratio is not None:
            o.compression_ratio = compression_ratio
        if L is not None:
            o.L = L
        if count_page_ahead is not None:
            o.count_page_ahead = count_page_ahead
        selective = None
        if o.enable_selective_cache and o.full_cache_layers:
            selective = SelectiveCacheConfig(full_cache_layers=tuple(o.full_cache_layers), subset_cache_size=o.subset_cache_size,
                                             compression_ratio=float(o.compression_ratio), L=o.L,
                                             count_page_ahead=bool(o.count_page_ahead))
        cfg = EngineConfig(max_batch=max_batch_size, max_seq_len=max_seq_length, page_size=page_size, num_pages=num_pages,
                           dtype=self.dtype, max_tokens_per_step=max_tokens_per_step,
                           cuda_graph_decode=self.cuda_graph_decode, check_kernel_errors=check_kernel_errors,
                           shuffle_pages=shuffle_pages, page_runs=page_runs,
                           options=dict(selective_cache=selective, rope_interleaved=rope_interleaved))
        self.engine_config = cfg
        self.runner = ModelRunner(self._model_dir, engine_config=cfg, config_json=self._config_json, seed=self._seed,
                                  device=self.device)
        self.scheduler = Scheduler(self.runner.cache, max_batch=max_batch_size, max_tokens_per_step=max_tokens_per_step,
                                   decode_singly=self.runner.model.decode_rows_differ())

    # ---- requests ---------------------------------------------------------------
    def add_requests(self, input_ids_list, max_lengths, eot_token_ids: Sequence[int] = (), *, temperature=0.0, top_p=1.0,
                     seed: int = 0, max_new_tokens: Optional[int] = None):
        """One request per prompt (lists or 1-D tensors of token ids).  ``max_lengths`` is a
        number or a list: the most tokens a request may reach, prompt included."""
        out = []
        for i, ids in enumerate(input_ids_list):
            ids = ids.tolist() if hasattr(ids, "tolist") else list(ids)
            ml = max_lengths[i] if isinstance(max_lengths, (list, tuple)) else max_lengths
            t = temperature[i] if isinstance(temperature, (list, tuple)) else temperature
            sp = SamplingParams(temperature=float(t), top_p=float(top_p), seed=int(seed) + len(self.scheduler.requests))
            out.append(self.scheduler.add_request(ids, ml, eot_token_ids, sp, max_new_tokens))
        return out

    # ---- the loop -----------------------------------------------------------------
    def step(self) -> List:
        """One scheduler step: plan, run, sample, book.  Returns the requests that finished.

        With ``record_timings`` every step is timed and the device is waited for at its end (so no
        step is launched ahead of the host); the record has the reference's five names
        (backend.py:1522-1533): ``collect_pages`` the host's filling of the staging block (block
        tables, positions, sampling parameters), ``plan`` the scheduler's decisions and page
        bookkeeping, ``model_forward`` the device time from the staging copy to the sampled tokens,
        ``postprocess`` asking for the tokens on the host, ``step_total`` the wall clock of the step."""
        sch, runner = self.scheduler, self.runner
        t0 = time.perf_counter()
        plan = sch.schedule()
        t_plan = time.perf_counter()
        if not plan:
            self._ahead = None
            if sch.has_work() and not sch.running:
                # nothing runs and the head of the queue cannot be admitted: it never will be
                r = sch.waiting.pop(0)
                sch._fail(r, "cannot be admitted: not enough cache pages")
                return [r]
            return []
        ahead, self._ahead = self._ahead, None
        reuse = None if (ahead is None or self.record_timings or self.on_step_logits) else self._match_ahead(plan, ahead)
        ev = None
        t_staged = t_plan
        if reuse is not None:
            # this step was launched while the host waited for the step before: only its result is read
            result, read = ahead["result"], ahead["read"]
        else:
            rows = []
            for x in plan:
                r = x.request
                toks = r.tokens[x.start:x.start + x.count]
                rows.append(RowInput(r.slot, toks, x.start, [x.count - 1] if x.samples else [],
                                     flags=ROW_DECODE if x.decode else 0, sampling=r.sampling))
            if self.record_timings:
                # the first event is recorded when the host has filled the staging buffer, right before
                # the step's first copy, so that the device time holds no wait for the host
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                staged = []

                def on_device_work():
                    staged.append(time.perf_counter())
                    ev[0].record()
                runner.on_device_work = on_device_work
            logits, _ = runner.step_and_sample(rows)
            runner.on_device_work = None
            if self.on_step_logits is not None:
                self.on_step_logits(plan, logits)
            result = runner.step_result
            if ev:
                t_staged = staged[0] if staged else t_plan
                ev[1].record()
            read = self._start_read(result)
            if ev:
                ev[2].record()      # after the copy to the host is asked for, before the host waits for it
        if reuse is None or reuse == list(range(len(ahead["rows"]))):
            self._run_ahead(plan, result)
        new_tokens = self._finish_read(read)
        if reuse is not None:
            new_tokens = [new_tokens[i] for i in reuse]
        if ev:
            torch.cuda.synchronize()
            self.step_timings.append(dict(step=len(self.step_timings) + 1, collect_pages_ms=(t_staged - t_plan) * 1e3,
                                          plan_ms=(t_plan - t0) * 1e3, model_forward_ms=ev[0].elapsed_time(ev[1]),
                                          postprocess_ms=ev[1].elapsed_time(ev[2]),
                                          step_total_ms=(time.perf_counter() - t0) * 1e3,
                                          active_bsz=len(plan), tokens=sum(x.count for x in plan),
                                          total_pages=sum(runner.cache.pages_in_use().values())))
        return sch.complete(plan, new_tokens)

    def _start_read(self, result: Optional[StepResult]):
        """Starts the device-to-host read of a step's result, through pinned memory (two buffers
        in turns: the read of the step that runs ahead is started before this one is finished).
        The kernels' error record comes with the tokens."""
        if result is None:
            return None
        n = result.tensor.shape[0]
        self._read_turn ^= 1
        buf = self._host_tokens[self._read_turn]
        if buf is None or buf.numel() < n:
            buf = self._host_tokens[self._read_turn] = torch.empty(max(n, 256), dtype=torch.int32, pin_memory=True)
        buf[:n].copy_(result.tensor, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return buf, done, result

    def _finish_read(self, read) -> List[int]:
        if read is None:
            return []
        buf, done, result = read
        done.synchronize()      # waits for this step only, not for the one launched after it
        if self.engine_config.check_kernel_errors:
            code, a, b, c = buf[result.status_at:result.status_at + 4].tolist()
            if code != 0:
                self._ahead = None
                torch.cuda.synchronize()
                self.runner.err.zero_()
                raise ops.KernelError(ops.error_text(code, a, b, c))
        return buf[:result.n_tokens].tolist()

    def _run_ahead(self, plan, result: Optional[StepResult]) -> None:
        """Launches the next decode step before the host has read this one's tokens.

        Only when the next step is certain but for stop tokens: every row of this step decodes one
        token and cannot reach a length limit with it, nothing waits for admission, decode steps of
        this size are replayed from a graph, and the pool has the pages.  The rows take their
        tokens from this step's result on the device.  If the next plan turns out otherwise (a
        request stopped, one was added), ``step`` drops what was launched here and runs the plan:
        the launched step wrote keys and values only at positions the plan writes again, with the
        same values."""
        from ..cache.page_pool import OutOfPages
        sch, runner = self.scheduler, self.runner
        if not (self.run_ahead and self.cuda_graph_decode) or self.record_timings or self.on_step_logits or sch.waiting or not plan or result is None:
            return
        if not runner.decode_graph_ready(len(plan)):
            return
        limit = runner.cache.max_seq_len
        for x in plan:
            r = x.request
            if x.count != 1 or not x.samples or x.start + 1 < len(r.prompt):
                return
            after = x.start + 2          # tokens the request holds once this step's token is appended
            if after >= min(r.max_length, limit):
                return
            if r.max_new_tokens is not None and len(r.output) + 1 >= r.max_new_tokens:
                return
        try:
            for x in plan:
                runner.cache.grow(x.request.slot, x.start + 2)
        except OutOfPages:
            return
        rows = [RowInput(x.request.slot, [0], x.start + 1, [0], flags=ROW_DECODE, sampling=x.request.sampling) for x in plan]
        runner.step_and_sample(rows, tokens_from=result.tensor)
        nxt = runner.step_result
        self._ahead = dict(rows=[(x.request.slot, x.start + 1) for x in plan], result=nxt, read=self._start_read(nxt))

    @staticmethod
    def _match_ahead(plan, ahead) -> Optional[List[int]]:
        """For every row of the plan its place in the step that was launched ahead, when the plan
        is that step or that step without some of its rows; else None."""
        where = {key: i for i, key in enumerate(ahead["rows"])}
        out = []
        for x in plan:
            i = where.get((x.request.slot, x.start))
            if i is None or x.count != 1 or not x.samples or (out and i <= out[-1]):
                return None
            out.append(i)
        return out

    def run_scheduler_loop(self) -> List[dict]:
        """Runs until every request is finished (or, in throughput mode, until the first one
        is: reference backend.py:1501-1505) and returns the per-request results."""
        sch = self.scheduler
        self.loop_start = time.perf_counter()
        while sch.has_work():
            finished = self.step()
            if self.throughput_mode and finished:
                sch.abort_all("throughput mode: first request finished")
                break
        torch.cuda.synchronize()
        self.loop_time = time.perf_counter() - self.loop_start
        if self.engine_config.check_kernel_errors:
            self.runner.check_errors()
        return self.get_detailed_results()

    def save_step_timings(self, folder="logs", meta: Optional[dict] = None) -> Optional[Path]:
        """Writes the per-step records of a run with ``record_timings`` to
        ``<folder>/step_timings_<time>.json`` as {"meta": ..., "steps": [...]}, the reference's file
        (backend.py:2240-2285).  Returns the path, or None when nothing was recorded."""
        if not self.step_timings:
            return None
        folder = Path(folder)
        folder.mkdir(parents=True, exist_ok=True)
        path = folder / f"step_timings_{time.strftime('%Y%m%d_%H%M%S')}.json"
        names = ["collect_pages", "plan", "model_forward", "postprocess", "step_total"]
        n = len(self.step_timings)
        summary = {k: dict(avg_ms=sum(r[k + "_ms"] for r in self.step_timings) / n,
                           total_ms=sum(r[k + "_ms"] for r in self.step_timings)) for k in names}
        cfg = self.engine_config
        info = dict(steps=n, dtype=cfg.dtype, max_batch=cfg.max_batch, max_seq_len=cfg.max_seq_len, page_size=cfg.page_size,
                    cuda_graph_decode=cfg.cuda_graph_decode, selective_cache=cfg.option("selective_cache") is not None,
                    graph_captures=self.runner.graph_captures, graph_replays=self.runner.graph_replays,
                    graph_fallbacks=dict(self.runner.graph_fallbacks), summary=summary)
        info.update(meta or {})
        path.write_text(json.dumps({"meta": info, "steps": self.step_timings}, indent=2))
        return path

    def get_detailed_results(self) -> List[dict]:
        res = self.scheduler.results()
        if self.tokenizer is not None:
            for r in res:
                req = self.scheduler.requests[r["request_id"]]
                r["input_text"] = self.tokenizer.decode(req.prompt, skip_special_tokens=True)
                r["output_text"] = self.tokenizer.decode(req.output, skip_special_tokens=True)
        return res

    # ---- convenience -----------------------------------------------------------------
    def generate(self, prompts, max_new_tokens: int, *, temperature=0.0, top_p=1.0, seed=0, stop_ids=()) -> List[List[int]]:
        """Token ids in, generated token ids out (host lists)."""
        first = len(self.scheduler.requests)
        limit = self.engine_config.max_seq_len
        self.add_requests(prompts, [min(limit, len(p) + max_new_tokens) for p in prompts], stop_ids, temperature=temperature,
                          top_p=top_p, seed=seed, max_new_tokens=max_new_tokens)
        self.run_scheduler_loop()
        return [list(r.output) for r in self.scheduler.requests[first:]]
