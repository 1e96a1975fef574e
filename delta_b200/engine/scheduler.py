"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.  It decides on the host and touches no device memory,
so it runs (and is tested) without a GPU; it books pages through the cache manager.

Reference counterpart: ``BatchScheduler`` and ``Request``
(DELTA/Engine/DELTA/scheduler.py:43-186) and the loop head of
``run_scheduler_loop`` (backend.py:1485-1553).  The reference admits a waiting
request whenever a slot is free, runs its whole prompt in that step beside
everyone's decode token, and sizes the pool so that it can never run out
(backend.py:253-254).  Here:

  * every step has a token budget: decode tokens first (one each), the rest goes to
    prompt portions, oldest request first;
  * a waiting request is admitted when a slot is free and every cache group can hold
    its whole prompt and one more token, beside what the step already promised;
  * when a running request cannot grow, the youngest running request is preempted:
    its pages are given back, it returns to the head of the queue and what it had
    computed is computed again once it is admitted again; a request that could not
    fit even alone fails.  What is computed again gives the logits of the first time:
    when the model treats decode rows like any other (``decode_singly`` False) prompt
    and generated tokens run as one prompt; when some part treats them otherwise (page
    selection applies to decode rows only) the prompt runs in portions and every
    generated token again as a decode row of its own, one per step, unsampled.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from ..sampling.sampler import SamplingParams

WAITING, RUNNING, FINISHED, FAILED = "waiting", "running", "finished", "failed"


@dataclass
class Request:
    id: int
    prompt: List[int]
    max_length: int                      # prompt + generated tokens (the reference's ``max_length``)
    stop_ids: Sequence[int] = ()
    sampling: SamplingParams = SamplingParams()
    max_new_tokens: Optional[int] = None
    status: str = WAITING
    output: List[int] = field(default_factory=list)
    slot: int = -1
    computed: int = 0                    # tokens of prompt + output that are in the cache
    admitted_order: int = -1
    preemptions: int = 0
    start_time: Optional[float] = None
    end_time: Optional[float] = None
    finish_reason: str = ""

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)

    def is_finished(self) -> bool:
        return self.status in (FINISHED, FAILED)


@dataclass
class PlannedRow:
    request: Request
    start: int          # position of the first token of this share
    count: int
    samples: bool       # the last token of the share yields a new token
    decode: bool        # a single token at or after the prompt's end (a decode row; ``samples`` False: one that is computed again)


class Scheduler:
    def __init__(self, cache, *, max_batch: int, max_tokens_per_step: int, decode_singly: bool = False, clock=time.perf_counter):
        self.cache = cache
        self.max_batch = int(max_batch)
        self.budget = int(max_tokens_per_step)
        # True: tokens at or after a prompt's end never run inside a prompt portion (see the module text)
        self.decode_singly = bool(decode_singly)
        self.clock = clock
        self.requests: List[Request] = []
        self.waiting: List[Request] = []
        self.running: List[Request] = []
        self._admitted = 0
        # False: no request decodes while another still has prompt tokens to run (prompts first)
        self.decode_while_prefill = True
        self.stats = dict(prompt_tokens=0, generated_tokens=0, steps=0, prefill_steps=0, decode_steps=0, preemptions=0)

    # ---- intake ------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], max_length: int, stop_ids: Sequence[int] = (),
                    sampling: Optional[SamplingParams] = None, max_new_tokens: Optional[int] = None) -> Request:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        r = Request(id=len(self.requests), prompt=prompt, max_length=int(max_length), stop_ids=tuple(stop_ids),
                    sampling=sampling or SamplingParams(), max_new_tokens=max_new_tokens)
        self.requests.append(r)
        limit = min(max(r.max_length, len(prompt)), self.cache.max_seq_len)
        if len(prompt) > self.cache.max_seq_len:
            self._fail(r, f"prompt of {len(prompt)} tokens is above the engine's limit of {self.cache.max_seq_len}")
        elif not self._fits_alone(limit):
            self._fail(r, f"{limit} tokens need more cache pages than the pool has")
        else:
            self.waiting.append(r)
        return r

    def _fits_alone(self, n_tokens: int) -> bool:
        for g in self.cache.groups.values():
            pages = (n_tokens + g.page_size - 1) // g.page_size
            if g.spec.window:
                # a windowed group keeps the window and what one step adds to it
                pages = min(pages, (g.spec.window + self.budget + g.page_size - 1) // g.page_size + 1)
            if pages > g.pool.num_pages:
                return False
        return True

    def _fail(self, r: Request, why: str) -> None:
        r.status, r.finish_reason = FAILED, why
        r.end_time = self.clock()
        if r.start_time is None:
            r.start_time = r.end_time

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step's plan -------------------------------------------------------
    def schedule(self) -> List[PlannedRow]:
        """Chooses what runs in the next step and books the pages for it."""
        budget = self.budget
        rows: List[PlannedRow] = []
        # 1. one token for every request that is decoding (or computing a decode position again)
        # With prompts first, decoding waits only while a prompt is really under way or about to be: a
        # waiting request that cannot be admitted (no slot, no pages) must not stop those that can end.
        hold = (not self.decode_while_prefill) and (
            any(q.computed < q.total_len - 1 for q in self.running)
            or bool(self.waiting and len(self.running) < self.max_batch and self.cache.free_slots > 0
                    and self._can_admit(self.waiting[0])))
        for r in sorted(self.running, key=lambda q: q.admitted_order):
            last = r.computed == r.total_len - 1
            if hold and last and r.output:
                continue
            again = self.decode_singly and len(r.prompt) <= r.computed < r.total_len - 1
            if r.status != RUNNING or not (last or again) or budget < 1:
                continue
            if not self._grow_or_preempt(r, r.computed + 1, protect=[x.request for x in rows]):
                continue
            rows.append(PlannedRow(r, r.computed, 1, samples=last, decode=r.computed >= len(r.prompt)))
            budget -= 1
        # 2. portions of prompts that are under way (after a preemption a prompt includes what was
        #    generated, unless decode positions run singly)
        for r in sorted(self.running, key=lambda q: q.admitted_order):
            if r.status != RUNNING or budget < 1 or any(x.request is r for x in rows):
                continue
            left = self._portion_end(r) - r.computed
            if left < 1 or r.computed == r.total_len - 1:
                continue
            count = min(left, budget)
            if not self._grow_or_preempt(r, r.computed + count, protect=[x.request for x in rows]):
                continue
            rows.append(PlannedRow(r, r.computed, count, samples=(r.computed + count == r.total_len), decode=False))
            budget -= count
        # 3. admit waiting requests, oldest first
        while self.waiting and budget >= 1 and len(self.running) < self.max_batch and self.cache.free_slots > 0:
            r = self.waiting[0]
            if not self._can_admit(r):
                break
            self.waiting.pop(0)
            r.slot = self.cache.acquire_slot()
            r.status = RUNNING
            r.computed = 0
            r.admitted_order = self._admitted
            self._admitted += 1
            if r.start_time is None:
                r.start_time = self.clock()
            self.running.append(r)
            count = min(self._portion_end(r), budget)
            self.cache.grow(r.slot, count)
            rows.append(PlannedRow(r, 0, count, samples=(count == r.total_len), decode=False))
            budget -= count
        return rows

    def _portion_end(self, r: Request) -> int:
        """Where the tokens end that may run as prompt portions."""
        return len(r.prompt) if self.decode_singly else r.total_len

    def _can_admit(self, r: Request) -> bool:
        """Room for the whole prompt and one more token in every group."""
        need_len = r.total_len + 1
        for g in self.cache.groups.values():
            pages = (need_len + g.page_size - 1) // g.page_size
            if g.spec.window:
                pages = min(pages, (g.spec.window + min(self.budget, need_len) + g.page_size - 1) // g.page_size + 1)
            if pages > g.pool.free_pages:
                return False
        return True

    def _grow_or_preempt(self, r: Request, new_len: int, protect: List[Request]) -> bool:
        """Books pages for ``r`` to hold ``new_len`` tokens, preempting the youngest running
        requests (never ``r`` itself nor those already planned) while the pool is short."""
        from ..cache.page_pool import OutOfPages
        while True:
            try:
                self.cache.grow(r.slot, new_len)
                return True
            except OutOfPages:
                victims = [q for q in self.running if q is not r and q not in protect and q.status == RUNNING]
                if not victims:
                    if len([q for q in self.running if q.status == RUNNING]) == 1 and not protect:
                        self._release(r)
                        self._fail(r, "out of cache pages although it runs alone")
                    return False
                self._preempt(max(victims, key=lambda q: q.admitted_order))

    def _preempt(self, r: Request) -> None:
        self._release(r)
        r.status = WAITING
        r.computed = 0
        r.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.insert(0, r)

    def _release(self, r: Request) -> None:
        if r.slot >= 0:
            self.cache.release_slot(r.slot)
            r.slot = -1
        if r in self.running:
            self.running.remove(r)

    # ---- after the step ------------------------------------------------------------
    def complete(self, rows: List[PlannedRow], new_tokens: Sequence[int]) -> List[Request]:
        """Books the step's result: ``new_tokens`` holds one token for every row with
        ``samples`` set, in order.  Returns the requests that finished."""
        finished = []
        it = iter(new_tokens)
        self.stats["steps"] += 1
        self.stats["decode_steps" if all(x.decode for x in rows) else "prefill_steps"] += 1
        for x in rows:
            r = x.request
            r.computed = x.start + x.count
            self.cache.advance(r.slot, r.computed)
            if not x.decode:
                self.stats["prompt_tokens"] += x.count
            if not x.samples:
                continue
            tok = int(next(it))
            r.output.append(tok)
            self.stats["generated_tokens"] += 1
            reason = ""
            if tok in r.stop_ids:
                reason = "stop token"
            elif r.total_len >= r.max_length or r.total_len >= self.cache.max_seq_len:
                reason = "length"
            elif r.max_new_tokens is not None and len(r.output) >= r.max_new_tokens:
                reason = "max_new_tokens"
            if reason:
                r.status, r.finish_reason = FINISHED, reason
                r.end_time = self.clock()
                self._release(r)
                finished.append(r)
        return finished

    def abort_all(self, reason: str = "aborted") -> None:
        """Finishes everything that runs or waits (the reference's throughput mode stops the
        loop at the first finished request, backend.py:1501-1505, 1555-1563)."""
        for r in list(self.running):
            r.status, r.finish_reason = FINISHED, reason
            r.end_time = self.clock()
            self._release(r)
        for r in list(self.waiting):
            r.status, r.finish_reason = FINISHED, reason
            r.end_time = r.start_time = self.clock()
        self.waiting.clear()

    def results(self) -> List[dict]:
        """Per-request results in the reference's shape (scheduler.py:158-186)."""
        out = []
        for r in self.requests:
            if not r.is_finished():
                continue
            total = (r.end_time - r.start_time) if (r.end_time and r.start_time) else 0.0
            out.append(dict(request_id=r.id, status=r.status, finish_reason=r.finish_reason, input_length=len(r.prompt),
                            output_length=len(r.output), tokens_generated=len(r.output), total_time=total,
                            tokens_per_second=len(r.output) / total if total > 0 else 0.0,
                            preemptions=r.preemptions, output_ids=list(r.output)))
        return out
