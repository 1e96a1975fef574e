"""Shared pieces of the tests: tiny configurations, model folders, ways of cutting
a request into steps."""
from __future__ import annotations

import json
import random
from pathlib import Path

import numpy as np
import torch


def tiny_config(which: str) -> dict:
    """config.json of the tiny models.  They differ in every size and option."""
    base = dict(architectures=["LlamaForCausalLM"], hidden_act="silu", tie_word_embeddings=False, model_type="llama",
                torch_dtype="float32")
    if which == "A":
        return dict(base, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                    intermediate_size=176, vocab_size=512, rope_theta=10000.0, rms_norm_eps=1e-6,
                    max_position_embeddings=256)
    if which == "B":
        return dict(base, architectures=["YiForCausalLM"], hidden_size=128, num_hidden_layers=3, num_attention_heads=4,
                    num_key_value_heads=1, intermediate_size=344, vocab_size=1000, rope_theta=5000000.0,
                    rms_norm_eps=1e-5, max_position_embeddings=512)
    if which == "C":  # head size given apart from the width, no power of two anywhere, two layers with a window
        return dict(base, hidden_size=80, num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
                    intermediate_size=200, vocab_size=777, rope_theta=250000.0, rms_norm_eps=3e-6,
                    max_position_embeddings=384, sliding_window=24,
                    layer_types=["full_attention", "sliding_attention", "full_attention", "sliding_attention"])
    if which == "D":  # head size 64: the sizes the tensor-core attention kernels take
        return dict(base, hidden_size=192, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
                    intermediate_size=208, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
                    max_position_embeddings=512)
    raise KeyError(which)


PAGE_SIZE = {"A": 16, "B": 8, "C": 32, "D": 16}
SEED = {"A": 0, "B": 1, "C": 2, "D": 3}


def make_model_folder(tmp_path, which: str, dtype=torch.float32) -> Path:
    from delta_b200.weights import write_random_model
    import delta_b200.models  # noqa: F401
    return write_random_model(Path(tmp_path) / f"tiny_{which}", tiny_config(which), SEED[which], dtype)


def random_tokens(n: int, vocab: int, seed: int) -> list:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# ---- ways of cutting requests into steps ------------------------------------
# A schedule is a list of steps; a step is a list of (request index, start, count).

def whole(lengths):
    return [[(i, 0, n)] for i, n in enumerate(lengths)]


def last_one_by_one(lengths, tail=32):
    steps = []
    for i, n in enumerate(lengths):
        head = max(n - tail, 1) if n > 1 else n
        steps.append([(i, 0, head)])
        for p in range(head, n):
            steps.append([(i, p, 1)])
    return steps


def changing_portions(lengths, seed=0, sizes=(7, 2, 13, 2, 5, 3, 16, 2, 9)):
    steps = []
    for i, n in enumerate(lengths):
        p, j = 0, (seed + i) % len(sizes)
        while p < n:
            c = min(sizes[j % len(sizes)], n - p)
            steps.append([(i, p, c)])
            p += c
            j += 1
    return steps


def mixed(lengths, prompt_lens, seed=0, max_live=4, portion_sizes=(5, 2, 11, 3, 17, 2)):
    """Up to ``max_live`` requests at a time; prompts go in portions, then tokens one by
    one, all live requests in the same steps.  Returns (steps, ends): ends[k] lists the
    requests finished after step k."""
    rng = random.Random(seed)
    waiting = list(range(len(lengths)))
    live = {}
    steps, ends = [], []
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        step, done = [], []
        for i in list(live):
            p = live[i]
            if rng.random() < 0.15 and len(live) > 1:
                continue  # this request sits the step out
            if p < prompt_lens[i]:
                c = min(portion_sizes[rng.randrange(len(portion_sizes))], prompt_lens[i] - p)
            else:
                c = 1
            step.append((i, p, c))
            live[i] = p + c
            if live[i] >= lengths[i]:
                done.append(i)
                del live[i]
        if step:
            steps.append(step)
            ends.append(done)
    return steps, ends


# ---- running a schedule through the engine's step function -----------------------

def run_schedule(runner, token_lists, steps, ends=None, prompt_lens=None, planned=None):
    """Feeds the schedule through ``runner`` (a ModelRunner) and returns
    {(request, position): logits row (CPU float32)}.  Logits are asked for at every
    token.  With ``prompt_lens`` the single tokens at or after a request's prompt
    length are flagged as decode rows (page selection applies to those)."""
    from delta_b200.engine.step import RowInput
    from delta_b200.parts.base import ROW_DECODE
    slots = {}
    out = {}
    if planned is not None:
        runner.capture = {}
    for k, step in enumerate(steps):
        rows, keys = [], []
        for (i, start, count) in step:
            if i not in slots:
                slots[i] = runner.cache.acquire_slot()
            dec = bool(count == 1 and prompt_lens is not None and start >= prompt_lens[i])
            rows.append(RowInput(slots[i], token_lists[i][start:start + count], start, list(range(count)),
                                 flags=ROW_DECODE if dec else 0))
            keys.extend((i, start + j) for j in range(count))
        logits = runner.run_rows(rows).float().cpu()
        assert logits.shape[0] == len(keys)
        if planned is not None:
            # what the planner layers chose in this step: {(request, layer, position): pages}
            who = {s: i for i, s in slots.items()}
            for (prefix, slot, pos), pages in runner.capture.pop("planned", {}).items():
                planned[(who[slot], int(prefix.split(".")[2]), pos)] = pages
        for key, row in zip(keys, logits):
            assert key not in out, f"position {key} was fed twice"
            out[key] = row
        for i in (ends[k] if ends is not None else []):
            runner.cache.release_slot(slots.pop(i))
        runner.cache.check()
    for i in list(slots):
        runner.cache.release_slot(slots.pop(i))
    runner.cache.check()
    if planned is not None:
        runner.capture = None
    return out


def stack_positions(results, request, length):
    return torch.stack([results[(request, p)] for p in range(length)])


def peak_pages(steps, ends, page_size):
    """Most pages held at any time when the schedule runs (no windows counted)."""
    held, peak = {}, 0
    for k, step in enumerate(steps):
        for (i, start, count) in step:
            held[i] = (start + count + page_size - 1) // page_size
        peak = max(peak, sum(held.values()))
        for i in (ends[k] if ends is not None else []):
            held.pop(i, None)
    return peak
