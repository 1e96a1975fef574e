"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives
``ModelRunner`` (the model, step function, cache manager and kernels that
generation uses).  Input: one JSON object a line,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` are one batch; ``want`` are the places among an entry's tokens whose
logits are asked for; ``end`` names requests that are finished after the step.
For a step that wants something, ``<out>/<step>.f32`` holds the logits
[wanted, vocab] as little-endian float32 in the order of the entries and of
``want``.  After every step ``done <step>`` is printed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np

MAX_LIVE = 4
ROUND_TO = 64


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each request rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from ..config.engine_config import EngineConfig
    from ..config.registry import read_config
    from .step import ModelRunner, RowInput
    import delta_b200.models  # noqa: F401  (registers the architectures)

    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    if ROUND_TO % args.page_size:
        raise SystemExit(f"--page-size {args.page_size} must divide {ROUND_TO}")
    _, mcfg = read_config(args.model)
    max_tokens = (args.max_tokens + ROUND_TO - 1) // ROUND_TO * ROUND_TO
    max_seq = max_tokens
    limit = getattr(mcfg, "max_position_embeddings", None)
    cfg = EngineConfig(max_batch=MAX_LIVE, max_seq_len=max_seq, page_size=args.page_size,
                       num_pages=max_tokens // args.page_size, dtype=args.dtype, max_tokens_per_step=max_tokens)
    runner = ModelRunner(args.model, engine_config=cfg, device=args.device)

    slots = {}    # request id -> slot
    length = {}   # request id -> tokens held
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        rows = []
        for e in rec.get("entries", []):
            rid = e["id"]
            toks = e["tokens"]
            if not toks:
                continue
            if rid not in slots:
                slots[rid] = runner.cache.acquire_slot()
                length[rid] = 0
            rows.append(RowInput(slot=slots[rid], tokens=toks, start_pos=length[rid], want=list(e.get("want", []))))
        logits = runner.run_rows(rows)
        for r in rows:
            rid = next(k for k, v in slots.items() if v == r.slot)
            length[rid] += len(r.tokens)
        if logits.shape[0] > 0:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            arr.tofile(out / f"{step}.f32")
        for rid in rec.get("end", []):
            if rid in slots:
                runner.cache.release_slot(slots.pop(rid))
                length.pop(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
