"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives
``ModelRunner`` (the model, step function, cache manager and kernels that
generation uses).  Input: one JSON object a line,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` are one batch; ``want`` are the places among an entry's tokens whose
logits are asked for; ``end`` names requests that are finished after the step.  An
entry may carry ``"decode": true``: its single token lies at or after the end of the
request's prompt, which matters to models whose parts treat such rows in a way of
their own (DELTA's page selection applies to them only).  For a step that wants
something, ``<out>/<step>.f32`` holds the logits [wanted, vocab] as little-endian
float32 in the order of the entries and of ``want``.  After every step
``done <step>`` is printed.

The selective-cache options have the names of the generation command line
(``--enable_selective_cache --full_cache_layers --subset_cache_size --L
--compression_ratio``); ``--cuda_graph_decode`` sends steps in which every entry
brings one token and wants its logits through the recorded decode step;
``--dump-selected`` writes ``<out>/<step>.selected.json`` with the pages every
planner chose in the step (eager steps only); ``--shuffle-pages SEED`` hands pages
out in a shuffled order; ``--num-pages`` and ``--max-live`` size the pool and the
request slots (default: the pages of ``--max-tokens``, four requests).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROUND_TO = 64


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each request rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--max-live", type=int, default=4, help="request slots: the most requests that are live at a time")
    ap.add_argument("--num-pages", type=int, default=None, help="pages in the pool (default: what --max-tokens needs)")
    ap.add_argument("--shuffle-pages", type=int, default=None, metavar="SEED", help="hand pages out in a shuffled order")
    ap.add_argument("--cuda_graph_decode", action="store_true",
                    help="steps of single tokens that want their logits are replayed from a recorded CUDA graph")
    ap.add_argument("--enable_selective_cache", action="store_true")
    ap.add_argument("--full_cache_layers", nargs="+", type=int, default=None)
    ap.add_argument("--subset_cache_size", type=int, default=1024)
    ap.add_argument("--compression_ratio", type=float, default=1.0)
    ap.add_argument("--L", type=int, default=8)
    ap.add_argument("--count_page_ahead", action="store_true",
                    help="count a request's pages as the reference does: one more, empty, once the newest is exactly full")
    ap.add_argument("--dump-selected", action="store_true", help="write the pages each planner chose, per step")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)

    from ..config.engine_config import EngineConfig
    from ..config.selective_cache import SelectiveCacheConfig
    from ..parts.base import ROW_DECODE
    from .step import ModelRunner, RowInput
    import delta_b200.models  # noqa: F401  (registers the architectures)

    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    if ROUND_TO % args.page_size:
        raise SystemExit(f"--page-size {args.page_size} must divide {ROUND_TO}")
    if args.max_live < 1:
        raise SystemExit("--max-live must be at least 1")
    max_tokens = (args.max_tokens + ROUND_TO - 1) // ROUND_TO * ROUND_TO
    selective = None
    if args.enable_selective_cache and args.full_cache_layers:
        selective = SelectiveCacheConfig(full_cache_layers=tuple(args.full_cache_layers), subset_cache_size=args.subset_cache_size,
                                         compression_ratio=args.compression_ratio, L=args.L,
                                         count_page_ahead=args.count_page_ahead)
    cfg = EngineConfig(max_batch=args.max_live, max_seq_len=max_tokens, page_size=args.page_size,
                       num_pages=args.num_pages if args.num_pages is not None else max_tokens // args.page_size,
                       dtype=args.dtype, max_tokens_per_step=max_tokens, cuda_graph_decode=args.cuda_graph_decode,
                       shuffle_pages=args.shuffle_pages, options=dict(selective_cache=selective))
    runner = ModelRunner(args.model, engine_config=cfg, device=args.device)
    if args.dump_selected:
        runner.capture = {}

    slots = {}    # request id -> slot
    length = {}   # request id -> tokens held
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        rows, ids = [], []
        for e in rec.get("entries", []):
            rid = e["id"]
            toks = e["tokens"]
            if not toks:
                continue
            if rid not in slots:
                slots[rid] = runner.cache.acquire_slot()
                length[rid] = 0
            if e.get("decode") and len(toks) != 1:
                raise SystemExit(f"step {step}: entry '{rid}' is marked decode and brings {len(toks)} tokens")
            rows.append(RowInput(slot=slots[rid], tokens=toks, start_pos=length[rid], want=list(e.get("want", [])),
                                 flags=ROW_DECODE if e.get("decode") else 0))
            ids.append(rid)
        for r in rows:
            runner.cache.grow(r.slot, r.start_pos + len(r.tokens))
        if args.cuda_graph_decode and rows and all(len(r.tokens) == 1 and list(r.want) == [0] for r in rows):
            logits, _ = runner.step_and_sample(rows)
            runner.check_errors()
        else:
            logits = runner.step(rows)
        for r, rid in zip(rows, ids):
            length[rid] += len(r.tokens)
            runner.cache.advance(r.slot, length[rid])
        if logits.shape[0] > 0:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            arr.tofile(out / f"{step}.f32")
        if args.dump_selected:
            who = {s: rid for rid, s in slots.items()}
            chosen = [dict(id=who[slot], part=part, position=pos, pages=pages)
                      for (part, slot, pos), pages in sorted(runner.capture.pop("planned", {}).items())]
            if chosen:
                (out / f"{step}.selected.json").write_text(json.dumps(chosen))
        for rid in rec.get("end", []):
            if rid in slots:
                runner.cache.release_slot(slots.pop(rid))
                length.pop(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
