#!/usr/bin/env python3
"""Runs the unmodified hoenza/DELTA engine on the bench's decode workload and prints one JSON line.

The reference tree is used as it is, from ``baseline/_ref`` (a plain copy: the project has no
setup.py, ``PYTHONPATH`` is how its own scripts find it, tests/reasoni.py:13).  Nothing of
delta_b200 is imported here.  The stock path of tests/reasoni.py:320-342, 449-455 is driven:

    LMBackend(dtype, device, cuda_graph_decode=..., **FINAL_DELTA_BACKEND_CONFIG)
    load_model(<dir named after the config>/model.pth) -> setup_caches -> add_requests -> run_scheduler_loop

The reference reads a converted ``model.pth`` whose parent folder names the configuration
(DELTA/Engine/utils.py:209-223); a random one with the reference's tensor names is written to a
temporary folder named ``Yi-1.5-6b`` and removed afterwards.  Its own per-step CUDA-event records
(backend.py:1522-1533) give the time of the decode steps.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import sys
import tempfile
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"

SHAPES = {  # folder name the reference's table knows -> sizes (DELTA/Engine/DELTA/model.py:87-88)
    "yi-6b": ("Yi-1.5-6b", dict(n_layer=32, dim=4096, n_head=32, n_local_heads=4, intermediate_size=11008, vocab_size=64000)),
    "yi-34b": ("Yi-1.5-34b-32k", dict(n_layer=60, dim=7168, n_head=56, n_local_heads=8, intermediate_size=20480, vocab_size=64000)),
}


def say(msg: str) -> None:
    print(f"[reference arm] {msg}", file=sys.stderr, flush=True)


def write_checkpoint(folder: Path, s: dict, seed: int = 0) -> Path:
    """A random checkpoint with the reference's tensor names (model.py:134-137, 333-336, 369-370, 498-500)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    d, hd = s["dim"], s["dim"] // s["n_head"]

    def normal(*shape):
        return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16).cpu()

    sd = {"tok_embeddings.weight": normal(s["vocab_size"], d), "norm.weight": torch.ones(d, dtype=torch.bfloat16),
          "output.weight": normal(s["vocab_size"], d)}
    for i in range(s["n_layer"]):
        p = f"layers.{i}."
        sd[p + "attention.wq.weight"] = normal(s["n_head"] * hd, d)
        sd[p + "attention.wk.weight"] = normal(s["n_local_heads"] * hd, d)
        sd[p + "attention.wv.weight"] = normal(s["n_local_heads"] * hd, d)
        sd[p + "attention.wo.weight"] = normal(d, d)
        sd[p + "feed_forward.w1.weight"] = normal(s["intermediate_size"], d)
        sd[p + "feed_forward.w3.weight"] = normal(s["intermediate_size"], d)
        sd[p + "feed_forward.w2.weight"] = normal(d, s["intermediate_size"])
        sd[p + "attention_norm.weight"] = torch.ones(d, dtype=torch.bfloat16)
        sd[p + "ffn_norm.weight"] = torch.ones(d, dtype=torch.bfloat16)
    folder.mkdir(parents=True, exist_ok=True)
    path = folder / "model.pth"
    torch.save(sd, str(path))
    return path


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--shape", choices=sorted(SHAPES), default="yi-6b")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--enable_selective_cache", action="store_true")
    ap.add_argument("--full_cache_layers", nargs="+", type=int, default=None)
    ap.add_argument("--subset_cache_size", type=int, default=64)
    args = ap.parse_args()
    if not (REF / "DELTA" / "Engine" / "DELTA" / "backend.py").is_file():
        print(json.dumps({"impl": "reference", "unavailable": "no copy of the reference under baseline/_ref"}))
        return 0
    sys.path.insert(0, str(REF))
    os.chdir(tempfile.gettempdir())        # the reference writes logs/step_timings_*.json into the working folder
    import torch
    folder_name, sizes = SHAPES[args.shape]
    work = Path(tempfile.mkdtemp(prefix="delta_ref_"))
    try:
        t0 = time.time()
        say(f"writing a random checkpoint for {folder_name} to {work}")
        ckpt = write_checkpoint(work / folder_name, sizes)
        say(f"checkpoint written in {time.time() - t0:.0f} s; importing the reference")
        from DELTA.Engine.DELTA.backend import LMBackend
        from DELTA.Engine.DELTA.public_config import FINAL_PUBLIC_DELTA_BACKEND_CONFIG
        from DELTA.Engine.utils import setup_seed
        setup_seed(123)
        eng = LMBackend(dtype=torch.bfloat16, device="cuda:0", cuda_graph_decode=not args.no_graph,
                        **dict(FINAL_PUBLIC_DELTA_BACKEND_CONFIG))
        eng.is_main_process = True
        eng.load_model(ckpt, use_tp=False, rank_group=[0], group=None)
        ckpt.unlink()
        c = eng.model.config
        c.enable_selective_cache = bool(args.enable_selective_cache)
        c.page_selector_version = FINAL_PUBLIC_DELTA_BACKEND_CONFIG["page_selector_version"]
        c.page_selector_v2 = True
        if args.full_cache_layers is not None:
            c.full_cache_layers = sorted(set(args.full_cache_layers))
            c.subset_cache_ratio, c.compression_ratio, c.subset_cache_size, c.L = 0.5, 1.0, args.subset_cache_size, 8
        eng.throughput_mode = True
        eng.setup_caches(max_batch_size=args.batch, max_seq_length=args.context)
        say(f"engine set up in {time.time() - t0:.0f} s")
        n_decode = args.warmup + args.steps
        plen = args.context - n_decode - 1
        gen = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, sizes["vocab_size"], (plen,), generator=gen) for _ in range(args.batch)]
        eng.add_requests(prompts, [args.context] * args.batch, [])
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        eng.run_scheduler_loop()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - w0) * 1e3
        recs = list(eng._step_records)
        decode = [r for r in recs[1:] if r["active_bsz"] == args.batch]     # the first step runs the prompts
        timed = decode[args.warmup:args.warmup + args.steps]
        if len(timed) < args.steps:
            raise RuntimeError(f"the reference recorded {len(decode)} decode steps, {args.warmup + args.steps} were expected")
        total = sum(r["step_total_ms"] for r in timed)
        untimed = sum(r["step_total_ms"] for r in recs if r not in timed)
        ms = total / len(timed)
        e2e_ms = max(wall_ms - untimed, total) / len(timed)
        out = {"impl": "reference", "metric": f"decode tok/s (Yi-6B shape, bf16, batch {args.batch}, context {args.context})",
               "value": args.batch / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": len(timed), "warmup": args.warmup,
               "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
               "data": "synthetic (random weights N(0,0.02), random token ids)",
               "config": {"model": folder_name, "layers": sizes["n_layer"], "global_batch": args.batch, "seq_len": args.context,
                          "cuda_graph_decode": not args.no_graph, "selective_cache": bool(args.enable_selective_cache),
                          "timing": "the reference's own per-step CUDA events (step_total)"},
               "e2e": {"value": args.batch / (e2e_ms / 1e3), "unit": "tokens/s",
                       "how": "wall clock of run_scheduler_loop minus the event time of the untimed steps"},
               "model_forward_ms": sum(r["model_forward_ms"] for r in timed) / len(timed)}
        print(json.dumps(out))
        return 0
    finally:
        shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    sys.exit(main())
