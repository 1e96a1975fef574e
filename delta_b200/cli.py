"""Command line in the manner of the reference's ``tests/reasoni.py``.

Options that the reference has keep their names and meanings
(tests/reasoni.py:226-263, reason_backend_utils.py:8-13): ``--model``, ``--B``,
``--max_len``, ``--seed``, ``--cuda_graph_decode``, ``--enable_selective_cache``,
``--full_cache_layers``, ``--subset_cache_size``, ``--compression_ratio``, ``--L``,
``--dataset`` (the synthetic ``dummy1tok`` / ``dummy4tok`` prompts of
tests/reasoni.py:70-121; the reasoning datasets are not part of this engine),
``--num_samples``, ``--dummy_token_id``, ``--printoutput``.  ``--model`` names a
model folder (config.json and safetensors) instead of a converted ``model.pth``.
Added: ``--random_weights SEED`` with ``--config`` for a model without a folder,
``--prompt_len``, ``--max_new_tokens``, ``--temperature``, ``--top_p``, ``--dtype``,
``--page_size``, ``--max_tokens_per_step``, ``--throughput_mode``, ``--out``,
``--step_timings`` (time every step with CUDA events, as the reference always does, and
write ``logs/step_timings_<time>.json``; without it the loop never waits for the device
except to read tokens, and launches decode steps ahead of the host), ``--tuning_file``
(save and reuse the measured choice of product kernels).

Example:
    python -m delta_b200.cli --model /models/Yi-1.5-6B --B 64 --max_len 4096 \\
        --dataset dummy4tok --num_samples 64 --cuda_graph_decode \\
        --enable_selective_cache --full_cache_layers 0 1 2 14 22 --subset_cache_size 64
"""
from __future__ import annotations

import argparse
import json
import random
import sys
import time
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="delta_b200", description="Generate with the delta_b200 engine.")
    p.add_argument("--model", type=Path, default=None, help="model folder (config.json + safetensors)")
    p.add_argument("--model_name", type=str, default=None, help="name or folder of the tokenizer (optional)")
    p.add_argument("--B", type=int, default=16, help="request slots: the most requests that run at a time")
    p.add_argument("--max_len", type=int, default=2048, help="most tokens a request may reach, prompt included (a multiple of 128)")
    p.add_argument("--seed", type=int, default=123, help="seed of the prompts and of temperature sampling")
    p.add_argument("--cuda_graph_decode", action="store_true",
                   help="replay steps in which every request decodes one token from a recorded CUDA graph")
    p.add_argument("--printoutput", action="store_true", help="print what the first requests generated")
    p.add_argument("--dataset", type=str, choices=["dummy1tok", "dummy4tok", "random"], default="dummy4tok",
                   help="synthetic prompts: one or four copies of one token, or random ids of --prompt_len")
    p.add_argument("--num_samples", type=int, default=16, help="how many requests are made")
    p.add_argument("--dummy_token_id", type=int, default=None, help="the token the dummy prompts repeat (default: bos_token_id, else 1)")
    p.add_argument("--full_cache_layers", nargs="+", type=int, default=None,
                   help="indices of the layers that read every page; a full layer followed by another kind chooses the pages")
    p.add_argument("--subset_cache_ratio", type=float, default=0.5, help="accepted and unused, as in the reference")
    p.add_argument("--compression_ratio", type=float, default=1.0,
                   help="a request reads a subset once its pages / min(pages, subset_cache_size) exceed this")
    p.add_argument("--subset_cache_size", type=int, default=1024, help="pages per request that the other layers read")
    p.add_argument("--L", type=int, default=8, help="the newest L pages are always among the chosen")
    p.add_argument("--enable_selective_cache", action="store_true", help="DELTA on: layers outside --full_cache_layers read chosen pages")
    # added
    p.add_argument("--count_page_ahead", action="store_true",
                   help="count a request's pages as the reference does: one more, empty, once the newest is exactly full")
    p.add_argument("--random_weights", type=int, default=None, metavar="SEED", help="random weights instead of a folder's")
    p.add_argument("--config", type=Path, default=None, help="config.json for --random_weights")
    p.add_argument("--prompt_len", type=int, default=128)
    p.add_argument("--max_new_tokens", type=int, default=None)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top_p", type=float, default=1.0)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--page_size", type=int, default=16)
    p.add_argument("--num_pages", type=int, default=None)
    p.add_argument("--max_tokens_per_step", type=int, default=2048)
    p.add_argument("--throughput_mode", action="store_true", help="stop when the first request finishes")
    p.add_argument("--out", type=Path, default=None, help="write the result JSON here")
    p.add_argument("--step_timings", action="store_true",
                   help="time every step (collect_pages, plan, model_forward, postprocess, step_total) and write logs/step_timings_<time>.json")
    p.add_argument("--tuning_file", type=Path, default=None,
                   help="JSON file with the measured choice of product kernels: read if it exists, written at the end")
    return p


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.max_len % 128:
        raise SystemExit("--max_len must be a multiple of 128")   # tests/reasoni.py:272
    if args.full_cache_layers is not None:
        args.full_cache_layers = sorted(set(args.full_cache_layers))
    if args.model is None and args.random_weights is None:
        raise SystemExit("give --model FOLDER, or --random_weights SEED with --config FILE")
    random.seed(args.seed)

    from .engine import LMBackend
    from .parts import linear
    if args.tuning_file is not None and args.tuning_file.is_file():
        linear.load_choices(args.tuning_file)
    eng = LMBackend(dtype=args.dtype, device="cuda:0", cuda_graph_decode=args.cuda_graph_decode)
    if args.random_weights is not None:
        cfg_path = args.config or (args.model / "config.json" if args.model else None)
        if cfg_path is None:
            raise SystemExit("--random_weights needs --config FILE (or --model FOLDER for its config.json)")
        config_json = json.loads(Path(cfg_path).read_text())
        eng.load_model(config_json=config_json, seed=args.random_weights)
    else:
        config_json = json.loads((args.model / "config.json").read_text())
        eng.load_model(args.model)
    eng.setup_caches(max_batch_size=args.B, max_seq_length=args.max_len, page_size=args.page_size, num_pages=args.num_pages,
                     max_tokens_per_step=args.max_tokens_per_step, enable_selective_cache=args.enable_selective_cache,
                     full_cache_layers=args.full_cache_layers, subset_cache_size=args.subset_cache_size,
                     compression_ratio=args.compression_ratio, L=args.L, count_page_ahead=args.count_page_ahead)
    eng.throughput_mode = args.throughput_mode
    eng.record_timings = bool(args.step_timings)
    tok = None
    if args.model_name:
        from transformers import AutoTokenizer   # the tokenizer only; no model code of that package is used
        tok = AutoTokenizer.from_pretrained(args.model_name, local_files_only=True)
        eng.set_tokenizer(tok)

    vocab = int(config_json["vocab_size"])
    if args.dataset == "random":
        rng = random.Random(args.seed)
        prompts = [[rng.randrange(vocab) for _ in range(args.prompt_len)] for _ in range(args.num_samples)]
    else:
        tid = args.dummy_token_id
        if tid is None:
            tid = config_json.get("bos_token_id")
            tid = 1 if tid is None else int(tid)
        n = 1 if args.dataset == "dummy1tok" else 4
        prompts = [[tid] * n for _ in range(args.num_samples)]
    eng.add_requests(prompts, [args.max_len] * len(prompts), [], temperature=args.temperature, top_p=args.top_p,
                     seed=args.seed, max_new_tokens=args.max_new_tokens)
    t0 = time.perf_counter()
    results = eng.run_scheduler_loop()
    total = time.perf_counter() - t0
    st = eng.scheduler.stats
    decode = [s for s in eng.step_timings if s["tokens"] == s["active_bsz"]]
    summary = dict(total_time_s=total, requests=len(results), prompt_tokens=st["prompt_tokens"],
                   generated_tokens=st["generated_tokens"], tokens_per_second=st["generated_tokens"] / total if total else 0.0,
                   steps=st["steps"], preemptions=st["preemptions"],
                   graph_captures=eng.runner.graph_captures, graph_replays=eng.runner.graph_replays,
                   graph_fallbacks=dict(eng.runner.graph_fallbacks),
                   decode_step_ms_mean=(sum(s["model_forward_ms"] for s in decode) / len(decode)) if decode else None)
    if args.step_timings:
        path = eng.save_step_timings("logs", meta=dict(args={k: str(v) for k, v in vars(args).items()}))
        summary["step_timings_file"] = str(path) if path else None
    if args.tuning_file is not None:
        linear.save_choices(args.tuning_file)
    print(json.dumps(summary))
    if args.printoutput:
        for r in results[:4]:
            print(r["request_id"], r.get("output_text", r["output_ids"][:32]))
    if args.out:
        args.out.parent.mkdir(parents=True, exist_ok=True)
        args.out.write_text(json.dumps(dict(args={k: str(v) for k, v in vars(args).items()}, summary=summary,
                                            results=results, step_timings=eng.step_timings)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
