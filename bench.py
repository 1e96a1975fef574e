#!/usr/bin/env python3
"""Decode and prefill throughput of the delta_b200 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers L] [--shape yi-6b|yi-9b|yi-34b]

Default run: the layer sizes of Yi-6B (32 layers, hidden 4096, 32 heads over 4
key-value heads of 128, intermediate 11008, vocabulary 64000), random bfloat16
weights, 8 requests decoding at a context of 4096 tokens.  One step is one decode
step.  It prints ONE JSON line:

  value      decoded tokens per second, device time of the K timed steps (model step
             and sampling, measured with CUDA events around each step)
  e2e        the same through the Python entry point (LMBackend.step), timed over further runs
             of K steps without the per-step synchronisation the device timing needs: every
             step copies its inputs (positions, block tables, sampling parameters, tokens) from
             pinned host memory and reads the new tokens back to the host.  ``value`` is the
             engine as it runs by default: a decode step is launched while the host still reads
             the step before, with its tokens taken from that step's result on the device;
             ``value_tokens_fed_back_through_host`` is the same with that switched off.
             (Run ahead, the loop can come out a little faster than ``value``: the steps of
             ``value`` are timed one by one, each starting on an idle GPU with its copies on the
             critical path, while here the next step's copies queue behind the running step.)
  prefill    one prompt of 2,048 tokens in one step; frac = flops / time / peak
  roofline   bytes a decode step has to read (every weight once, and the cache of the
             live requests) / its time, against the copy bandwidth
  points     decode tokens per second at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file when it is there, else from the
fallback figures of an earlier measurement of a B200.  The engine runs on one GPU
only: for --gpus above 1 it says so and exits with 2.

Other workloads (``--workload``), each printing one JSON line of the same shape:

  baseline     2,048-token prompts and 512 generated tokens each through ``run_scheduler_loop`` at
               batch 1, 8 and 64 (Yi-6B shape): tokens per second = generated tokens / time of the
               decode steps, and the same over the wall clock of the whole loop
  yi9b-long    Yi-1.5-9B shape, 16 requests of 256 + 3,584 tokens, once with the full cache and
               once with DELTA (``--full_cache_layers 2 --subset_cache_size 64``); both rates and
               their ratio
  yi34b-mixed  Yi-34B shape: steps of one 2,048-token prompt portion beside up to 63 decoding
               requests; milliseconds per mixed step, tokens per second of both kinds, and the
               portion's share of the tensor-core peak
  long-prompt  Yi-6B shape, one prompt of 30,000 tokens (``--context``) in portions of 2,048: milliseconds of the
               first and the last portion, of the whole prompt, and of a decode step behind it
  grown        Yi-6B shape, 64 requests (``--batch``) of 64 + 2,400 tokens: nearly every page is taken
               during decoding, a page at a time in turns with the other requests; the last sixth of
               the decode steps, with the pool handing pages out in runs and one by one

``--impl reference`` runs the unmodified hoenza/DELTA engine (baseline/reference_arm.py) on the
default workload and prints its line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

YI_6B = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096, num_hidden_layers=32,
             num_attention_heads=32, num_key_value_heads=4, intermediate_size=11008, vocab_size=64000,
             rope_theta=5000000.0, rms_norm_eps=1e-5, max_position_embeddings=4096, hidden_act="silu",
             tie_word_embeddings=False, torch_dtype="bfloat16")
# other shapes of the same architecture, for runs beside the default one (--shape)
SHAPES = {
    "yi-6b": ("Yi-6B shape", YI_6B),
    "yi-9b": ("Yi-1.5-9B shape", dict(YI_6B, num_hidden_layers=48, rms_norm_eps=1e-6)),
    "yi-34b": ("Yi-34B shape", dict(YI_6B, hidden_size=7168, num_hidden_layers=60, num_attention_heads=56,
                                    num_key_value_heads=8, intermediate_size=20480)),
}
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            out = dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                       source="measured")
            return out
        except Exception:  # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return dict(sm_mhz=mhz[len(mhz) // 2] if mhz else None, sm_max_mhz=mx, reasons=sorted(reasons), samples=len(mhz))


def model_numbers(cfg: dict, layers: int):
    d, H, KV = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or d // H
    I, V = cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = (H + 2 * KV) * hd * d + H * hd * d + 3 * I * d
    weight_bytes = 2 * (layers * (per_layer + 2 * d) + V * d + d)
    kv_bytes_per_token = layers * 2 * KV * hd * 2

    def prefill_flops(T):
        gemm = 2 * T * layers * per_layer + 2 * V * d  # logits for one row
        attn = layers * 4 * hd * H * (T * (T + 1) // 2)
        return gemm + attn
    return weight_bytes, kv_bytes_per_token, prefill_flops


def reference_arm(args) -> int:
    """The unmodified reference on the same decode workload: ``baseline/reference_arm.py`` in a
    process of its own (nothing of delta_b200 is imported there); its JSON line is printed as it
    is.  Whatever goes wrong becomes the ``unavailable`` line with the reason."""
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:400]}))
        return 0
    if args.gpus != 1:
        return unavailable("the reference arm is set up for one GPU")
    script = ROOT / "baseline" / "reference_arm.py"
    if not (ROOT / "baseline" / "_ref" / "DELTA").is_dir():
        return unavailable("no copy of hoenza/DELTA under baseline/_ref (it has no setup.py or pyproject.toml, so pip "
                           "cannot install it; a plain copy of the tree is what its own scripts use)")
    if args.shape == "yi-9b":
        return unavailable("the reference's table of models has no 48-layer Yi entry (DELTA/Engine/DELTA/model.py:72-97)")
    cmd = [sys.executable, str(script), "--batch", str(args.batch), "--context", str(args.context), "--steps", str(args.steps),
           "--warmup", str(max(3, args.warmup)), "--shape", args.shape]
    if args.no_graph:
        cmd.append("--no-graph")
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    except subprocess.TimeoutExpired:
        return unavailable("the reference did not finish within 1500 s")
    sys.stderr.write(r.stderr[-4000:])
    for line in reversed(r.stdout.splitlines()):
        if line.startswith('{"impl"'):
            print(line)
            return 0
    tail = (r.stderr.strip().splitlines() or r.stdout.strip().splitlines() or ["no output"])[-1]
    return unavailable(f"the reference ended with code {r.returncode}: {tail}")


def _flat_config(shape_name, cfg, layers, **more) -> dict:
    d = cfg["hidden_size"]
    out = {"model": shape_name, "layers": layers, "layers_of_named_config": cfg["num_hidden_layers"], "hidden": d,
           "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
           "head_dim": cfg.get("head_dim") or d // cfg["num_attention_heads"], "intermediate": cfg["intermediate_size"],
           "vocab": cfg["vocab_size"], "page_size": 16, "parallelism": "single GPU"}
    out.update(more)
    return out


def _loop(eng, prompts, max_new, timed: bool):
    """Runs the requests through ``run_scheduler_loop``.  Timed: every step between CUDA events
    (returns the decode steps' records); untimed: as a user runs it, wall clock only."""
    import torch
    eng.step_timings.clear()
    eng.record_timings = timed
    eng.add_requests(prompts, [len(p) + max_new for p in prompts], [], max_new_tokens=max_new)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.run_scheduler_loop()
    wall = time.perf_counter() - t0
    eng.record_timings = False
    decode = [r for r in eng.step_timings if r["tokens"] == r["active_bsz"]]
    return decode, wall


def other_workload(args) -> int:
    import torch
    from delta_b200.engine import LMBackend
    from delta_b200.kernels import ops
    pk = peaks()
    gen = torch.Generator().manual_seed(1)
    name = args.workload
    shape = {"baseline": "yi-6b", "yi9b-long": "yi-9b", "yi34b-mixed": "yi-34b", "grown": "yi-6b", "long-prompt": "yi-6b"}[name]
    shape_name, shape_cfg = SHAPES[shape]
    layers = args.layers or shape_cfg["num_hidden_layers"]
    cfg = dict(shape_cfg, num_hidden_layers=layers)
    weight_bytes, kv_per_tok, prefill_flops = model_numbers(cfg, layers)

    def prompts(n, length):
        return [torch.randint(0, cfg["vocab_size"], (length,), generator=gen).tolist() for _ in range(n)]

    def engine(max_batch, max_len, **kw):
        e = LMBackend(dtype=torch.bfloat16, device="cuda:0", cuda_graph_decode=not args.no_graph)
        e.load_model(config_json=cfg, seed=0)
        e.setup_caches(max_batch_size=max_batch, max_seq_length=max_len, page_size=16, **kw)
        e.scheduler.decode_while_prefill = False
        return e

    clocks = ClockSampler()
    if name == "baseline":
        plen, new = 2048, args.generate or 512
        eng = engine(64, plen + new, max_tokens_per_step=2048)
        points, e2e, ms = {}, {}, {}
        clocks.start()
        for b in (1, 8, 64):
            _loop(eng, prompts(b, plen), 24, True)                     # records the graphs of this batch size
            decode, _ = _loop(eng, prompts(b, plen), new, True)
            full = [r for r in decode if r["active_bsz"] == b]
            t = sum(r["model_forward_ms"] + r["postprocess_ms"] for r in full)
            points[f"decode_b{b}"] = b * len(full) / (t / 1e3)
            ms[f"b{b}"] = t / len(full)
            l0 = ops.launch_count()
            _, wall = _loop(eng, prompts(b, plen), new, False)
            e2e[f"b{b}"] = b * new / wall        # prompts included in the time: what a user of the loop sees
        clk = clocks.stop()
        ctx = plen + new / 2
        achieved = (weight_bytes + 8 * ctx * kv_per_tok) / (ms["b8"] / 1e3) / 1e9
        out = {"workload": name, "metric": f"decode tok/s ({shape_name}, bf16, 2,048-token prompts + {new} generated, batch 1/8/64)",
               "value": points["decode_b8"], "unit": "tokens/s", "n_gpus": 1, "ms_per_step": ms["b8"], "higher_is_better": True,
               "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), random token ids)",
               "config": _flat_config(shape_name, shape_cfg, layers, global_batch=8, seq_len=plen + new, prompt_len=plen,
                                      generated=new, cuda_graph_decode=not args.no_graph, peaks=pk["source"]),
               "points": points, "ms_per_decode_step": ms,
               "e2e": {"unit": "generated tokens/s over the wall clock of the whole loop, prompts included", **e2e},
               "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
               "clocks": clk}
    elif name == "yi9b-long":
        B, plen, new = 16, 256, args.generate or 3584
        res = {}
        clocks.start()
        for mode in ("full", "delta"):
            eng = engine(B, plen + new, max_tokens_per_step=4096, enable_selective_cache=mode == "delta",
                         full_cache_layers=[2] if mode == "delta" else None, subset_cache_size=64)
            _loop(eng, prompts(B, plen), 24, True)
            decode, _ = _loop(eng, prompts(B, plen), new, True)
            t = sum(r["model_forward_ms"] + r["postprocess_ms"] for r in decode)
            _, wall = _loop(eng, prompts(B, plen), new, False)
            tail = decode[-max(1, len(decode) // 8):]       # the last eighth: the longest contexts
            res[mode] = dict(tokens_per_s=B * len(decode) / (t / 1e3), ms_per_step=t / len(decode),
                             ms_per_step_last_eighth=sum(r["model_forward_ms"] + r["postprocess_ms"] for r in tail) / len(tail),
                             e2e_tokens_per_s=B * new / wall, steps=len(decode))
            del eng
            torch.cuda.empty_cache()
        clk = clocks.stop()
        out = {"workload": name, "metric": f"decode tok/s ({shape_name}, bf16, batch {B}, {plen}-token prompts + {new} generated)",
               "value": res["delta"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "ms_per_step": res["delta"]["ms_per_step"],
               "higher_is_better": True, "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), random token ids)",
               "config": _flat_config(shape_name, shape_cfg, layers, global_batch=B, seq_len=plen + new, prompt_len=plen,
                                      generated=new, full_cache_layers="2", subset_cache_size=64, cuda_graph_decode=not args.no_graph),
               "full_cache": res["full"], "delta": res["delta"],
               "delta_over_full": res["delta"]["tokens_per_s"] / res["full"]["tokens_per_s"], "clocks": clk}
    elif name == "long-prompt":
        # One prompt of 30,000 tokens (--context sets another length) in portions of 2,048, then 16 decoded tokens: the
        # portions' attention reads what the portions before left in the cache, so the later ones are bound by it.
        plen = args.context if args.context != 4096 else 30000
        cfg = dict(cfg, max_position_embeddings=max(cfg.get("max_position_embeddings", 0), plen + 64))
        eng = engine(2, plen + 64, max_tokens_per_step=2048)
        clocks.start()
        for _ in range(2):              # the second run is the measured one (kernels chosen, buffers made)
            records, _ = None, None
            eng.step_timings.clear()
            eng.record_timings = True
            eng.add_requests(prompts(1, plen), [plen + 16], [], max_new_tokens=16)
            eng.run_scheduler_loop()
            eng.record_timings = False
            records = list(eng.step_timings)
        clk = clocks.stop()
        pre = [r["model_forward_ms"] + r["postprocess_ms"] for r in records if r["tokens"] > 1]
        dec = [r["model_forward_ms"] + r["postprocess_ms"] for r in records if r["tokens"] == 1]
        flops = prefill_flops(plen)
        out = {"workload": name, "metric": f"prefill tok/s ({shape_name}, bf16, one prompt of {plen} tokens in portions of 2,048)",
               "value": plen / (sum(pre) / 1e3), "unit": "tokens/s", "n_gpus": 1, "ms_per_step": sum(pre) / len(pre), "higher_is_better": True,
               "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), random token ids)",
               "config": _flat_config(shape_name, shape_cfg, layers, global_batch=1, seq_len=plen, portion=2048, peaks=pk["source"]),
               "prompt_ms": sum(pre), "first_portion_ms": pre[0], "last_full_portion_ms": pre[-2] if len(pre) > 1 else pre[-1],
               "decode_ms_per_step_at_the_end": sum(dec) / max(1, len(dec)),
               "prefill": {"value": plen / (sum(pre) / 1e3), "tokens": plen, "ms": sum(pre), "frac": flops / (sum(pre) / 1e3) / (pk["bf16_tflops"] * 1e12)},
               "clocks": clk}
    elif name == "grown":
        # Many requests with short prompts that decode for a long time, in turns: nearly every page of a request
        # is taken during decoding, one at a time, between the pages the other requests take.  Measured with the
        # pool handing out runs of pages, and with the one-page last-in-first-out stack.
        B, plen, new = args.batch if args.batch != 8 else 64, 64, args.generate or 2400
        res = {}
        clocks.start()
        for runs in (True, False):
            eng = engine(B, plen + new, max_tokens_per_step=4096, page_runs=runs)
            _loop(eng, prompts(B, plen), 24, True)
            decode, _ = _loop(eng, prompts(B, plen), new, True)
            tail = decode[-max(1, len(decode) // 6):]
            res[runs] = sum(r["model_forward_ms"] + r["postprocess_ms"] for r in tail) / len(tail)
            del eng
            torch.cuda.empty_cache()
        clk = clocks.stop()
        ctx = plen + new * 11 / 12
        achieved = (weight_bytes + B * ctx * kv_per_tok) / (res[True] / 1e3) / 1e9
        out = {"workload": name, "metric": f"decode tok/s ({shape_name}, bf16, batch {B}, {plen}-token prompts + {new} generated, last sixth of the steps)",
               "value": B / (res[True] / 1e3), "unit": "tokens/s", "n_gpus": 1, "ms_per_step": res[True], "higher_is_better": True,
               "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), random token ids)",
               "config": _flat_config(shape_name, shape_cfg, layers, global_batch=B, seq_len=plen + new, prompt_len=plen, generated=new,
                                      cuda_graph_decode=not args.no_graph, peaks=pk["source"]),
               "ms_per_step_pages_in_runs": res[True], "ms_per_step_pages_one_by_one": res[False],
               "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
               "clocks": clk}
    else:
        B, portion, ctx_len = 64, 2048, 4096
        eng = engine(B, ctx_len, max_tokens_per_step=portion + B)
        eng.scheduler.decode_while_prefill = True
        n_mixed = max(4, min(args.steps, 12))
        # 63 requests decode from a context of 1,024 tokens on; then one prompt of 2,048 tokens is added per step
        eng.add_requests(prompts(B - 1, 1024), [ctx_len] * (B - 1), [])
        while eng.scheduler.waiting or any(not r.output for r in eng.scheduler.running):
            eng.step()
        for _ in range(4):
            eng.step()
        records = []
        clocks.start()
        eng.record_timings = True
        for k in range(n_mixed + 2):
            eng.add_requests(prompts(1, portion), [portion + 1], [])     # ends after its first token: its slot is free again
            eng.step_timings.clear()
            eng.step()
            records.extend(eng.step_timings)
        eng.record_timings = False
        clk = clocks.stop()
        mixed = [r for r in records if r["tokens"] > portion][2:]
        t = sum(r["model_forward_ms"] + r["postprocess_ms"] for r in mixed) / len(mixed)
        dec = sum(r["active_bsz"] - 1 for r in mixed) / len(mixed)
        out = {"workload": name, "metric": f"mixed step ({shape_name}, bf16): one {portion}-token prompt portion beside {B - 1} decoding requests",
               "value": (portion + dec) / (t / 1e3), "unit": "tokens/s", "n_gpus": 1, "ms_per_step": t, "higher_is_better": True,
               "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), random token ids)",
               "config": _flat_config(shape_name, shape_cfg, layers, global_batch=B, seq_len=ctx_len, portion=portion, steps=len(mixed)),
               "prefill_tokens_per_s": portion / (t / 1e3), "decode_tokens_per_s": dec / (t / 1e3),
               "chunk": {"flops": prefill_flops(portion), "frac": prefill_flops(portion) / (t / 1e3) / (pk["bf16_tflops"] * 1e12),
                         "peak_tflops": pk["bf16_tflops"]},
               "weights_gb": weight_bytes / 1e9, "clocks": clk}
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (both numbers go into config)")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="yi-6b")
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--enable_selective_cache", action="store_true", help="DELTA on (not the default run)")
    ap.add_argument("--full_cache_layers", nargs="+", type=int, default=[0, 1, 2, 14, 22])
    ap.add_argument("--subset_cache_size", type=int, default=64)
    ap.add_argument("--workload", choices=["decode", "baseline", "yi9b-long", "yi34b-mixed", "grown", "long-prompt"], default="decode")
    ap.add_argument("--generate", type=int, default=None, help="tokens generated per request in the other workloads (default: what the workload names)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported (single-GPU engine tier)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.workload != "decode":
        return other_workload(args)

    import torch
    from delta_b200.engine import LMBackend
    from delta_b200.kernels import ops

    shape_name, shape_cfg = SHAPES[args.shape]
    full_layers = shape_cfg["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    cfg = dict(shape_cfg, num_hidden_layers=args.layers)
    pk = peaks()
    weight_bytes, kv_per_tok, prefill_flops = model_numbers(cfg, args.layers)
    ctx_len = args.context
    max_b = 64 if not args.skip_points else args.batch
    eng = LMBackend(dtype=torch.bfloat16, device="cuda:0", cuda_graph_decode=not args.no_graph)
    eng.load_model(config_json=cfg, seed=0)
    eng.setup_caches(max_batch_size=max(max_b, args.batch), max_seq_length=ctx_len, page_size=16, max_tokens_per_step=2048,
                     enable_selective_cache=args.enable_selective_cache,
                     full_cache_layers=args.full_cache_layers if args.enable_selective_cache else None,
                     subset_cache_size=args.subset_cache_size)
    gen = torch.Generator().manual_seed(1)

    def fresh_prompts(n, length):
        return [torch.randint(0, cfg["vocab_size"], (length,), generator=gen).tolist() for _ in range(n)]

    def run_decode(batch, steps, warmup, through_api_wall=False):
        """Prefills ``batch`` requests so that the timed decode steps end at the context
        length, then times ``steps`` decode steps.  Returns (device ms per step, end-to-end
        ms per step, launches per step, bytes in, bytes out, mean context)."""
        total_new = warmup + 3 * steps + 3
        plen = ctx_len - total_new
        sch = eng.scheduler
        sch.decode_while_prefill = False
        eng.add_requests(fresh_prompts(batch, plen), [ctx_len] * batch, [])
        while sch.waiting or any(not r.output for r in sch.running):
            eng.step()
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        l0 = ops.launch_count()
        dev_ms = 0.0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        eng.record_timings = True
        eng.step_timings.clear()
        for _ in range(steps):
            eng.step()
        torch.cuda.synchronize()
        eng.record_timings = False
        dev_ms = sum(s["model_forward_ms"] + s["postprocess_ms"] for s in eng.step_timings) / steps
        launches = (ops.launch_count() - l0) / steps
        mean_ctx = plen + warmup + steps / 2
        # the same number of steps again as a user drives them: no per-step synchronisation for
        # timing, so the engine launches each decode step while the host still reads the one before
        e2e = []
        for ahead in (False, True):     # tokens fed back through the host; then on the device, one step ahead
            eng.run_ahead = ahead
            eng.step()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(steps):
                eng.step()
            e1.record()
            torch.cuda.synchronize()
            e2e.append(e0.elapsed_time(e1) / steps)
        e2e_ms = tuple(e2e)
        h2d = eng.runner.last_staging_bytes
        sch.abort_all("bench")
        return dev_ms, e2e_ms, launches, h2d, 4 * batch, mean_ctx

    # ---- prefill of 2,048 tokens ------------------------------------------------
    T = 2048
    pre_ms = []
    for i in range(3):
        eng.add_requests(fresh_prompts(1, T), [T + 1], [])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        eng.step()
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
        eng.scheduler.abort_all("bench")
    pre = min(pre_ms[1:])
    prefill = dict(value=T / (pre / 1e3), tokens=T, ms=pre, frac=prefill_flops(T) / (pre / 1e3) / (pk["bf16_tflops"] * 1e12))

    # ---- the headline: decode at the default batch --------------------------------
    clocks = ClockSampler()
    clocks.start()
    dev_ms, e2e_ms, launches, h2d, d2h, mean_ctx = run_decode(args.batch, args.steps, args.warmup)
    clk = clocks.stop()
    value = args.batch / (dev_ms / 1e3)
    bytes_step = weight_bytes + args.batch * mean_ctx * kv_per_tok
    achieved = bytes_step / (dev_ms / 1e3) / 1e9
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            d_ms, _, _, _, _, _ = run_decode(b, max(16, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = b / (d_ms / 1e3)

    out = {
        "metric": f"decode tok/s ({shape_name}, bf16, batch {args.batch}, context {ctx_len})", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), random token ids)",
        "config": _flat_config(shape_name, shape_cfg, args.layers, global_batch=args.batch, seq_len=ctx_len,
                               cuda_graph_decode=not args.no_graph, selective_cache=bool(args.enable_selective_cache),
                               l2="inputs larger than L2 (weights %.1f GB)" % (weight_bytes / 1e9), peaks=pk["source"]),
        "e2e": {"value": args.batch / (e2e_ms[1] / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "value_tokens_fed_back_through_host": args.batch / (e2e_ms[0] / 1e3)},
        "gpu_launches": int(round(launches * args.steps)),
        "clocks": clk,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
        "points": points,
    }
    from delta_b200.parts import linear
    print("kernels chosen per product (rows bucket, N, K, swiglu, out): " +
          "; ".join(f"{k[0]}x{k[1]}x{k[2]}{'sw' if k[3] else ''}->{v}" for k, v in sorted(linear.choices().items(), key=str)),
          file=sys.stderr)
    print("measured in isolation, us:",
          "; ".join(f"{k[0]}x{k[1]}x{k[2]}{'sw' if k[3] else ''}: " + " ".join(f"{c}={t:.1f}" for c, t in v.items())
                    for k, v in sorted(linear.timings().items(), key=str)), file=sys.stderr)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
