"""Matrix products  y = x W^T  of the parts.

32-bit activations go through the plain FMA kernel (true 32 bit: no
reduced-precision matrix mode, no split over K).  bfloat16 activations go
through the tensor cores.  For large batches (prompt portions) that is the
library product the reference uses for its ``nn.Linear`` layers
(DELTA/Engine/DELTA/model.py:369-370, 498-500), measured once per shape against
the tcgen05 kernel of this package taking the rows in chunks (which has lost on
every shape measured so far).  For the few rows of a decode
step the product is a stream over the weights and four kernels compete: the
warp-level MMA kernel that loads weights straight into fragments, the persistent
tcgen05/TMA kernel that cuts the (tile, K step) sequence into one piece per SM,
the tcgen05/TMA kernel with one block per tile (1, 2, 4 or 8 blocks sharing K as
a cluster), and the library.  Which one is fastest depends on the shape, so each (rows bucket, N, K,
epilogue) is measured once on the real weights, with the L2 flushed between runs,
and the winner is kept.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..kernels import ops

SMALL_M = 128          # up to this many rows a product counts as weight streaming
MANY_M = 4096          # up to this many rows the library's product is measured against the tcgen05 kernel in chunks of rows
_BUCKETS = (8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096)
_choice: Dict[tuple, str] = {}
_times: Dict[tuple, Dict[str, float]] = {}
_flush: Optional[torch.Tensor] = None
# Another kernel replaces the preferred one only when it is faster by more than ``margin(t)`` microseconds: a
# product of another kind than its neighbours costs 2 to 3 us more in the step than alone, and below 3 % two
# measurements of the same kernel differ.  (A margin of 8 % of the time, as it was, kept the small-batch kernel
# for the 50 to 140 us products of the Yi-34B shape where the library is 6 to 9 us faster, in some runs and
# not in others: 14.4 against 13.2 ms a step.)
MARGIN_US = 2.5
MARGIN_REL = 0.03


def margin(t_us: float) -> float:
    return max(MARGIN_US, MARGIN_REL * t_us)


TUNE = os.environ.get("DELTA_B200_NO_TUNE") != "1"   # off: the first candidate of a shape is taken unmeasured


def _bucket(m: int) -> int:
    for b in _BUCKETS:
        if m <= b:
            return b
    return 0


def _candidates(m: int, n: int, k: int, swiglu: bool, out_dtype) -> List[str]:
    c = []
    if m > SMALL_M:
        # prompt portions: the library (what the reference uses) unless the kernel of this package beats it
        if out_dtype == torch.bfloat16:
            c.append("lib")
        if ops.gemm_tc_many_rows_supported(m, n, k, swiglu):
            c.append("tcr")
        return c
    if m <= 64 and ops.gemm_small_m_supported(m, n, k, swiglu):
        c.append("small")
    if ops.gemm_tc_supported(m, n, k, swiglu):
        for s in (1, 2, 4, 8):
            if s == 1 or k // (256 * s) >= 2:
                c.append(f"tc{s}")
        if m <= 64:
            c.append("tc1d")     # two blocks per SM (shorter stages): for more tiles than SMs, up to twice as many
            if k // 512 >= 2:
                c.append("tc2d")
    if out_dtype == torch.bfloat16:
        c.append("lib")
    if ops.gemm_stream_k_supported(m, n, k, swiglu):
        c.append("sk")       # last: a tie in isolation goes to the kernels that end sooner on most SMs
    return c


def _run(kind: str, x, w, out, swiglu: bool, err=None):
    if kind == "small":
        return ops.gemm_small_m(x, w, out, swiglu=swiglu)
    if kind == "sk":
        return ops.gemm_stream_k(x, w, out, swiglu=swiglu, err=err)
    if kind == "tcr":
        return ops.gemm_tc(x, w, out, swiglu=swiglu, err=err)
    if kind.startswith("tc"):
        two = kind.endswith("d")
        return ops.gemm_tc(x, w, out, swiglu=swiglu, splits=int(kind[2:3]), err=err, per_sm=2 if two else 1)
    ops.count_launch()
    if swiglu:
        gu = torch.mm(x, w.t())
        return ops.silu_mul(gu, out)
    return torch.mm(x, w.t(), out=out)


def _time(fn, reps: int = 12) -> float:
    """Median microseconds of fn on the current stream, each run after a flush of the L2 and
    between its own pair of events.  The flush takes longer than the host needs to enqueue the
    events and fn, so the host's launch overhead does not count, as in a captured decode step.
    Nothing is captured and no other stream is used: a CUDA graph recorded here before the decode
    step's own, or work on a second stream, left the decode step 3 % slower for the rest of the
    process (measured at Yi-6B sizes, batch 8)."""
    fn()
    pairs = []
    for _ in range(reps):
        _flush.zero_()
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        pairs.append((e0, e1))
    torch.cuda.synchronize()
    times = sorted(e0.elapsed_time(e1) for e0, e1 in pairs)
    return 1e3 * times[len(times) // 2]


def _tune(m: int, x, w, swiglu: bool, out_dtype, err) -> str:
    """Times every candidate on these weights with ``m`` rows.  The first candidate (the order of
    ``_candidates`` is the order of preference) stays unless another is faster by more than
    ``margin``: differences below that are within the noise of a measurement in isolation, and a
    choice that changes from run to run costs more in the step than it gains here."""
    global _flush
    n, k = w.shape
    cands = _candidates(m, n, k, swiglu, out_dtype)
    if not cands:
        return "none"
    if len(cands) == 1 or not TUNE or torch.cuda.is_current_stream_capturing():
        return cands[0]
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device=x.device)   # larger than the L2
    xs = torch.randn((m, k), device=x.device, dtype=torch.float32).to(x.dtype)
    out = torch.empty((m, n // 2 if swiglu else n), dtype=out_dtype, device=x.device)
    torch.cuda.synchronize()
    best, best_t = cands[0], float("inf")
    for kind in cands:
        try:
            t = _time(lambda: _run(kind, xs, w, out, swiglu, err))    # (its first call is untimed: set-up, workspaces)
        except (ops.KernelError, RuntimeError):
            continue
        _times.setdefault((m, n, k, swiglu), {})[kind] = t
        if best_t == float("inf") or t < best_t - margin(best_t):
            best, best_t = kind, t
    torch.cuda.synchronize()
    return best


def choose(m: int, w: torch.Tensor, x: torch.Tensor, swiglu: bool, out_dtype, err=None) -> str:
    key = (_bucket(m), w.shape[0], w.shape[1], swiglu, out_dtype)
    kind = _choice.get(key)
    if kind is None:
        kind = _tune(key[0], x, w, swiglu, out_dtype, err)
        if not torch.cuda.is_current_stream_capturing():
            _choice[key] = kind
    return kind


def timings() -> Dict[tuple, Dict[str, float]]:
    """Microseconds measured per candidate: (rows, N, K, swiglu) -> {kernel: us}."""
    return {k: dict(v) for k, v in _times.items()}


def choices() -> Dict[tuple, str]:
    """What the measurements chose so far: (rows bucket, N, K, swiglu, out dtype) -> kernel."""
    return dict(_choice)


def save_choices(path) -> None:
    """Writes what the measurements chose (and the times they saw) as JSON, so that a later
    run starts without measuring and takes the same kernels (the same bfloat16 bits)."""
    import json
    items = [dict(rows=k[0], n=k[1], k=k[2], swiglu=bool(k[3]), out=str(k[4]).replace("torch.", ""), kernel=v,
                  times_us=_times.get((k[0], k[1], k[2], k[3]), {})) for k, v in sorted(_choice.items(), key=str)]
    with open(path, "w") as f:
        json.dump({"product_kernels": items}, f, indent=1)


def load_choices(path) -> int:
    """Takes the choices of a file written by ``save_choices``; returns how many it held.  A
    kernel name that this build does not know is an error, not a silent new measurement."""
    import json
    with open(path) as f:
        items = json.load(f)["product_kernels"]
    known = {"small", "lib", "sk", "none", "tc1", "tc2", "tc4", "tc8", "tc1d", "tc2d", "tcr"}
    for it in items:
        if it["kernel"] not in known:
            raise ValueError(f"{path}: unknown product kernel '{it['kernel']}'")
        _choice[(int(it["rows"]), int(it["n"]), int(it["k"]), bool(it["swiglu"]), getattr(torch, it["out"]))] = it["kernel"]
    return len(items)


def swiglu_linear(ctx, x: torch.Tensor, w_gate_up: torch.Tensor):
    """silu(x gate^T) * (x up^T) with the gate fused into the product's epilogue when the batch
    is small enough for the streaming kernels; else None."""
    T = x.shape[0]
    if x.dtype != torch.bfloat16 or ("products" in ctx.plain_kernels) or not (0 < T <= MANY_M):
        return None
    kind = choose(T, w_gate_up, x, True, x.dtype, ctx.err)
    if kind == "none" or (kind == "lib" and T > SMALL_M):
        return None       # (the caller's library product and SwiGLU kernel)
    out = torch.empty((T, w_gate_up.shape[0] // 2), dtype=x.dtype, device=x.device)
    _run(kind, x, w_gate_up, out, True, ctx.err)
    return out


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """x [T, K], w [N, K] -> [T, N] in ``out_dtype`` (the type of x by default)."""
    out_dtype = out_dtype or x.dtype
    T, N = x.shape[0], w.shape[0]
    if x.dtype == torch.float32 or ("products" in ctx.plain_kernels):
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
        if T:
            ops.gemm_nt_plain(x, w, out)
        return out
    if 0 < T <= MANY_M:
        kind = choose(T, w, x, False, out_dtype, ctx.err)
        if kind not in ("none", "lib") or (kind == "lib" and T <= SMALL_M):
            out = torch.empty((T, N), dtype=out_dtype, device=x.device)
            _run(kind, x, w, out, False, ctx.err)
            return out
    if out_dtype == x.dtype:
        ops.count_launch()
        return torch.mm(x, w.t())
    out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    if T:
        ops.gemm_nt_plain(x, w, out)
    return out
