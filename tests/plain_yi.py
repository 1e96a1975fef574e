"""Plain, slow implementation of the Yi decoder and of DELTA's page selection.

It is the thing the engine is compared with.  It works on whole sequences,
keeps no cache, has one function per part and shares no code with the
``delta_b200`` package: it has its own reader for the model folder too.

Every function is written from the formulas of hoenza/DELTA; the docstrings
cite the file and line (paths inside that project).  Attention, rotary
positions and the cache append cannot be run from that project on a CPU (its
ops are CUDA only), so those rest on the formulas; RMSNorm, SwiGLU, the fused
QKV row order, the page score and the page selection are also compared once
with the project's own code, see ``tests/golden/make_golden.py``.

All arithmetic is done in ``dtype`` (float32 by default, float64 to measure
the rounding of the float32 one).  ``rounding="bfloat16"`` rounds weights and
every intermediate tensor to bfloat16 at the places where the bfloat16 engine
stores one, which makes a tight comparison with that path possible.
"""
from __future__ import annotations

import json
import math
import struct
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import torch


# --------------------------------------------------------------------------
# model folder (own reader; the engine's loader is not used here)
# --------------------------------------------------------------------------

_ST_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2), "I32": (np.int32, 4), "I64": (np.int64, 8), "F64": (np.float64, 8)}


def read_safetensors_plain(path) -> dict[str, torch.Tensor]:
    """safetensors: u64 little-endian header length, JSON header, raw data."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        npdt, _ = _ST_DTYPES[meta["dtype"]]
        b, e = meta["data_offsets"]
        arr = np.frombuffer(raw[base + b:base + e], dtype=npdt).reshape(meta["shape"]).copy()
        if meta["dtype"] == "BF16":
            t = torch.from_numpy(arr.astype(np.int32) << 16).view(torch.float32)
        else:
            t = torch.from_numpy(arr)
        out[name] = t
    return out


@dataclass
class PlainConfig:
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    eps: float
    theta: float
    interleaved: bool = False
    # per layer: None (all keys) or a window in tokens
    windows: list = field(default_factory=list)
    # order in which layers run: (layer index, index of the cache it reads and writes, writes?)
    plan: list = field(default_factory=list)

    @staticmethod
    def from_folder(folder) -> "PlainConfig":
        c = json.loads((Path(folder) / "config.json").read_text())
        h = c["hidden_size"]
        nh = c["num_attention_heads"]
        nl = c["num_hidden_layers"]
        lt = c.get("layer_types")
        win = c.get("sliding_window")
        windows = [win if (lt is not None and lt[i] == "sliding_attention") else None for i in range(nl)]
        return PlainConfig(
            hidden=h, layers=nl, heads=nh, kv_heads=c.get("num_key_value_heads", nh),
            head_dim=c.get("head_dim") or h // nh, intermediate=c["intermediate_size"],
            vocab=c["vocab_size"], eps=c["rms_norm_eps"], theta=float(c.get("rope_theta", 10000.0)),
            windows=windows, plan=[(i, i, True) for i in range(nl)])


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype)


# --------------------------------------------------------------------------
# the parts, one function each
# --------------------------------------------------------------------------

def embedding(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """x = E[idx]  (DELTA/Engine/DELTA/model.py:199)."""
    return table[tokens.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, rnd=None) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps), then times the weight
    (DELTA/Engine/DELTA/model.py:527-532).  With a rounding function the
    normalised value is rounded before the weight multiply, as the reference's
    ``.type_as(x)`` does at line 531."""
    n = x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    if rnd is not None:
        n = rnd(n)
    return n * w


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float, interleaved: bool) -> torch.Tensor:
    """Rotary positions on x[T, heads, hd] (DELTA/Engine/DELTA/model.py:165-175:
    apply_rope(..., rope_scale=1, rope_theta=theta)).  Pair j has the angle
    pos / theta^(2j/hd).  ``interleaved`` pairs (2j, 2j+1) as the reference does
    on its converted checkpoints; otherwise (j, j+hd/2), which is the same
    function on the unconverted tensor rows of a model folder."""
    hd = x.shape[-1]
    half = hd // 2
    j = torch.arange(half, dtype=torch.float64)
    inv = theta ** (-2.0 * j / hd)
    ang = pos.to(torch.float64)[:, None] * inv[None, :]
    cos = torch.cos(ang).to(x.dtype)[:, None, :]
    sin = torch.sin(ang).to(x.dtype)[:, None, :]
    out = torch.empty_like(x)
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = a * sin + b * cos
    else:
        a, b = x[..., :half], x[..., half:]
        out[..., :half] = a * cos - b * sin
        out[..., half:] = a * sin + b * cos
    return out


def attention_scores(q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
    """s[h, p, t] = (q[p,h] . k[t, h // G]) / sqrt(hd)   (sm_scale explicit at
    DELTA/Engine/DELTA/backend.py:542; grouped heads: model.py:456-459)."""
    T, H, hd = q.shape
    KV = k.shape[1]
    G = H // KV
    kk = k.repeat_interleave(G, dim=1)  # [T, H, hd]
    return torch.einsum("phd,thd->hpt", q, kk) / math.sqrt(hd)


def attention(q, k, v, mask: torch.Tensor):
    """Softmax attention of one whole sequence under a boolean mask [T, T]
    (True = query p may see key t).  Causal masking as the reference asks for it
    (causal=True, DELTA/Engine/DELTA/backend.py:1103) is part of the mask.
    Returns y[T, H, hd] and the scaled scores s[H, T, T]."""
    H = q.shape[1]
    G = H // k.shape[1]
    s = attention_scores(q, k)
    sm = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(sm, dim=-1)
    vv = v.repeat_interleave(G, dim=1)
    y = torch.einsum("hpt,thd->phd", p, vv)
    return y, s


def swiglu(x, w_gate, w_up, w_down, rnd=None):
    """w2(silu(w1 x) * w3 x)   (DELTA/Engine/DELTA/model.py:514)."""
    r = rnd or (lambda t: t)
    g = r(x @ w_gate.T)
    u = r(x @ w_up.T)
    a = r(torch.nn.functional.silu(g) * u)
    return r(a @ w_down.T)


def causal_mask(T: int, window=None) -> torch.Tensor:
    p = torch.arange(T)[:, None]
    t = torch.arange(T)[None, :]
    m = t <= p
    if window is not None:
        m = m & (t > p - window)
    return m


# --------------------------------------------------------------------------
# DELTA: page score and page selection
# --------------------------------------------------------------------------

def page_scores(z: torch.Tensor, seq_len: int, page_size: int) -> torch.Tensor:
    """z[H, seq_len]: scaled scores of one decode query against all its keys.
    p = softmax_t(z) per head; m[t] = max_h p[h,t]; score[j] = sum of m over the
    tokens of page j   (DELTA/Engine/DELTA/backend.py:887-904)."""
    p = torch.softmax(z.to(torch.float32), dim=-1)
    m = p.amax(dim=0)
    n_pages = (seq_len + page_size - 1) // page_size
    pad = n_pages * page_size - seq_len
    if pad:
        m = torch.cat([m, m.new_zeros(pad)])
    return m.reshape(n_pages, page_size).sum(dim=-1)


def select_pages(score: torch.Tensor, n_pages: int, k: int, L: int, bias: float = 1e-7) -> list[int]:
    """DELTA's single top-k selector (DELTA/Engine/DELTA/page_selector_v2.py:113-130
    and 136-150): NaN and -inf to -inf, a position bias of -bias*j, +inf on the
    last L pages, -inf past the request's pages, top-k, indices sorted upwards.
    A request with at most k pages keeps them all (valid count min(n, k),
    line 153).  Ties between finite scores go to the older page; L is clamped
    to k, since a larger L would make the reference pick among equal +inf
    scores arbitrarily."""
    if n_pages <= k:
        return list(range(n_pages))
    L = min(L, k)
    sc = torch.nan_to_num(score[:n_pages].to(torch.float32).clone(), nan=float("-inf"), neginf=float("-inf"))
    j = torch.arange(n_pages, dtype=torch.float32)
    sc = sc + (-j * torch.tensor(bias, dtype=torch.float32))
    sc[max(n_pages - L, 0):n_pages] = float("inf")
    order = sorted(range(n_pages), key=lambda i: (-sc[i].item(), i))
    return sorted(order[:k])


def recent_pages(n_pages: int, k: int) -> list[int]:
    """The subset before any planner has run in a step: the last k pages
    (DELTA/Engine/DELTA/backend.py:1871-1873, 2054-2055)."""
    return list(range(max(n_pages - k, 0), n_pages))


def selection_active(n_pages: int, k: int, ratio: float) -> bool:
    """Per-request form of DELTA/Engine/DELTA/backend.py:1893-1897:
    full pages / subset pages > compression_ratio."""
    return n_pages / min(n_pages, k) > ratio


@dataclass
class Selective:
    full_layers: list  # indices of layers that read the whole cache
    k: int             # pages a subset layer reads
    L: int = 8
    ratio: float = 1.0
    page_size: int = 16
    prompt_len: int = 0  # positions >= prompt_len are decode positions
    # The reference's page accounting: a request whose length has just reached a multiple of the page size
    # already holds the next, still empty page (DELTA/Engine/DELTA/scheduler.py:60-74), which counts among its
    # pages in the selection.  The engine holds ceil(len / page_size) pages; this switch is for comparisons
    # with outputs of the reference itself.
    trailing_empty_page: bool = False

    def pages_at(self, p: int) -> int:
        """Pages the request counts when the token at position p is decoded."""
        return (p + 1) // self.page_size + 1 if self.trailing_empty_page else p // self.page_size + 1

    def role(self, layer: int, n_layers: int) -> str:
        """full / planner / subset   (DELTA/Engine/DELTA/model.py:177-194)."""
        if not self.full_layers:
            return "full"
        if layer in self.full_layers:
            nxt_full = True if layer + 1 >= n_layers else (layer + 1) in self.full_layers
            return "full" if nxt_full else "planner"
        return "subset"


# --------------------------------------------------------------------------
# the whole model
# --------------------------------------------------------------------------

class PlainYi:
    def __init__(self, folder, dtype=torch.float32, rounding: str | None = None, interleaved=False):
        self.cfg = PlainConfig.from_folder(folder)
        self.cfg.interleaved = interleaved
        self.dtype = dtype
        self.rnd = bf16_round if rounding == "bfloat16" else None
        w = read_safetensors_plain(Path(folder) / "model.safetensors")
        self.w = {}
        for n, t in w.items():
            t = t.to(torch.float32)
            if rounding == "bfloat16" and t.dim() == 2:
                t = bf16_round(t)
            self.w[n] = t.to(dtype)
        self.last_selection = {}  # (layer, position) -> list of pages, for the tests

    def _r(self, x):
        return self.rnd(x) if self.rnd is not None else x

    def layer(self, i: int, x: torch.Tensor, pos: torch.Tensor, mask: torch.Tensor, kv_from=None):
        """One pre-norm block: h = x + wo(attn(norm(x))); out = h + mlp(norm(h))
        (DELTA/Engine/DELTA/model.py:338-341).  Returns out, (k, v) and the scaled
        scores."""
        c, w = self.cfg, self.w
        pre = f"model.layers.{i}."
        a = self._r(rms_norm(x, w[pre + "input_layernorm.weight"], c.eps, self.rnd))
        T = x.shape[0]
        q = self._r(a @ w[pre + "self_attn.q_proj.weight"].T).view(T, c.heads, c.head_dim)
        k = self._r(a @ w[pre + "self_attn.k_proj.weight"].T).view(T, c.kv_heads, c.head_dim)
        v = self._r(a @ w[pre + "self_attn.v_proj.weight"].T).view(T, c.kv_heads, c.head_dim)
        q = self._r(rope(q, pos, c.theta, c.interleaved))
        k = self._r(rope(k, pos, c.theta, c.interleaved))
        if kv_from is not None:
            k, v = kv_from
        y, s = attention(q, k, v, mask)
        y = self._r(y).reshape(T, c.heads * c.head_dim)
        h = self._r(x + self._r(y @ w[pre + "self_attn.o_proj.weight"].T))
        f = self._r(rms_norm(h, w[pre + "post_attention_layernorm.weight"], c.eps, self.rnd))
        m = swiglu(f, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"], w[pre + "mlp.down_proj.weight"], self.rnd)
        return self._r(h + m), (k, v), s

    def forward(self, tokens, selective: Selective | None = None, forced: dict | None = None) -> torch.Tensor:
        """Logits [T, V] of one whole sequence (DELTA/Engine/DELTA/model.py:198-206,
        without the argmax of line 323).  With ``selective`` the positions from
        ``prompt_len`` on are decode positions: in subset layers they see only the
        pages chosen for them (DELTA/Engine/DELTA/backend.py:486-516, 787-853)."""
        c, w = self.cfg, self.w
        tokens = torch.as_tensor(tokens)
        T = tokens.shape[0]
        pos = torch.arange(T)
        x = self._r(embedding(w["model.embed_tokens.weight"], tokens))
        ps = selective.page_size if selective else 1
        # chosen[p] = pages that position p sees in subset layers (None: everything)
        chosen = [None] * T
        if selective:
            for p in range(selective.prompt_len, T):
                n = selective.pages_at(p)
                if selection_active(n, selective.k, selective.ratio):
                    chosen[p] = recent_pages(n, selective.k)
        caches = {}
        self.last_selection = {}
        self.last_planned = {}     # (planner layer, position) -> pages it chose
        for (i, cache_id, writes) in c.plan:
            # a layer with a window reads a bounded number of keys already and takes no page selection
            role = selective.role(i, c.layers) if (selective and c.windows[i] is None) else "full"
            mask = causal_mask(T, c.windows[i])
            if role == "subset":
                for p in range(T):
                    if chosen[p] is not None:
                        row = torch.zeros(T, dtype=torch.bool)
                        for j in chosen[p]:
                            row[j * ps:(j + 1) * ps] = True
                        mask[p] &= row
                        self.last_selection[(i, p)] = list(chosen[p])
            x, kv, s = self.layer(i, x, pos, mask, None if writes else caches[cache_id])
            if writes:
                caches[cache_id] = kv
            if role == "planner":
                for p in range(selective.prompt_len, T):
                    n = selective.pages_at(p)
                    if selection_active(n, selective.k, selective.ratio):
                        if forced is not None and (i, p) in forced:
                            # attend to the pages somebody else chose (a comparison in reduced precision,
                            # where two nearly equal page scores may come out in the other order)
                            chosen[p] = list(forced[(i, p)])
                            continue
                        sc = page_scores(s[:, p, :p + 1], p + 1, ps)
                        if sc.shape[0] < n:      # the reference's empty trailing page: no keys, score zero
                            sc = torch.cat([sc, sc.new_zeros(n - sc.shape[0])])
                        chosen[p] = select_pages(sc, n, selective.k, selective.L)
                        self.last_planned[(i, p)] = list(chosen[p])
        x = self._r(rms_norm(x, w["model.norm.weight"], c.eps, self.rnd))
        return (x @ w["lm_head.weight"].T).to(torch.float32)


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

def greedy(logits: torch.Tensor) -> int:
    """argmax over the vocabulary (DELTA/Engine/DELTA/model.py:323); the lowest
    index wins a tie, as torch.argmax does on the CPU."""
    return int(torch.argmax(logits.to(torch.float32)).item())


def temperature_probs(logits: torch.Tensor, temperature: float, top_p: float = 1.0) -> torch.Tensor:
    """softmax(logits / T), after the top-p filter of
    DELTA/Engine/utils.py:81-101: sort downwards, drop the tokens after the
    cumulative probability first exceeds top_p (the first such token is kept)."""
    z = logits.to(torch.float64) / temperature
    if top_p < 1.0:
        sz, idx = torch.sort(z, descending=True)
        cum = torch.cumsum(torch.softmax(sz, dim=-1), dim=-1)
        drop = cum > top_p
        drop[1:] = drop[:-1].clone()
        drop[0] = False
        z = z.clone()
        z[idx[drop]] = float("-inf")
    return torch.softmax(z, dim=-1)
