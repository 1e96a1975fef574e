"""Each CUDA kernel alone against a plain float32 PyTorch reference of the same op, at
sizes other than the engine's tiny models use (head sizes in steps of 16, odd numbers of
heads and groups, widths and vocabularies that are no power of two)."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(1234)


def ops():
    from delta_b200.kernels import ops as o
    return o


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def assert_heads_close(got, ref, H, hd, what="", rel=1e-2):
    """Per (token, head): the difference's norm is at most ``rel`` times the reference's norm.  An
    absolute bound would let a kernel drop a page among hundreds of keys: the output there is a mean
    of many values and small all over."""
    g = got.float().cpu().reshape(-1, H, hd)
    r = ref.float().cpu().reshape(-1, H, hd)
    err = (g - r).norm(dim=-1)
    bad = (err > rel * r.norm(dim=-1) + 1e-6).nonzero()
    if bad.numel():
        t, h = int(bad[0, 0]), int(bad[0, 1])
        raise AssertionError(f"{what}: token {t}, head {h}: |difference| {err[t, h].item():.3e} against |reference| {r[t, h].norm().item():.3e}")


# ------------------------------------------------------------------ elementwise

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(dtype):
    o = ops()
    table = torch.randn(777, 72, device=DEV).to(dtype)
    tok = i32([0, 776, 5, 5, 300])
    out = torch.empty(5, 72, dtype=dtype, device=DEV)
    o.embedding(tok, table, out)
    assert torch.equal(out, table[tok.long()])
    err = o.new_error_record(DEV)
    o.embedding(i32([3, 777]), table, out[:2], err=err)
    with pytest.raises(Exception, match="token id out of range"):
        o.raise_if_error(err)


@pytest.mark.parametrize("dtype, wdtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("d", [48, 1000, 4096])
def test_rms_norm(dtype, wdtype, d):
    o = ops()
    x = torch.randn(7, d, device=DEV).to(dtype)
    add = torch.randn(7, d, device=DEV).to(dtype)
    w = (1 + 0.1 * torch.randn(d, device=DEV)).to(wdtype)
    eps = 3e-6

    def ref(v, cast_first):
        v = v.float()
        n = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
        if cast_first:
            n = n.to(dtype).float()
        return (n * w.float()).to(dtype)

    for cast_first in (False, True):
        out = torch.empty_like(x)
        o.rms_norm(x.clone(), w, eps, out, cast_first=cast_first)
        assert torch.allclose(out.float(), ref(x, cast_first).float(), **tol(dtype))
    # fused residual add on chosen rows: x[rows] += add[rows] in place, the other rows stay
    rows = i32([5, 0, 2])
    xs = x.clone()
    out = torch.empty(3, d, dtype=dtype, device=DEV)
    o.rms_norm(xs, w, eps, out, add=add, rows=rows)
    summed = (x.float() + add.float()).to(dtype)
    assert torch.equal(xs[[5, 0, 2]], summed[[5, 0, 2]]) and torch.equal(xs[[1, 3, 4, 6]], x[[1, 3, 4, 6]])
    assert torch.allclose(out.float(), ref(summed[[5, 0, 2]], False).float(), **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T, I", [(9, 344), (5, 345), (300, 11008), (1, 8)])
def test_silu_mul(dtype, T, I):
    """Widths that take the 16-byte path and one that does not; more rows than one pass of the grid."""
    o = ops()
    gu = (torch.randn(T, 2 * I, device=DEV) * 3).to(dtype)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    o.silu_mul(gu, out)
    g, u = gu[:, :I].float(), gu[:, I:].float()
    assert torch.allclose(out.float(), (torch.nn.functional.silu(g) * u).to(dtype).float(), **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_append(dtype, interleaved):
    from delta_b200.parts.rope import RotaryPositions
    o = ops()
    H, KV, hd, ps, pages = 6, 3, 48, 8, 10
    T = 11
    rope = RotaryPositions(hd, 250000.0, 64, interleaved)
    table = rope.table(torch.device(DEV))
    qkv = torch.randn(T, (H + 2 * KV) * hd, device=DEV).to(dtype)
    pos = [0, 1, 2, 3, 4, 5, 6, 7, 8, 30, 31]      # request 0 crosses a page's edge; request 1 sits at its end
    row = [0] * 9 + [1, 1]
    bt = i32([[7, 2, -1, -1], [4, 9, 1, 5]])
    kv = torch.zeros(pages, 2, KV, ps, hd, dtype=dtype, device=DEV)
    orig = qkv.clone()
    o.rope_append(qkv, i32(pos), i32(row), bt, kv, table, H, KV, hd, ps, interleaved)
    half = hd // 2
    v3 = orig.float().view(T, H + 2 * KV, hd)
    for t in range(T):
        c, s = table[pos[t], :, 0], table[pos[t], :, 1]
        x = v3[t, :H + KV]
        if interleaved:
            a, b = x[:, 0::2], x[:, 1::2]
            r = torch.empty_like(x)
            r[:, 0::2], r[:, 1::2] = a * c - b * s, a * s + b * c
        else:
            a, b = x[:, :half], x[:, half:]
            r = torch.cat([a * c - b * s, a * s + b * c], -1)
        r = r.to(dtype)
        got = qkv[t].view(H + 2 * KV, hd)
        assert torch.allclose(got[:H].float(), r[:H].float(), **tol(dtype))
        page = int(bt[row[t], pos[t] // ps])
        assert torch.allclose(kv[page, 0, :, pos[t] % ps].float(), r[H:].float(), **tol(dtype))
        assert torch.equal(kv[page, 1, :, pos[t] % ps], orig[t].view(H + 2 * KV, hd)[H + KV:])
    assert kv[[0, 3, 6, 8]].abs().sum() == 0            # pages of nobody stay untouched
    # without a table nothing is rotated; without a cache nothing is appended
    q2 = orig.clone()
    o.rope_append(q2, i32(pos), i32(row), bt, None, None, H, KV, hd, ps, interleaved)
    assert torch.equal(q2, orig)
    # a position without a page is reported, not written
    err = o.new_error_record(DEV)
    o.rope_append(orig.clone()[:1], i32([20]), i32([0]), bt, kv, table, H, KV, hd, ps, interleaved, err=err)
    with pytest.raises(Exception, match="page id out of range"):
        o.raise_if_error(err)


# ------------------------------------------------------------------ matrix products

@pytest.mark.parametrize("M, N, K", [(1, 48, 40), (5, 1000, 344), (70, 130, 257), (129, 64, 16)])
def test_gemm_plain_float32_is_true_32_bit(M, N, K):
    o = ops()
    a = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV)
    out = torch.empty(M, N, device=DEV)
    o.gemm_nt_plain(a, w, out)
    ref = (a.double() @ w.double().T)
    assert torch.allclose(out.double(), ref, atol=1e-4, rtol=1e-5)   # a tf32 product would miss this by 1e-2
    # the sum over k does not depend on how many rows share the batch
    one = torch.empty(1, N, device=DEV)
    o.gemm_nt_plain(a[M // 2:M // 2 + 1].contiguous(), w, one)
    assert torch.equal(one[0], out[M // 2])


@pytest.mark.parametrize("M", [1, 3, 8, 9, 17, 33, 64])
@pytest.mark.parametrize("N, K", [(96, 40), (1056, 344), (4096, 4096), (7168, 264)])   # 7,168 rows: the variant held to four blocks per SM
def test_gemm_small_m(M, N, K):
    o = ops()
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().T
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    o.gemm_small_m(x, w, out)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2)
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    o.gemm_small_m(x, w, out32)
    assert torch.allclose(out32, ref, atol=1e-3, rtol=1e-4)
    # SwiGLU epilogue: rows [0, N/2) are the gate, rows [N/2, N) the up projection
    act = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
    o.gemm_small_m(x, w, act, swiglu=True)
    want = torch.nn.functional.silu(ref[:, :N // 2]) * ref[:, N // 2:]
    assert torch.allclose(act.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [1, 8, 17, 64, 100, 128])
@pytest.mark.parametrize("N, K, splits", [(128, 64, 1), (1000, 344, 1), (4096, 4096, 4), (1408, 11008, 8), (2048, 520, 2)])
def test_gemm_tc(M, N, K, splits):
    """The tcgen05/TMA product: one block per 128 weight rows, K shared by a cluster of blocks
    whose partial sums are added over distributed shared memory; sizes that end inside a tile,
    inside a 64-element box and inside a stage of several boxes."""
    o = ops()
    torch.manual_seed(M * 7 + splits)
    err = o.new_error_record(DEV)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().T
    out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(x, w, out, splits=splits, err=err)
    o.raise_if_error(err)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2)
    out32 = torch.full((M, N), 9.0, dtype=torch.float32, device=DEV)
    o.gemm_tc(x, w, out32, splits=splits, err=err)
    o.raise_if_error(err)
    assert torch.allclose(out32, ref, atol=1e-3, rtol=1e-4)
    # the same result whatever the split: float sums of K terms below 0.1 in another order differ
    # by at most about K * 2^-24 * 0.1, which is 7e-5 for the longest K here
    other = torch.empty_like(out32)
    o.gemm_tc(x, w, other, splits=1, err=err)
    o.raise_if_error(err)
    assert torch.allclose(other.float(), ref, atol=2e-2, rtol=1e-2)
    if M <= 64:         # shorter stages, two blocks to an SM
        other.fill_(9.0)
        o.gemm_tc(x, w, other, splits=min(splits, 2), err=err, per_sm=2)
        o.raise_if_error(err)
    assert torch.allclose(other, out32, atol=5e-4, rtol=1e-5)


@pytest.mark.parametrize("M", [3, 64])
@pytest.mark.parametrize("I, K, splits", [(64, 128, 1), (704, 344, 1), (11008, 4096, 2)])
def test_gemm_tc_swiglu(M, I, K, splits):
    o = ops()
    torch.manual_seed(M + I)
    err = o.new_error_record(DEV)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().T
    want = torch.nn.functional.silu(ref[:, :I]) * ref[:, I:]
    act = torch.full((M, I), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(x, w, act, swiglu=True, splits=splits, err=err, per_sm=2 if M == 64 else 1)
    o.raise_if_error(err)
    assert torch.allclose(act.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [129, 200, 256, 257, 600, 2048])
@pytest.mark.parametrize("N, K", [(128, 64), (1000, 344), (4096, 1024), (1408, 520)])
def test_gemm_tc_many_rows(M, N, K):
    """More than 128 rows in chunks of up to 256, one block per (tile, chunk): a chunk that is not
    full, a last chunk of one row, and rows beyond the last that must stay untouched."""
    o = ops()
    torch.manual_seed(M + N)
    err = o.new_error_record(DEV)
    assert o.gemm_tc_many_rows_supported(M, N, K) and not o.gemm_tc_many_rows_supported(128, N, K)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().T
    whole = torch.full((M + 3, N), 9.0, dtype=torch.float32, device=DEV)
    o.gemm_tc(x, w, whole[:M], err=err)
    o.raise_if_error(err)
    assert torch.allclose(whole[:M], ref, atol=1e-3, rtol=1e-4)
    assert bool((whole[M:] == 9.0).all())
    out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(x, w, out, err=err)
    o.raise_if_error(err)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2)
    with pytest.raises(o.KernelError, match="splits=1"):
        o.gemm_tc(x, w, out, splits=2, err=err)
    if N % 128 == 0:
        I = N // 2
        want = torch.nn.functional.silu(ref[:, :I]) * ref[:, I:]
        act = torch.full((M, I), 9.0, dtype=torch.bfloat16, device=DEV)
        o.gemm_tc(x, w, act, swiglu=True, err=err)
        o.raise_if_error(err)
        assert torch.allclose(act.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [1, 8, 17, 64, 100, 128])
@pytest.mark.parametrize("N, K", [(128, 64), (1000, 344), (4096, 4096), (1408, 11008), (2048, 520), (20000, 256)])
def test_gemm_stream_k(M, N, K):
    """The persistent tcgen05 product: the (tile, K step) sequence in one equal piece per SM.  One
    piece for the whole product; tiles shared by three and by six blocks; pieces of many whole
    tiles with a shared tile at either end; sizes that end inside a tile, a box and a step.  The
    second and third launch use the same workspace (flags carry the launch's number) and give the
    same bits."""
    o = ops()
    torch.manual_seed(M * 5 + N)
    err = o.new_error_record(DEV)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().T
    out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_stream_k(x, w, out, err=err)
    o.raise_if_error(err)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2)
    out32 = torch.full((M, N), 9.0, dtype=torch.float32, device=DEV)
    o.gemm_stream_k(x, w, out32, err=err)
    o.raise_if_error(err)
    assert torch.allclose(out32, ref, atol=1e-3, rtol=1e-4)
    again = torch.full((M, N), 9.0, dtype=torch.float32, device=DEV)
    o.gemm_stream_k(x, w, again, err=err)
    o.raise_if_error(err)
    assert torch.equal(again, out32)


@pytest.mark.parametrize("M", [3, 64])
@pytest.mark.parametrize("I, K", [(64, 128), (704, 344), (11008, 4096)])
def test_gemm_stream_k_swiglu(M, I, K):
    o = ops()
    torch.manual_seed(M + I)
    err = o.new_error_record(DEV)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().T
    want = torch.nn.functional.silu(ref[:, :I]) * ref[:, I:]
    act = torch.full((M, I), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_stream_k(x, w, act, swiglu=True, err=err)
    o.raise_if_error(err)
    assert torch.allclose(act.float(), want, atol=2e-2, rtol=2e-2)


def test_gemm_small_m_refuses_what_it_does_not_take():
    o = ops()
    assert not o.gemm_small_m_supported(65, 64, 64)
    assert not o.gemm_small_m_supported(4, 50, 64)      # columns no multiple of 16
    assert not o.gemm_small_m_supported(4, 64, 36)      # K no multiple of 8
    x = torch.zeros(4, 36, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 36, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception, match="sizes not taken"):
        o.gemm_small_m(x, w, torch.empty(4, 64, dtype=torch.bfloat16, device=DEV))


# ------------------------------------------------------------------ attention

class PagedCase:
    """Random requests in a random paged cache, with the plain float32 answer."""

    def __init__(self, dtype, H, KV, hd, ps, seq_lens, q_lens, seed=0, scatter=True, counting=False):
        """``counting``: queries are zero, so every key a row may read weighs the same, and the value of
        a key is the unit vector of its page's number (modulo the head size): the output then counts,
        exactly, how many keys of which pages were read."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.dtype, self.H, self.KV, self.hd, self.ps = dtype, H, KV, hd, ps
        self.seq_lens, self.q_lens = seq_lens, q_lens
        B = len(seq_lens)
        max_pages = max((n + ps - 1) // ps for n in seq_lens) + 1
        total = sum((n + ps - 1) // ps for n in seq_lens)
        ids = list(range(total + 3))
        if scatter:
            random.Random(seed).shuffle(ids)
        self.k = [torch.randn(n, KV, hd, generator=g).to(dtype) for n in seq_lens]
        self.v = [torch.randn(n, KV, hd, generator=g).to(dtype) for n in seq_lens]
        self.q = [torch.randn(ql, H, hd, generator=g).to(dtype) for ql in q_lens]
        if counting:
            self.q = [torch.zeros_like(q) for q in self.q]
            self.v = [torch.nn.functional.one_hot((torch.arange(n) // ps) % hd, hd).to(dtype)[:, None, :].repeat(1, KV, 1)
                      for n in seq_lens]
        kv = torch.zeros(total + 3, 2, KV, ps, hd, dtype=dtype)
        bt = torch.full((B, max_pages), -1, dtype=torch.int32)
        nxt = 0
        for b, n in enumerate(seq_lens):
            for lp in range((n + ps - 1) // ps):
                page = ids[nxt]
                nxt += 1
                bt[b, lp] = page
                cnt = min(ps, n - lp * ps)
                kv[page, 0, :, :cnt] = self.k[b][lp * ps:lp * ps + cnt].transpose(0, 1)
                kv[page, 1, :, :cnt] = self.v[b][lp * ps:lp * ps + cnt].transpose(0, 1)
        self.kv, self.bt = kv.to(DEV), bt.to(DEV)
        tok_row, tok_pos, q_start = [], [], []
        for b, (n, ql) in enumerate(zip(seq_lens, q_lens)):
            q_start.append(len(tok_row))
            tok_row += [b] * ql
            tok_pos += list(range(n - ql, n))
        self.tok_row, self.tok_pos = i32(tok_row), i32(tok_pos)
        self.row_q_start, self.row_q_len = i32(q_start), i32(q_lens)
        self.row_pos_start = i32([n - ql for n, ql in zip(seq_lens, q_lens)])
        self.row_slot = i32(list(range(B)))
        self.qcat = torch.cat(self.q).reshape(-1, H * hd).contiguous().to(DEV)
        self.T = len(tok_row)

    def params(self, out, **kw):
        return ops().make_attn_params(
            q=self.qcat, q_stride=self.H * self.hd, out=out, kv=self.kv, block_table=self.bt, tok_row=self.tok_row,
            tok_pos=self.tok_pos, H=self.H, KV=self.KV, hd=self.hd, ps=self.ps, scale=1.0 / math.sqrt(self.hd),
            row_slot=self.row_slot, row_q_start=self.row_q_start, row_q_len=self.row_q_len,
            row_pos_start=self.row_pos_start, **kw)

    def reference(self, window=0, pages=None):
        """float32 answer; ``pages[b]``: the logical pages row b may read (None: all)."""
        outs, lses, scores = [], [], []
        G = self.H // self.KV
        for b, (n, ql) in enumerate(zip(self.seq_lens, self.q_lens)):
            k = self.k[b].float().repeat_interleave(G, 1)
            v = self.v[b].float().repeat_interleave(G, 1)
            q = self.q[b].float()
            s = torch.einsum("phd,thd->hpt", q, k) / math.sqrt(self.hd)
            p_abs = torch.arange(n - ql, n)[:, None]
            t = torch.arange(n)[None, :]
            mask = t <= p_abs
            if window:
                mask &= t > p_abs - window
            if pages is not None and pages[b] is not None:
                allowed = torch.zeros(n, dtype=torch.bool)
                for lp in pages[b]:
                    allowed[lp * self.ps:(lp + 1) * self.ps] = True
                mask &= allowed[None, :]
            sm = s.masked_fill(~mask[None], float("-inf"))
            outs.append(torch.einsum("hpt,thd->phd", torch.softmax(sm, -1), v).reshape(ql, -1))
            lses.append(torch.logsumexp(sm, -1).T)
            scores.append(s)
        return torch.cat(outs), torch.cat(lses), scores


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, KV, hd, ps", [(6, 3, 48, 8), (5, 5, 16, 32), (8, 1, 128, 16), (4, 2, 208, 64)])
def test_attention_plain(dtype, H, KV, hd, ps):
    o = ops()
    case = PagedCase(dtype, H, KV, hd, ps, seq_lens=[1, 37, 200, 129], q_lens=[1, 5, 64, 2], seed=H)
    out = torch.empty(case.T, H * hd, dtype=dtype, device=DEV)
    lse = torch.empty(case.T, H, device=DEV)
    o.attention_plain(case.params(out, lse=lse))
    ref, ref_lse, _ = case.reference()
    assert torch.allclose(out.float().cpu(), ref, **tol(dtype))
    assert torch.allclose(lse.cpu(), ref_lse, atol=1e-4 if dtype == torch.float32 else 2e-2, rtol=1e-4)
    # a window whose edge falls inside a page
    out2 = torch.empty_like(out)
    o.attention_plain(case.params(out2, window=ps + 3))
    ref2, _, _ = case.reference(window=ps + 3)
    assert torch.allclose(out2.float().cpu(), ref2, **tol(dtype))


def make_far_key_stand_out(case, b, far, h):
    """Scales one key so that head h's last query of request b attends to position ``far`` alone."""
    g = h // (case.H // case.KV)
    q = case.q[b][-1, h].float()
    case.k[b][far, g] = (q / q.norm() * 60.0).to(case.dtype)
    lp, off = far // case.ps, far % case.ps
    page = int(case.bt[b, lp])
    case.kv[page, 0, g, off] = case.k[b][far, g].to(DEV)


@pytest.mark.parametrize("pages", ["scattered", "runs", "scattered, told so"])
@pytest.mark.parametrize("G, KV, hd, ps", [(8, 4, 128, 16), (1, 3, 64, 8), (16, 1, 128, 64), (5, 2, 64, 32), (4, 2, 128, 16)])
def test_attention_decode_against_plain(G, KV, hd, ps, pages):
    """The split-key tensor-core kernel against the plain kernel and the float32 answer:
    contexts from one key to hundreds, ends of pages, a far key that dominates.  With pages in
    runs the kernel fetches whole tiles by TMA, with scattered pages by cp.async in the same
    layout; told that the pages are scattered it runs its variant without TMA."""
    o = ops()
    H = G * KV
    dtype = torch.bfloat16
    seq_lens = [1, ps, ps + 1, 63, 64, 65, 400, 1000]
    case = PagedCase(dtype, H, KV, hd, ps, seq_lens, [1] * len(seq_lens), seed=G + hd, scatter=pages != "runs")
    if pages == "scattered, told so":
        inner = case.params

        def told(out, **kw):
            p = inner(out, **kw)
            p.reserved = 1
            return p
        case.params = told
    make_far_key_stand_out(case, 7, 3, H - 1)        # among 1000 keys, the fourth one wins for the last head
    ref, ref_lse, _ = case.reference()
    assert ref[7].view(H, hd)[H - 1].sub(case.v[7][3, KV - 1].float()).abs().max() < 1e-3
    plain = torch.empty(case.T, H * hd, dtype=dtype, device=DEV)
    o.attention_plain(case.params(plain))
    for splits in (1, 2, 5, 16):
        out = torch.empty_like(plain)
        lse = torch.empty(case.T, H, device=DEV)
        n = o.attention_decode_scratch_floats(case.T, H, hd, splits)
        scratch = torch.empty(max(n, 1), device=DEV)
        p = case.params(out, lse=lse, scratch=scratch, splits=splits)
        o.attention_decode(p)
        assert_heads_close(out, ref, H, hd, f"splits={splits}")
        assert_heads_close(out, plain, H, hd, f"splits={splits}, against the plain kernel")
        assert torch.allclose(lse.cpu(), ref_lse, atol=1e-3, rtol=1e-5)
    # a window whose edge lies inside a page, and beyond the first pages
    out = torch.empty_like(plain)
    scratch = torch.empty(o.attention_decode_scratch_floats(case.T, H, hd, 3), device=DEV)
    o.attention_decode(case.params(out, window=ps + 5, scratch=scratch, splits=3))
    refw, _, _ = case.reference(window=ps + 5)
    assert_heads_close(out, refw, H, hd, "window")


@pytest.mark.parametrize("kernel", ["mma_sync", "tcgen05"])
def test_attention_prefill_among_many_single_tokens(kernel):
    """A step of many single tokens (the decode kernel's) with the rows that bring several tokens in their midst:
    the prefill kernels take exactly those rows, wherever they stand, and leave the others alone."""
    o = ops()
    H, KV, hd, ps = 8, 2, 128, 16
    q_lens = [1] * 9 + [300] + [1] * 5 + [2] + [1] * 20 + [131] + [1] * 3
    seq_lens = [50 + 7 * i for i in range(len(q_lens))]
    for i, q in enumerate(q_lens):
        seq_lens[i] = max(seq_lens[i], q)
    case = PagedCase(torch.bfloat16, H, KV, hd, ps, seq_lens, q_lens, seed=5, scatter=True)
    ref, _, _ = case.reference()
    prefill = o.attention_prefill if kernel == "mma_sync" else o.attention_prefill_tc
    err = o.new_error_record(DEV)
    out = torch.full((case.T, H * hd), 9.0, dtype=torch.bfloat16, device=DEV)
    prefill(case.params(out, row_filter=2, err=err), max(q_lens))
    o.raise_if_error(err)
    starts = [sum(q_lens[:i]) for i in range(len(q_lens))]
    single = torch.tensor([s for s, q in zip(starts, q_lens) if q == 1], device=DEV)
    several = torch.tensor([s + j for s, q in zip(starts, q_lens) if q > 1 for j in range(q)], device=DEV)
    assert bool((out[single] == 9.0).all()), "a single token's output was written"
    assert_heads_close(out[several], ref[several.cpu()], H, hd, kernel)


@pytest.mark.parametrize("pages", ["scattered, told so", "runs"])
@pytest.mark.parametrize("G, KV, hd, ps", [(8, 4, 128, 16), (1, 3, 64, 8), (16, 1, 128, 64), (5, 2, 64, 32)])
def test_attention_decode_splits_merged_by_a_cluster(G, KV, hd, ps, pages):
    """Two to eight splits launched as one thread-block cluster, which merges them over distributed shared
    memory, give the bits of the same splits merged by the second kernel: outputs and log-sum-exp, whole
    contexts, a window, chosen pages, the score dump; requests shorter than the splits leave blocks empty."""
    o = ops()
    H = G * KV
    seq_lens = [1, ps + 1, 63, 64, 65, 400, 1000, 2500]
    B = len(seq_lens)
    case = PagedCase(torch.bfloat16, H, KV, hd, ps, seq_lens, [1] * B, seed=G + hd + 1, scatter=pages != "runs")
    ref, ref_lse, _ = case.reference()
    k = 12
    flags = i32([1] * B)
    sel_pages = torch.zeros(B, k, dtype=torch.int32, device=DEV)
    sel_count = torch.full((B,), -1, dtype=torch.int32, device=DEV)
    for b, n in enumerate(seq_lens):
        npg = (n + ps - 1) // ps
        if npg > k:
            chosen = sorted(random.Random(b).sample(range(npg - 1), k - 1) + [npg - 1])
            sel_pages[b] = i32(chosen)
            sel_count[b] = k
    variants = [dict(), dict(window=ps + 5), dict(row_flags=flags, sel_pages=sel_pages, sel_count=sel_count)]
    if pages != "runs":
        variants.append(dict(row_flags=flags, dump=True))
    for splits in (2, 3, 5, 8):
        scratch = torch.empty(o.attention_decode_scratch_floats(B, H, hd, splits), device=DEV)
        for kw in variants:
            got = {}
            for cluster in (False, True):
                kw2 = dict(kw)
                dump = None
                if kw2.pop("dump", False):
                    dump = torch.full((B, H, 2560), float("nan"), device=DEV)
                    kw2["dump"] = dump
                out = torch.full((B, H * hd), 9.0, dtype=torch.bfloat16, device=DEV)
                lse = torch.full((B, H), 9.0, device=DEV)
                p = case.params(out, lse=lse, scratch=None if cluster else scratch, splits=splits, **kw2)
                p.reserved = (1 if pages != "runs" else 0) | (2 if cluster else 0)
                o.attention_decode(p)
                got[cluster] = (out, lse, dump)
            what = f"splits={splits}, {sorted(kw)}"
            assert torch.equal(got[True][0], got[False][0]), what
            assert torch.equal(got[True][1], got[False][1]), what + ": log-sum-exp"
            if got[True][2] is not None:
                assert torch.equal(torch.nan_to_num(got[True][2], nan=-7.0), torch.nan_to_num(got[False][2], nan=-7.0)), what + ": dump"
            if not kw:
                assert_heads_close(got[True][0], ref, H, hd, what)
                assert torch.allclose(got[True][1].cpu(), ref_lse, atol=1e-3, rtol=1e-5)
    with pytest.raises(o.KernelError, match="at most 8 splits"):
        p = case.params(torch.empty((B, H * hd), dtype=torch.bfloat16, device=DEV), splits=9)
        p.reserved = 2
        o.attention_decode(p)


@pytest.mark.parametrize("kernel", ["mma_sync", "tcgen05", "tcgen05_runs"])
@pytest.mark.parametrize("H, KV, hd, ps", [(8, 2, 128, 16), (3, 3, 64, 8), (4, 1, 64, 64), (32, 4, 128, 32)])
def test_attention_prefill_against_plain(H, KV, hd, ps, kernel):
    """The two tiled tensor-core prefill kernels (warp-level MMA with 64-query tiles; tcgen05 with
    128-query tiles and accumulators in tensor memory): whole prompts, portions that start inside
    a page, tiles that end before a page does, single tokens left to the decode kernel."""
    o = ops()
    dtype = torch.bfloat16
    prefill = o.attention_prefill if kernel == "mma_sync" else o.attention_prefill_tc
    if kernel != "mma_sync":
        assert o.attention_prefill_tc_supported(dtype, H, KV, hd, ps, H * hd)
    seq_lens = [200, 129, 64, 300, 1000, 65, 1]
    q_lens = [200, 5, 64, 2, 37, 1, 1]
    # "runs": a request's pages follow one another in the pool, which the tcgen05 kernel fetches
    # with one copy per tile; else the pages are scattered and fetched one by one
    case = PagedCase(dtype, H, KV, hd, ps, seq_lens, q_lens, seed=H + ps, scatter=kernel != "tcgen05_runs")
    make_far_key_stand_out(case, 4, 2, 0)            # the last query of request 4 looks far back
    ref, ref_lse, _ = case.reference()
    out = torch.zeros(case.T, H * hd, dtype=dtype, device=DEV)
    lse = torch.zeros(case.T, H, device=DEV)
    err = o.new_error_record(DEV)
    prefill(case.params(out, lse=lse, err=err), max(q_lens))
    assert err.cpu().tolist() == [0, 0, 0, 0]
    assert_heads_close(out, ref, H, hd, kernel)
    assert torch.allclose(lse.cpu(), ref_lse, atol=1e-3, rtol=1e-5)
    # single tokens are skipped with row_filter 2 and taken by the decode kernel with row_filter 1
    out2 = torch.zeros_like(out)
    prefill(case.params(out2, row_filter=2), max(q_lens))
    singles = [sum(q_lens[:5]), sum(q_lens[:6])]
    assert out2[singles].abs().sum() == 0
    if H // KV <= 16:
        scratch = torch.empty(o.attention_decode_scratch_floats(len(seq_lens), H, hd, 2), device=DEV)
        o.attention_decode(case.params(out2, row_filter=1, scratch=scratch, splits=2))
    else:
        out2[singles] = out[singles]
    assert_heads_close(out2, ref, H, hd, "singles by the decode kernel")
    # a window whose edge lies inside a tile and inside a page
    out3 = torch.zeros_like(out)
    prefill(case.params(out3, window=ps + 7), max(q_lens))
    refw, _, _ = case.reference(window=ps + 7)
    assert_heads_close(out3, refw, H, hd, "window inside a tile")
    # a window of several tiles, whose far edge lies inside a tile
    out4 = torch.zeros_like(out)
    prefill(case.params(out4, window=300), max(q_lens))
    refw, _, _ = case.reference(window=300)
    assert_heads_close(out4, refw, H, hd, "window of several tiles")


def test_attention_prefill_tc_long_rows_and_maximum_that_grows():
    """The tcgen05 prefill kernel over many tiles: a long cached prefix, scores that grow along
    the row (so the accumulators in tensor memory are rescaled more than once), and one far key
    that outweighs everything after it."""
    o = ops()
    H, KV, hd, ps = 4, 2, 128, 16
    seq_lens, q_lens = [1500, 700], [333, 700]
    case = PagedCase(torch.bfloat16, H, KV, hd, ps, seq_lens, q_lens, seed=11)
    # keys grow with their position in request 1: later tiles bring larger maxima
    ramp = torch.linspace(0.2, 3.0, seq_lens[1])[:, None, None]
    case.k[1] = (case.k[1].float() * ramp).to(torch.bfloat16)
    for lp in range((seq_lens[1] + ps - 1) // ps):
        cnt = min(ps, seq_lens[1] - lp * ps)
        case.kv[case.bt[1, lp], 0, :, :cnt] = case.k[1][lp * ps:lp * ps + cnt].transpose(0, 1).to(DEV)
    make_far_key_stand_out(case, 0, 1, 3)
    ref, ref_lse, _ = case.reference()
    out = torch.zeros(case.T, H * hd, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(case.T, H, device=DEV)
    err = o.new_error_record(DEV)
    o.attention_prefill_tc(case.params(out, lse=lse, err=err), max(q_lens))
    assert err.cpu().tolist() == [0, 0, 0, 0]
    assert_heads_close(out, ref, H, hd, "long rows")
    assert torch.allclose(lse.cpu(), ref_lse, atol=1e-3, rtol=1e-5)


@pytest.mark.parametrize("G, KV, hd, ps", [(8, 4, 128, 16), (3, 2, 64, 8), (16, 1, 128, 32)])
def test_attention_decode_fused_rope_and_append(G, KV, hd, ps):
    """The decode kernel that rotates q and k and appends the new token itself against the
    separate rotary/append kernel followed by the plain decode kernel: same cache, same output."""
    from delta_b200.parts.rope import RotaryPositions
    o = ops()
    H = G * KV
    dtype = torch.bfloat16
    seq_lens = [1, ps, ps + 1, 64, 65, 300, 777]          # the new token opens a page, ends one, sits inside one
    B = len(seq_lens)
    case = PagedCase(dtype, H, KV, hd, ps, seq_lens, [1] * B, seed=G)
    table = RotaryPositions(hd, 5000000.0, 1024).table(torch.device(DEV))
    qkv = torch.randn(B, (H + 2 * KV) * hd, device=DEV).to(dtype)
    for b, n in enumerate(seq_lens):                       # the newest key and value are not in the cache yet
        page = int(case.bt[b, (n - 1) // ps])
        case.kv[page, :, :, (n - 1) % ps] = 0
    def params(out, kv, **kw):
        return o.make_attn_params(q=qkv_in, q_stride=qkv.shape[1], out=out, kv=kv, block_table=case.bt, tok_row=case.tok_row,
                                  tok_pos=case.tok_pos, H=H, KV=KV, hd=hd, ps=ps, scale=1.0 / math.sqrt(hd), row_slot=case.row_slot,
                                  row_q_start=case.row_q_start, row_q_len=case.row_q_len, row_pos_start=case.row_pos_start, **kw)
    for splits in (1, 4):
        scratch = torch.zeros(max(1, o.attention_decode_scratch_floats(B, H, hd, splits)), device=DEV)
        # separate kernels
        qkv_in, kv_a = qkv.clone(), case.kv.clone()
        o.rope_append(qkv_in, case.tok_pos, case.tok_row, case.bt, kv_a, table, H, KV, hd, ps, False)
        want = torch.zeros(B, H * hd, dtype=dtype, device=DEV)
        o.attention_decode(params(want, kv_a, scratch=scratch, splits=splits))
        # fused
        qkv_in, kv_b = qkv.clone(), case.kv.clone()
        got = torch.zeros_like(want)
        o.attention_decode(params(got, kv_b, scratch=scratch, splits=splits, fuse=2, rope_table=table))
        assert torch.equal(kv_a, kv_b), f"splits={splits}: the caches differ"
        assert torch.equal(got, want), f"splits={splits}"
        assert torch.equal(qkv_in, qkv)                    # the fused kernel leaves its input rows alone
        # fuse=1 rotates q but appends nothing (a layer that reads another layer's cache)
        kv_c = kv_a.clone()
        got1 = torch.zeros_like(want)
        o.attention_decode(params(got1, kv_c, scratch=scratch, splits=splits, fuse=1, rope_table=table))
        assert torch.equal(kv_c, kv_a) and torch.equal(got1, want)


@pytest.mark.parametrize("kernel", ["plain", "decode"])
def test_attention_on_chosen_pages_and_score_dump(kernel):
    """Rows flagged for selection read only their chosen pages; a planner's dump holds the
    scaled scores of every key and the log-sum-exp."""
    o = ops()
    H, KV, hd, ps, k = 8, 2, 64, 16, 3
    dtype = torch.bfloat16
    seq_lens = [200, 90, 33, 300]
    B = len(seq_lens)
    case = PagedCase(dtype, H, KV, hd, ps, seq_lens, [1] * B, seed=5)
    flags = i32([1, 1, 0, 1])
    slots = [2, 0, 3, 1]
    case.row_slot = i32(slots)
    sel_pages = torch.zeros(4, k, dtype=torch.int32, device=DEV)
    sel_count = torch.full((4,), -1, dtype=torch.int32, device=DEV)
    chosen = {0: [1, 7, 12], 1: None, 2: None, 3: [0, 9, 18]}       # row 1: flagged but reads everything (count -1)
    for b, pg in chosen.items():
        if pg is not None:
            sel_pages[slots[b]] = i32(pg)
            sel_count[slots[b]] = k
    run = o.attention_plain if kernel == "plain" else o.attention_decode
    out = torch.empty(B, H * hd, dtype=dtype, device=DEV)
    scratch = torch.empty(max(1, o.attention_decode_scratch_floats(B, H, hd, 2)), device=DEV)
    run(case.params(out, row_flags=flags, sel_pages=sel_pages, sel_count=sel_count, scratch=scratch, splits=2 if kernel == "decode" else 0))
    ref, _, _ = case.reference(pages=[chosen[b] for b in range(B)])
    assert_heads_close(out, ref, H, hd, "chosen pages")
    # the dump of a planner layer
    stride = 304
    dump = torch.full((B, H, stride), float("nan"), device=DEV)
    lse = torch.empty(B, H, device=DEV)
    run(case.params(out, row_flags=flags, dump=dump, lse=lse, scratch=scratch, splits=2 if kernel == "decode" else 0))
    ref, ref_lse, scores = case.reference()
    assert_heads_close(out, ref, H, hd, "with a dump")
    for b, n in enumerate(seq_lens):
        if b == 2:
            assert torch.isnan(dump[b]).all()                       # not flagged: nothing is dumped
        else:
            assert torch.allclose(dump[b, :, :n].cpu(), scores[b][:, 0, :], atol=2e-2, rtol=2e-2)
            assert torch.isnan(dump[b, :, n:]).all()
    assert torch.allclose(lse.cpu(), ref_lse, atol=2e-2, rtol=1e-3)


# ------------------------------------------------------------------ DELTA

def test_recent_pages_scores_and_selection():
    from plain_yi import page_scores as plain_scores, select_pages as plain_select
    o = ops()
    ps, k, H = 8, 4, 6
    seqs = [100, 17, 33, 64]          # 13, 3, 5, 8 pages
    B = len(seqs)
    flags = i32([1, 1, 1, 0])
    slots = i32([3, 1, 0, 2])
    pos_start = i32([n - 1 for n in seqs])
    q_len = i32([1] * B)
    q_start = i32(list(range(B)))
    sel_pages = torch.zeros(4, k, dtype=torch.int32, device=DEV)
    sel_count = torch.zeros(4, dtype=torch.int32, device=DEV)
    o.recent_pages(slots, flags, pos_start, q_len, sel_pages, sel_count, ps, 1.0)
    assert sel_count.tolist() == [k, -1, -1, k]                     # slots 0 (5 pages) and 3 (13 pages) select
    assert sel_pages[3].tolist() == [9, 10, 11, 12] and sel_pages[0].tolist() == [1, 2, 3, 4]
    o.recent_pages(slots, flags, pos_start, q_len, sel_pages, sel_count, ps, 1.5)
    assert sel_count.tolist() == [-1, -1, -1, k]                    # 5 / 4 is below the ratio 1.5

    stride = 104
    z = torch.randn(B, H, stride, device=DEV) * 2
    lse = torch.stack([torch.logsumexp(z[b, :, :n], -1) for b, n in enumerate(seqs)])
    scores = torch.full((B, 16), float("nan"), device=DEV)
    o.page_scores(z, lse, flags, q_start, pos_start, q_len, scores, ps, k, 1.0)
    for b, n in enumerate(seqs):
        npg = (n + ps - 1) // ps
        if b in (0, 2):
            want = plain_scores(z[b, :, :n].cpu(), n, ps)
            assert torch.allclose(scores[b, :npg].cpu(), want, atol=1e-6, rtol=1e-4)
        else:
            assert torch.isnan(scores[b]).all()                     # short or unflagged rows are left alone
    # make ties and a NaN, then select
    scores[0, 2] = scores[0, 5]
    scores[2, 0] = float("nan")
    for keep_last in (1, 2, 4):
        o.recent_pages(slots, flags, pos_start, q_len, sel_pages, sel_count, ps, 1.0)
        o.select_pages(scores, slots, flags, pos_start, q_len, sel_pages, sel_count, keep_last, ps, 1e-7, 1.0)
        for b in (0, 2):
            npg = (seqs[b] + ps - 1) // ps
            want = plain_select(scores[b].cpu(), npg, k, keep_last)
            s = int(slots[b])
            assert sel_count[s] == k and sel_pages[s].tolist() == want, (keep_last, b)


def test_selection_with_the_page_counted_ahead():
    """Requests whose newest page is exactly full count one more, empty page: it scores zero, takes a place
    among the newest L, and is left out of the list; a request of the block table's full width (the
    counted page would lie behind the table) and one with a partly filled page beside them."""
    from plain_yi import select_pages as plain_select
    o = ops()
    ps, k, H, max_pages = 8, 4, 3, 16
    seqs = [128, 64, 61, 40]          # 16 pages (+1 counted), 8 (+1), 8, 5 (+1)
    B = len(seqs)
    flags, slots = i32([1] * B), i32([2, 0, 3, 1])
    pos_start, q_len, q_start = i32([n - 1 for n in seqs]), i32([1] * B), i32(list(range(B)))
    sel_pages = torch.full((4, k), -7, dtype=torch.int32, device=DEV)
    sel_count = torch.zeros(4, dtype=torch.int32, device=DEV)
    o.recent_pages(slots, flags, pos_start, q_len, sel_pages, sel_count, ps, 1.0, page_ahead=True)
    assert sel_count.tolist() == [k - 1, k - 1, k - 1, k]
    assert sel_pages[2, :3].tolist() == [13, 14, 15] and sel_pages[0, :3].tolist() == [5, 6, 7]
    assert sel_pages[3].tolist() == [4, 5, 6, 7] and sel_pages[1, :3].tolist() == [2, 3, 4]
    z = torch.randn(B, H, max_pages * ps, device=DEV) * 2
    lse = torch.stack([torch.logsumexp(z[b, :, :n], -1) for b, n in enumerate(seqs)])
    scores = torch.full((B, max_pages), float("nan"), device=DEV)
    o.page_scores(z, lse, flags, q_start, pos_start, q_len, scores, ps, k, 1.0, page_ahead=True)
    for b, n in enumerate(seqs):
        held = (n + ps - 1) // ps
        assert not torch.isnan(scores[b, :held]).any() and torch.isnan(scores[b, held:]).all()
    for keep_last in (2, 3, 4):
        o.select_pages(scores, slots, flags, pos_start, q_len, sel_pages, sel_count, keep_last, ps, 1e-7, 1.0, page_ahead=True)
        for b, n in enumerate(seqs):
            held, counted = (n + ps - 1) // ps, n // ps + 1
            sc = torch.cat([scores[b, :held].cpu(), torch.zeros(counted - held)])
            want = [j for j in plain_select(sc, counted, k, keep_last) if j < held]
            s = int(slots[b])
            assert len(want) == k - (counted - held)
            assert sel_count[s] == len(want) and sel_pages[s, :len(want)].tolist() == want, (keep_last, b)


# ------------------------------------------------------------------ sampling

def test_greedy_takes_the_lowest_index_among_equals():
    o = ops()
    logits = torch.randn(5, 64000, device=DEV)
    logits[1, 777] = logits[1, 50000] = 9.0
    logits[3, 63999] = 11.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    o.sample(logits, out)
    want = torch.argmax(logits, -1).tolist()
    want[1] = 777
    assert out.tolist() == want


def test_temperature_and_top_p():
    from delta_b200.sampling import uniform_of
    from plain_yi import temperature_probs
    o = ops()
    V, R = 1000, 64
    logits = torch.randn(R, V, device=DEV) * 3
    temps = torch.full((R,), 0.7, device=DEV)
    seeds = torch.arange(R, dtype=torch.int64, device=DEV) * 7919
    pos = torch.arange(R, dtype=torch.int32, device=DEV) + 5
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    o.sample(logits, out, temperature=temps, seeds=seeds, positions=pos)
    for r in range(R):
        cdf = torch.cumsum(temperature_probs(logits[r].cpu(), 0.7), 0)
        u = uniform_of(int(seeds[r]), int(pos[r]))
        t = int(out[r])
        assert (cdf[t - 1].item() if t else 0.0) - 1e-5 <= u <= cdf[t].item() + 1e-5
    # top-p: every draw lies in the kept set of the plain filter, and the draw follows the renormalised distribution
    top_p = torch.full((R,), 0.6, device=DEV)
    o.sample(logits, out, temperature=temps, top_p=top_p, seeds=seeds, positions=pos)
    for r in range(R):
        probs = temperature_probs(logits[r].cpu(), 0.7, top_p=0.6)
        t = int(out[r])
        assert probs[t] > 0
        cdf = torch.cumsum(probs, 0)
        u = uniform_of(int(seeds[r]), int(pos[r]))
        assert (cdf[t - 1].item() if t else 0.0) - 1e-4 <= u <= cdf[t].item() + 1e-4
    # many draws of one row follow its distribution
    row = torch.tensor([[2.0, 1.0, 0.0, -1.0] + [-30.0] * 12], device=DEV).repeat(4000, 1)
    out = torch.empty(4000, dtype=torch.int32, device=DEV)
    o.sample(row, out, temperature=torch.ones(4000, device=DEV), seeds=torch.full((4000,), 42, dtype=torch.int64, device=DEV),
             positions=torch.arange(4000, dtype=torch.int32, device=DEV))
    freq = torch.bincount(out.long().cpu(), minlength=16)[:4].float() / 4000
    want = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]), 0)
    assert (freq - want).abs().max() < 0.03


def test_product_tuner_keeps_the_preferred_kernel_within_the_margin(monkeypatch):
    """The tuner's rule with made-up times: a later candidate replaces an earlier one only when it
    is faster by more than the margin; every candidate it names really runs and gives the product."""
    from delta_b200.parts import linear
    o = ops()
    err = o.new_error_record(DEV)
    M, N, K = 16, 512, 256
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    cands = linear._candidates(M, N, K, False, torch.bfloat16)
    assert cands[0] == "small" and cands[-1] == "sk" and "lib" in cands and "tc1" in cands
    ref = x.float() @ w.float().T
    for kind in cands:
        out = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=DEV)
        linear._run(kind, x, w, out, False, err)
        o.raise_if_error(err)
        assert torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2), kind

    def tuned(times):
        order = iter(times)
        monkeypatch.setattr(linear, "_time", lambda fn, reps=12: next(order))
        return linear._tune(M, x, w, False, torch.bfloat16, err)

    n = len(cands)
    assert linear.margin(20.0) == 2.5 and linear.margin(200.0) == 6.0
    assert tuned([20.0] * n) == cands[0]
    assert tuned([20.0] + [17.6] * (n - 1)) == cands[0]                                    # 2.4 us faster: not enough
    assert tuned([20.0, 17.0] + [20.0] * (n - 2)) == cands[1]                              # 3 us faster
    assert tuned([20.0, 17.0] + [20.0] * (n - 3) + [15.0]) == cands[1]                     # 2 us on the second: stays
    assert tuned([20.0, 17.0] + [20.0] * (n - 3) + [14.0]) == cands[-1]
    assert tuned([200.0, 195.0] + [200.0] * (n - 2)) == cands[0]                           # 2.5 % of a long product: noise
    assert tuned([200.0, 193.0] + [200.0] * (n - 2)) == cands[1]


def test_decode_attention_splits_follow_the_occupancy_at_long_contexts():
    """The split count of the decode kernel comes from the device: SM count times the blocks of the kernel an
    SM holds.  The page ids a block keeps in shared memory must be counted with the split count that is
    chosen, not with the whole block table: at 32,768 keys the whole table would halve the occupancy, and
    with it the splits, for nothing."""
    from delta_b200.parts import attention_kernels as ak
    o = ops()
    sms = torch.cuda.get_device_properties(DEV).multi_processor_count
    H, KV, hd, ps = 32, 4, 128, 16
    free = o.attention_decode_blocks_per_sm(H, KV, hd, 0)
    assert free >= 2
    for rows, keys in ((8, 4096), (8, 32768), (1, 32768), (64, 4096)):
        max_pages = keys // ps
        splits = ak.decode_splits(rows, KV, keys, sms, free)
        held = o.attention_decode_blocks_per_sm(H, KV, hd, -(-max_pages // splits))
        assert held == free, (rows, keys, splits, held)        # the split's share of the table costs no occupancy
        assert 1 <= splits <= ak.MAX_SPLITS and splits * rows * KV <= max(free * sms, rows * KV)
    assert o.attention_decode_blocks_per_sm(H, KV, hd, 8192) < free    # the whole table of a 131,072-key request would
