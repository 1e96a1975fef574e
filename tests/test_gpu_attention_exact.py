"""Tests that a kernel cannot pass by being roughly right.

Every page counts: with queries of zero every key a row may read weighs the same, and with the unit
vector of its page's number as each key's value the output is, exactly, the share of every page among
the keys read.  A kernel that drops or doubles one 16-token page among 4,000 keys moves a component
by 1/250 of itself; the bound is 2^-8 of each component (the output's own rounding to bfloat16 is
2^-9), and the log-sum-exp must be log(keys read).  Long contexts, every split count, windows and
chosen pages, for the decode kernel in its three variants, both tiled prefill kernels and the plain
kernel.

A negative control: one entry of a request's block table is overwritten with another of its pages on
the host, so that one page is read twice and one never; the engine's logits must then fail the
comparison that the other tests pass.  (Swapping two full pages would change nothing: keys carry
their positions in their rotation, and attention does not care in which order it meets them.)

A wait that runs out: a kernel whose only wait is bounded by a millisecond and can never be satisfied
returns with the error record set, the host raises with the "wait ran out" text, the next launch works.
"""
import math

import pytest
import torch

import helpers
from plain_yi import PlainYi
from test_gpu_kernels import DEV, PagedCase, i32, ops
from test_gpu_model import bound_for, compare

pytestmark = pytest.mark.gpu


def assert_counts(got, ref, what):
    g, r = got.float().cpu(), ref.float()
    bad = ((g - r).abs() > r.abs() / 256 + 1e-9).nonzero()
    if bad.numel():
        t, c = int(bad[0, 0]), int(bad[0, 1])
        raise AssertionError(f"{what}: token {t}, component {c}: got {g[t, c].item():.6f}, the share of that page is {r[t, c].item():.6f}")


def chosen_pages(n_tokens, ps, k, seed):
    """k logical pages of a request, ascending, the last one included (as page selection gives them)."""
    import random
    n = (n_tokens + ps - 1) // ps
    rng = random.Random(seed)
    return sorted(rng.sample(range(n - 1), min(k - 1, n - 1)) + [n - 1])


@pytest.mark.parametrize("pages", ["scattered", "runs", "scattered, told so"])
@pytest.mark.parametrize("G, KV, hd, ps", [(8, 4, 128, 16), (4, 2, 64, 16), (16, 1, 128, 32), (3, 2, 64, 8)])
def test_every_page_counts_in_the_decode_kernel(G, KV, hd, ps, pages):
    o = ops()
    H = G * KV
    seq_lens = [1000, 2500, 4000, 3071, 1, 1025]
    B = len(seq_lens)
    case = PagedCase(torch.bfloat16, H, KV, hd, ps, seq_lens, [1] * B, seed=3, scatter=pages != "runs", counting=True)
    told = pages == "scattered, told so"
    ref, ref_lse, _ = case.reference()
    for splits in (1, 2, 7, 16, 64):
        out = torch.full((B, H * hd), 9.0, dtype=torch.bfloat16, device=DEV)
        lse = torch.empty(B, H, device=DEV)
        scratch = torch.empty(max(1, o.attention_decode_scratch_floats(B, H, hd, splits)), device=DEV)
        p = case.params(out, lse=lse, scratch=scratch, splits=splits)
        p.reserved = 1 if told else 0
        o.attention_decode(p)
        assert_counts(out, ref, f"splits={splits}")
        assert torch.allclose(lse.cpu(), ref_lse, atol=1e-3, rtol=0), f"splits={splits}: log-sum-exp"
    # a window that begins inside a page, far back
    for window in (1500 + 5, ps + 1):
        out = torch.full((B, H * hd), 9.0, dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(o.attention_decode_scratch_floats(B, H, hd, 5), device=DEV)
        p = case.params(out, window=window, scratch=scratch, splits=5)
        p.reserved = 1 if told else 0
        o.attention_decode(p)
        refw, _, _ = case.reference(window=window)
        assert_counts(out, refw, f"window={window}")
    # chosen pages: rows 0..3 read 40 pages each, the others everything
    k = 40
    flags = i32([1, 1, 1, 1, 0, 1])
    sel_pages = torch.zeros(B, k, dtype=torch.int32, device=DEV)
    sel_count = torch.full((B,), -1, dtype=torch.int32, device=DEV)
    chosen = [chosen_pages(n, ps, k, 10 + b) if b < 4 else None for b, n in enumerate(seq_lens)]
    for b in range(4):
        sel_pages[b, :len(chosen[b])] = i32(chosen[b])
        sel_count[b] = len(chosen[b])
    refc, refc_lse, _ = case.reference(pages=chosen)
    for splits in (1, 3, 16):
        out = torch.full((B, H * hd), 9.0, dtype=torch.bfloat16, device=DEV)
        lse = torch.empty(B, H, device=DEV)
        scratch = torch.empty(max(1, o.attention_decode_scratch_floats(B, H, hd, splits)), device=DEV)
        p = case.params(out, lse=lse, row_flags=flags, sel_pages=sel_pages, sel_count=sel_count, scratch=scratch, splits=splits)
        p.reserved = 1 if told else 0
        o.attention_decode(p)
        assert_counts(out, refc, f"chosen pages, splits={splits}")
        assert torch.allclose(lse.cpu(), refc_lse, atol=1e-3, rtol=0)


@pytest.mark.parametrize("kernel", ["plain float32", "plain bfloat16", "mma_sync", "tcgen05", "tcgen05_runs"])
def test_every_page_counts_in_the_prefill_and_plain_kernels(kernel):
    o = ops()
    H, KV, hd, ps = 8, 2, 128, 16
    dtype = torch.float32 if kernel == "plain float32" else torch.bfloat16
    seq_lens = [1000, 4000, 2049, 3000, 130]
    q_lens = [37, 200, 2049, 1, 130]
    case = PagedCase(dtype, H, KV, hd, ps, seq_lens, q_lens, seed=4, scatter=kernel != "tcgen05_runs", counting=True)
    run = {"plain float32": lambda p: o.attention_plain(p), "plain bfloat16": lambda p: o.attention_plain(p),
           "mma_sync": lambda p: o.attention_prefill(p, max(q_lens)), "tcgen05": lambda p: o.attention_prefill_tc(p, max(q_lens)),
           "tcgen05_runs": lambda p: o.attention_prefill_tc(p, max(q_lens))}[kernel]
    err = o.new_error_record(DEV)
    for window in (0, 1500 + 5, ps + 1):
        out = torch.full((case.T, H * hd), 9.0, dtype=dtype, device=DEV)
        lse = torch.empty(case.T, H, device=DEV)
        run(case.params(out, lse=lse, window=window, err=err))
        o.raise_if_error(err)
        ref, ref_lse, _ = case.reference(window=window)
        assert_counts(out, ref, f"{kernel}, window={window}")
        assert torch.allclose(lse.cpu(), ref_lse, atol=1e-3, rtol=0), f"{kernel}, window={window}: log-sum-exp"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wrong_block_table_entry_is_noticed(model_folders, dtype):
    """Negative control: the comparison that every engine test relies on must fail when a request
    reads one of its ten pages twice and another one never."""
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner, RowInput
    which = "D"
    folder, ps = model_folders[which], helpers.PAGE_SIZE[which]
    plain = PlainYi(folder, rounding="bfloat16" if dtype == "bfloat16" else None)
    n = 150
    toks = helpers.random_tokens(n, plain.cfg.vocab, 77)
    ref = plain.forward(toks)
    for wrong in (False, True):
        r = ModelRunner(folder, engine_config=EngineConfig(max_batch=2, max_seq_len=256, page_size=ps, dtype=dtype))
        slot = r.cache.acquire_slot()
        r.run_rows([RowInput(slot, toks[:100], 0, [])])
        if wrong:
            for g in r.cache.groups.values():
                g.table[slot, 1] = g.table[slot, 4]
        res = {}
        for p in range(100, n):
            res[(0, p)] = r.run_rows([RowInput(slot, toks[p:p + 1], p, [0])])[0].float().cpu()
        got = {(0, p - 100): row for (_, p), row in res.items()}
        if wrong:
            with pytest.raises(AssertionError, match="first differs"):
                compare(got, [ref[100:]], [n - 100], dtype, "a page read twice")
        else:
            compare(got, [ref[100:]], [n - 100], dtype, "pages in order")


def test_a_wait_that_runs_out_is_reported_and_the_next_launch_works():
    o = ops()
    err = o.new_error_record(DEV)
    o.wait_check(err, limit_ms=1.0)
    with pytest.raises(o.KernelError, match="a wait inside a kernel ran out"):
        o.raise_if_error(err)
    assert err.tolist() == [0, 0, 0, 0]          # reading the record clears it
    with pytest.raises(o.KernelError, match="limit"):
        o.wait_check(err, limit_ms=50.0)          # a longer limit than ten milliseconds is refused
    # the context is as it was: a product on the tensor cores, then a clean record
    x = torch.randn(8, 256, device=DEV).to(torch.bfloat16)
    w = torch.randn(128, 256, device=DEV).to(torch.bfloat16)
    out = torch.empty(8, 128, dtype=torch.bfloat16, device=DEV)
    assert o.gemm_tc_supported(8, 128, 256)
    o.gemm_tc(x, w, out, err=err)
    o.raise_if_error(err)
    assert torch.allclose(out.float(), x.float() @ w.float().T, atol=0.5, rtol=2e-2)
