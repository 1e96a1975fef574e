"""The plain implementation against outputs of hoenza/DELTA's own code (stored by
tests/golden/make_golden.py), for the parts of it that run on a CPU."""
from pathlib import Path

import torch

import plain_yi as P

G = torch.load(Path(__file__).resolve().parent / "golden" / "reference_parts.pt")


def test_rms_norm_float32():
    y = P.rms_norm(G["norm_x"], G["norm_w"], 1e-6)
    assert torch.allclose(y, G["norm_y_f32"], atol=1e-6, rtol=1e-6)


def test_rms_norm_bfloat16_casts_before_the_weight():
    x = P.bf16_round(G["norm_x"])
    w = P.bf16_round(G["norm_w"])
    y = P.bf16_round(P.rms_norm(x, w, 1e-6, P.bf16_round))
    assert torch.equal(y, G["norm_y_bf16"])


def test_swiglu():
    y = P.swiglu(G["ff_x"], G["ff_w1"], G["ff_w3"], G["ff_w2"])
    assert torch.allclose(y, G["ff_y"], atol=1e-6, rtol=1e-5)


def test_fused_qkv_row_order():
    p = G["qkv_parts"]
    assert torch.equal(torch.cat([p["wq.weight"], p["wk.weight"], p["wv.weight"]]), G["wqkv"])


def test_pages_held():
    # the reference holds one page more than ceil(n / 16) once a page is exactly full
    # (scheduler.py:60-74); the engine holds ceil(n / 16)
    for n, held in enumerate(G["pages_after_tokens"].tolist(), start=1):
        assert held == n // 16 + 1
        assert (n + 15) // 16 <= held


def test_page_scores():
    z, lens = G["score_z"], G["score_lens"].tolist()
    for b, n in enumerate(lens):
        s = P.page_scores(z[b, :, :n], n, 16)
        assert torch.allclose(s, G["score_pages"][b, :s.shape[0]], atol=1e-6, rtol=1e-5)


def test_page_selection():
    for case in G["select_cases"]:
        k, L = case["k"], case["L"]
        ptr = case["indptr"].tolist()
        base = 0
        for b, n in enumerate(case["n_pages"].tolist()):
            mine = P.select_pages(case["scores"][b], n, k, L)
            ref = (case["indices"][ptr[b]:ptr[b + 1]] - 100 - base).tolist()
            assert mine == ref, (k, L, b, mine, ref)
            base += n
