"""The plain implementation against outputs of hoenza/DELTA's own code: the parts of it that run
on a CPU (stored by tests/golden/make_golden.py), and the logits of its whole model on a GPU, run
through its own entry point on a tiny random model (stored by
tests/golden/make_reference_model_golden.py)."""
import sys
from pathlib import Path

import pytest
import torch

import plain_yi as P

GOLDEN = Path(__file__).resolve().parent / "golden"
G = torch.load(GOLDEN / "reference_parts.pt")


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


# ---- the whole model: rotary positions, cache append, attention, layer order, output matrix --------

@pytest.fixture(scope="module")
def reference_model(tmp_path_factory):
    """(stored logits of the reference, the tiny model folder they were made from, written again here
    from its configuration and seed and checked against the stored checksum of the weights)."""
    sys.path.insert(0, str(GOLDEN))
    from make_reference_model_golden import checksum
    from delta_b200.weights import write_random_model
    import delta_b200.models  # noqa: F401
    M = torch.load(GOLDEN / "reference_model_logits.pt")
    folder = write_random_model(tmp_path_factory.mktemp("golden") / "hf", M["config"], M["seed"], torch.float32)
    if checksum(P.read_safetensors_plain(folder / "model.safetensors")) != M["weights_sha256"]:
        pytest.skip("this torch draws other random weights from the seed than the one the stored logits were made with")
    return M, folder


def test_whole_model_logits_equal_the_reference(reference_model):
    """The reference ran a converted checkpoint (q and k rows in neighbour pairs) with its
    neighbour-pair rotation in bfloat16; the plain implementation reads the unconverted folder and
    rotates pairs (j, j + head/2).  Every position's logits agree to the rounding of bfloat16
    (0.9 % of the largest logit is the worst seen; the bound is 1.5 %), prompts of 40, 23 and 1
    tokens and 24 decoded tokens each, and the greedy tokens follow."""
    M, folder = reference_model
    plain = P.PlainYi(folder, rounding="bfloat16")
    for i, (prompt, out) in enumerate(zip(M["prompts"], M["outputs"])):
        ref = M["logits"][i].float()
        got = plain.forward(prompt + out[:-1])
        assert got.shape == ref.shape
        scale = ref.abs().max().item()
        err = (got - ref).abs().amax(dim=-1)
        assert err.max().item() <= 0.015 * scale, f"request {i}: position {int(err.argmax())} differs by {err.max().item():.4f} (largest logit {scale:.3f})"
        # greedy tokens, wherever the reference's best two logits are further apart than the rounding
        top = ref.topk(2, dim=-1).values
        clear = (top[:, 0] - top[:, 1]) > 0.03 * scale
        assert bool((got.argmax(-1) == ref.argmax(-1))[clear].all()) and int(clear.sum()) > len(prompt) // 2


def test_the_other_pairing_or_head_mapping_would_not_pass(reference_model):
    """What the comparison above is able to see: neighbour-pair rotation on the unconverted rows, or
    query heads mapped to key-value heads the other way round, miss the reference by several bounds."""
    M, folder = reference_model
    prompt, out = M["prompts"][0], M["outputs"][0]
    ref = M["logits"][0].float()
    scale = ref.abs().max().item()
    wrong = P.PlainYi(folder, rounding="bfloat16", interleaved=True).forward(prompt + out[:-1])
    assert (wrong - ref).abs().max().item() > 0.04 * scale
    swapped = P.PlainYi(folder, rounding="bfloat16")
    c = swapped.cfg
    for l in range(c.layers):       # exchange the two key-value heads: query heads 0,1 then read what belongs to 2,3
        for name in ("k_proj", "v_proj"):
            w = swapped.w[f"model.layers.{l}.self_attn.{name}.weight"]
            swapped.w[f"model.layers.{l}.self_attn.{name}.weight"] = w.view(c.kv_heads, c.head_dim, -1).flip(0).reshape(w.shape)
    assert (swapped.forward(prompt + out[:-1]) - ref).abs().max().item() > 0.04 * scale


# ---- DELTA on: the newest pages, the page scores, the choice, and the reading of chosen pages ------

@pytest.fixture(scope="module")
def reference_selective(tmp_path_factory):
    sys.path.insert(0, str(GOLDEN))
    from make_reference_model_golden import checksum
    from delta_b200.weights import write_random_model
    import delta_b200.models  # noqa: F401
    M = torch.load(GOLDEN / "reference_selective_logits.pt")
    folder = write_random_model(tmp_path_factory.mktemp("golden_sel") / "hf", M["config"], M["seed"], torch.float32)
    if checksum(P.read_safetensors_plain(folder / "model.safetensors")) != M["weights_sha256"]:
        pytest.skip("this torch draws other random weights from the seed than the one the stored logits were made with")
    return M, folder


def selective_of(M, **more):
    s = M["selective"]
    return P.Selective(full_layers=tuple(s["full_cache_layers"]), k=s["subset_cache_size"], L=s["L"], ratio=s["compression_ratio"],
                       page_size=M["page_size"], prompt_len=len(M["prompt"]), **more)


def test_selective_logits_equal_the_reference(reference_selective):
    """The reference ran one request of 20 prompt tokens and 100 decoded ones with DELTA on: three layers,
    layer 0 reads the newest 4 pages, layer 1 scores and chooses 4 pages (the newest 2 always), layer 2 reads
    them.  With the reference's count of pages the plain implementation agrees at all 119 positions to the
    rounding of bfloat16 (1.0 % of the largest logit is the worst seen; the bound is 1.5 %)."""
    M, folder = reference_selective
    ref = M["logits"].float()
    seq = M["prompt"] + M["output"][:-1]
    plain = P.PlainYi(folder, rounding="bfloat16")
    got = plain.forward(seq, selective_of(M, trailing_empty_page=True))
    scale = ref.abs().max().item()
    err = (got - ref).abs().amax(dim=-1)
    assert err.max().item() <= 0.015 * scale, f"position {int(err.argmax())} differs by {err.max().item():.4f} (largest logit {scale:.3f})"
    assert len(plain.last_planned) >= 50          # the choice was made at more than half of the decoded positions


def test_what_the_selective_comparison_sees(reference_selective):
    """Reading everything instead of the chosen pages misses the stored logits by a quarter of the largest one;
    counting only the pages that hold tokens differs where a page has just filled, and only from there on."""
    M, folder = reference_selective
    ref = M["logits"].float()
    seq = M["prompt"] + M["output"][:-1]
    scale = ref.abs().max().item()
    plain = P.PlainYi(folder, rounding="bfloat16")
    everything = (plain.forward(seq) - ref).abs().amax(dim=-1) / scale
    assert everything.max().item() > 0.25
    own = (plain.forward(seq, selective_of(M)) - ref).abs().amax(dim=-1) / scale
    first = int((own > 0.015).nonzero()[0])
    assert own.max().item() > 0.05 and (first + 1) % M["page_size"] == 0
