"""Makes tests/golden/reference_parts.pt: small outputs of hoenza/DELTA's own code on the CPU.

Run once with the reference on the path:

    PYTHONPATH=/path/to/hoenza-DELTA python tests/golden/make_golden.py

What of the reference runs on a CPU: RMSNorm (DELTA/Engine/DELTA/model.py:521-532),
FeedForward (495-518), the wq|wk|wv row order of Attention.load_hook (394-399),
PageManager/Request page accounting (DELTA/Engine/DELTA/scheduler.py:8-74),
PageSelectorV2 (DELTA/Engine/DELTA/page_selector_v2.py) and the page-score formula
(the three torch lines of DELTA/Engine/DELTA/backend.py:899-904, which need no
GPU; they are restated here word for word because the method they sit in reads
GPU buffers of the engine object).  Attention, rotary positions, the cache append
and the whole model's logits do not run without a GPU there (their ops are CUDA
only), so for those the plain implementation rests on the formulas.

tests/test_plain_against_reference.py compares the plain implementation with the
stored outputs.
"""
import sys
from pathlib import Path

import torch

from DELTA.Engine.DELTA.model import Attention, FeedForward, ModelArgs, RMSNorm
from DELTA.Engine.DELTA.page_selector_v2 import PageSelectorV2
from DELTA.Engine.DELTA.scheduler import PageManager, Request


def main():
    torch.manual_seed(0)
    out = {}
    args = ModelArgs(dim=64, n_head=4, n_local_heads=2, intermediate_size=176, vocab_size=512, n_layer=2, norm_eps=1e-6)

    # RMSNorm in float32 and in bfloat16 (cast before the weight multiply)
    norm = RMSNorm(64, eps=1e-6)
    norm.weight.data = 1.0 + (torch.rand(64) * 0.2 - 0.1)
    x = torch.randn(5, 64)
    out["norm_w"], out["norm_x"] = norm.weight.data.clone(), x.clone()
    out["norm_y_f32"] = norm(x).detach()
    nb = RMSNorm(64, eps=1e-6)
    nb.weight.data = norm.weight.data.to(torch.bfloat16)
    out["norm_y_bf16"] = nb(x.to(torch.bfloat16)).detach().float()

    # SwiGLU
    ff = FeedForward(args)
    for p in ff.parameters():
        p.data.normal_(0, 0.02)
    out["ff_w1"], out["ff_w2"], out["ff_w3"] = ff.w1.weight.data.clone(), ff.w2.weight.data.clone(), ff.w3.weight.data.clone()
    out["ff_x"] = x.clone()
    out["ff_y"] = ff(x, None).detach()

    # fused QKV row order
    att = Attention(args)
    sd = {"wq.weight": torch.randn(64, 64), "wk.weight": torch.randn(32, 64), "wv.weight": torch.randn(32, 64),
          "wo.weight": torch.randn(64, 64)}
    out["qkv_parts"] = {k: v.clone() for k, v in sd.items()}
    att.load_state_dict(sd)
    out["wqkv"] = att.wqkv.weight.data.clone()

    # page accounting: pages a request holds after n tokens
    pm = PageManager(64, seed=0)
    req = Request(0, torch.zeros(1, dtype=torch.long), 10 ** 6, [], pm)
    req.initialize_pages(0, 64)
    held = []
    for n in range(1, 50):
        req.plan(1, 16)
        held.append(len(req.page_indices))
    out["pages_after_tokens"] = torch.tensor(held)

    # page score (backend.py:899-904) on random scaled scores
    B, H, S, ps = 3, 4, 80, 16
    lens = [80, 37, 64]
    z = torch.randn(B, H, 1, S) * 2
    for b, n in enumerate(lens):
        z[b, :, :, n:] = float("-inf")
    probs = torch.softmax(z.to(torch.float32), dim=-1)
    scores_1d = probs.amax(dim=1).sum(dim=1)
    out["score_z"], out["score_lens"] = z[:, :, 0, :].clone(), torch.tensor(lens)
    out["score_pages"] = scores_1d.reshape(B, S // ps, ps).sum(dim=-1)

    # selection (page_selector_v2.py) for several k, L on those scores, with ties and NaN
    cases = []
    for (k, L) in [(2, 1), (3, 2), (4, 4), (4, 3)]:
        sel = PageSelectorV2(B, S // ps, True, k, 1.0, L, "cpu")
        n_pages = torch.tensor([(n + ps - 1) // ps for n in lens], dtype=torch.int32)
        indptr = torch.zeros(B + 1, dtype=torch.int32)
        indptr[1:] = torch.cumsum(n_pages, 0)
        indices = torch.arange(int(indptr[-1]), dtype=torch.int32) + 100   # physical ids = 100 + running index
        sub = torch.zeros_like(indices)
        sel.plan(torch.arange(B + 1, dtype=torch.int32), indices, indptr, torch.ones(B, dtype=torch.int32), sub,
                 torch.zeros(B + 1, dtype=torch.int32))
        sc = out["score_pages"].clone()
        sc[0, 1] = sc[0, 2]          # a tie
        sc[2, 0] = float("nan")
        idx, ptr = sel.select(sc)
        cases.append(dict(k=k, L=L, scores=sc.clone(), n_pages=n_pages.clone(), indices=idx.clone(), indptr=ptr.clone()))
    out["select_cases"] = cases
    path = Path(__file__).resolve().parent / "reference_parts.pt"
    torch.save(out, path)
    print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
