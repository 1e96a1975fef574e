"""The engine against the plain implementation, on the GPU, in 32 bit and in bfloat16:
each request alone and whole; most of it in one step and the last 32 tokens one by
one; in portions of changing size down to two tokens; and mixed, up to four live
requests with so few pages that they are used again."""
import pytest
import torch

import helpers
from plain_yi import PlainYi

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 90], "B": [1, 9, 40, 100], "C": [3, 50, 75, 120], "D": [2, 70, 131, 200]}
# Tolerances, as a fraction of the largest logit of the request's reference.  float32 against a
# float32 plain implementation differs by the rounding of sums in another order: 7e-7 of the largest
# logit is the worst seen over the four configurations.  bfloat16 against the plain implementation
# that rounds to bfloat16 at the same places differs by single roundings that flip: 4.3e-3 to 5.4e-3
# of the largest logit is the worst seen per configuration (the test prints them).  The bounds are
# about twice that.
TOL = {"float32": 2e-6, "bfloat16": 1e-2}


def bound_for(ref: torch.Tensor, dtype: str) -> float:
    """The largest difference allowed to any logit of a request whose reference logits are ``ref``."""
    return TOL[dtype] * ref.abs().max().item()


def make_runner(folder, which, dtype, num_pages, **kw):
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    cfg = EngineConfig(max_batch=4, max_seq_len=256, page_size=helpers.PAGE_SIZE[which], num_pages=num_pages, dtype=dtype, **kw)
    return ModelRunner(folder, engine_config=cfg)


def reference_logits(folder, which, dtype, token_lists):
    plain = PlainYi(folder, rounding="bfloat16" if dtype == "bfloat16" else None)
    return [plain.forward(t) for t in token_lists]


def compare(results, refs, lengths, dtype, what):
    worst = 0.0
    for i, n in enumerate(lengths):
        got = helpers.stack_positions(results, i, n)
        err = (got - refs[i]).abs()
        bad = (err > bound_for(refs[i], dtype)).nonzero()
        if bad.numel():
            p = int(bad[0, 0])
            raise AssertionError(f"{what}: request {i} first differs at position {p} (of {n}): "
                                 f"max error {err[p].max().item():.3e}, logit scale {refs[i][p].abs().max().item():.3f}")
        worst = max(worst, err.max().item())
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
def test_every_way_of_cutting(model_folders, which, dtype):
    folder = model_folders[which]
    lengths = LENGTHS[which]
    cfgv = PlainYi(folder).cfg.vocab
    toks = [helpers.random_tokens(n, cfgv, 100 + i) for i, n in enumerate(lengths)]
    refs = reference_logits(folder, which, dtype, toks)
    ps = helpers.PAGE_SIZE[which]

    runner = make_runner(folder, which, dtype, num_pages=4 * (256 // ps))
    worst = {}
    res = helpers.run_schedule(runner, toks, helpers.whole(lengths))
    worst["whole"] = compare(res, refs, lengths, dtype, "whole")
    res = helpers.run_schedule(runner, toks, helpers.last_one_by_one(lengths))
    worst["one by one"] = compare(res, refs, lengths, dtype, "last 32 one by one")
    res = helpers.run_schedule(runner, toks, helpers.changing_portions(lengths, seed=1))
    worst["portions"] = compare(res, refs, lengths, dtype, "changing portions")

    # mixed, with a pool so small that pages of finished requests are used again
    prompt_lens = [max(1, n // 2) for n in lengths]
    steps, ends = helpers.mixed(lengths * 2, prompt_lens * 2, seed=3)
    tight = make_runner(folder, which, dtype, num_pages=helpers.peak_pages(steps, ends, ps))
    res = helpers.run_schedule(tight, toks * 2, steps, ends)
    worst["mixed"] = compare(res, refs * 2, lengths * 2, dtype, "mixed with page reuse")
    scale = max(r.abs().max().item() for r in refs)
    print(f"\nworst logit error {which} {dtype} (largest logit {scale:.2f}): " + ", ".join(f"{k} {v:.2e}" for k, v in worst.items()))
