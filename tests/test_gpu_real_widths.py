"""Two layers with the widths of Yi-6B (hidden 4096, 32 heads, 4 key-value heads, head size 128,
feed-forward 11008) in bfloat16: the tensor-core kernels as the engine launches them at real sizes
(tcgen05 prefill attention over 32 heads, the library and the small-batch products at these widths,
the split-key decode attention with runs of pages fetched by TMA) against the same engine on its plain
kernels.  The tiny configurations of the other tests never reach these grids."""
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

CFG = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096, num_hidden_layers=2,
           num_attention_heads=32, num_key_value_heads=4, intermediate_size=11008, vocab_size=4000,
           rope_theta=5000000.0, rms_norm_eps=1e-5, max_position_embeddings=2048, hidden_act="silu",
           tie_word_embeddings=False, torch_dtype="bfloat16")


def compare(results, refs, lengths, what):
    """Both sides round to bfloat16 on the way, at different places (the library product rounds its
    output, the plain one a float sum; the order of the sums over 4096 and 11008 differs), so the bound
    is set by the size of a position's logits: 2 % of their largest magnitude."""
    for i, n in enumerate(lengths):
        got = helpers.stack_positions(results, i, n)
        err = (got - refs[i]).abs().amax(dim=-1)
        bound = 2e-2 * refs[i].abs().amax(dim=-1)
        bad = (err > bound).nonzero()
        if bad.numel():
            p = int(bad[0, 0])
            raise AssertionError(f"{what}: request {i} first differs at position {p} (of {n}): "
                                 f"max error {err[p].item():.3e}, logit scale {refs[i][p].abs().max().item():.3f}")


def test_real_widths_fast_kernels_against_plain_kernels(monkeypatch):
    from delta_b200.config import EngineConfig
    from delta_b200.parts import attention_kernels
    from delta_b200.engine.step import ModelRunner
    monkeypatch.setattr(attention_kernels, "TMA_MIN_TILES", 1)    # short blocks too take the TMA variant here
    lengths = [700, 300, 1100]
    toks = [helpers.random_tokens(n, CFG["vocab_size"], 500 + i) for i, n in enumerate(lengths)]

    def runner(plain):
        r = ModelRunner(None, engine_config=EngineConfig(max_batch=4, max_seq_len=1152, page_size=16, dtype="bfloat16"),
                        config_json=CFG, seed=3)
        r.plain_kernels = {"products", "attention"} if plain else set()
        return r

    slow = runner(True)
    res = helpers.run_schedule(slow, toks, helpers.whole(lengths))
    refs = [helpers.stack_positions(res, i, n) for i, n in enumerate(lengths)]
    del slow
    torch.cuda.empty_cache()
    fast = runner(False)
    res = helpers.run_schedule(fast, toks, helpers.last_one_by_one(lengths, tail=12))
    compare(res, refs, lengths, "real widths: last 12 one by one")
    steps, ends = helpers.mixed(lengths, [n // 2 for n in lengths], seed=5)
    res = helpers.run_schedule(fast, toks, steps, ends)
    compare(res, refs, lengths, "real widths: mixed")


def test_real_widths_against_the_plain_implementation(tmp_path):
    """The same widths against the plain implementation on the CPU (short requests, so that it stays a matter of
    seconds).  At a width of 4,096 and sums over 11,008 the rounding to bfloat16 itself moves the logits by 1.6 % of
    the largest one (plain implementation in bfloat16 against itself in 32 bit), more than the 1 % that bounds the
    tiny models; the bound here is that measured size of the rounding: the engine may differ from the plain
    implementation in bfloat16 by no more than bfloat16 differs from 32 bit (1.2 % is what it does differ by).
    A fault of the cache or of a kernel at these grids moves logits by many times that."""
    from plain_yi import PlainYi
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    from delta_b200.weights import write_random_model
    import delta_b200.models  # noqa: F401
    folder = write_random_model(tmp_path / "real_widths", CFG, 3, torch.bfloat16)
    lengths = [150, 40]
    toks = [helpers.random_tokens(n, CFG["vocab_size"], 500 + i) for i, n in enumerate(lengths)]
    refs = [PlainYi(folder, rounding="bfloat16").forward(t) for t in toks]
    exact = [PlainYi(folder).forward(t) for t in toks]
    bounds = [(a - b).abs().max().item() for a, b in zip(refs, exact)]
    assert all(0.005 * b.abs().max().item() < bound < 0.03 * b.abs().max().item() for bound, b in zip(bounds, exact)), bounds
    r = ModelRunner(folder, engine_config=EngineConfig(max_batch=4, max_seq_len=256, page_size=16, dtype="bfloat16"))
    for what, sched in (("whole", helpers.whole(lengths)), ("last 12 one by one", helpers.last_one_by_one(lengths, tail=12)),
                        ("changing portions", helpers.changing_portions(lengths, seed=1))):
        res = helpers.run_schedule(r, toks, sched)
        for i, n in enumerate(lengths):
            err = (helpers.stack_positions(res, i, n) - refs[i]).abs().amax(dim=-1)
            assert err.max().item() <= bounds[i], (f"real widths, {what}: request {i} position {int(err.argmax())} differs by "
                                                   f"{err.max().item():.4f}, the rounding's own size is {bounds[i]:.4f}")
