"""Preemptions on the GPU: a request that lost its pages and was computed again gives the
logits and the tokens it gives when the pool is large, with the full cache and with DELTA's
selective cache, where the positions it had generated must be decode positions again."""
import pytest
import torch

import helpers
from plain_yi import PlainYi, Selective
from test_gpu_model import bound_for

pytestmark = pytest.mark.gpu

PROMPT_LENS = [30, 22, 41, 17]
NEW = 40
SEL = dict(full_cache_layers=[1], subset_cache_size=4, L=2)


def generate(folder, dtype, selective, num_pages, prompts, graphs=False):
    """Runs the requests through the entry point and returns (outputs, {(request, position): logits row},
    {(request, layer, position): chosen pages}, the backend)."""
    from delta_b200.engine import LMBackend
    e = LMBackend(dtype=dtype, device="cuda:0", cuda_graph_decode=graphs)
    e.load_model(folder)
    e.setup_caches(max_batch_size=4, max_seq_length=128, page_size=helpers.PAGE_SIZE["B"], num_pages=num_pages,
                   max_tokens_per_step=64, enable_selective_cache=selective, **SEL)
    logits, planned = {}, {}
    e.runner.capture = {}

    def keep(plan, lg):
        rows = [x for x in plan if x.samples]
        assert lg.shape[0] == len(rows)
        for x, row in zip(rows, lg.float().cpu()):
            key = (x.request.id, x.start + x.count - 1)
            # a position that is computed again after a preemption is not sampled again
            assert key not in logits, f"position {key} was sampled twice"
            logits[key] = row
        who = {x.request.slot: x.request.id for x in plan}
        for (prefix, slot, pos), pages in e.runner.capture.pop("planned", {}).items():
            key = (who[slot], int(prefix.split(".")[2]), pos)
            if key in planned and dtype == "float32":      # chosen again when the position is computed again: the same pages
                assert planned[key] == pages, f"{key}: other pages were chosen when the position was computed again"
            planned[key] = pages
    e.on_step_logits = keep
    e.add_requests(prompts, [len(p) + NEW for p in prompts], [], max_new_tokens=NEW)
    e.run_scheduler_loop()
    e.runner.cache.check()
    assert all(v == 0 for v in e.runner.cache.pages_in_use().values())
    return [list(r.output) for r in e.scheduler.requests], logits, planned, e


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("selective", [False, True])
def test_preempted_requests_keep_their_logits(model_folders, selective, dtype):
    folder = model_folders["B"]
    ps = helpers.PAGE_SIZE["B"]
    plain = PlainYi(folder, rounding="bfloat16" if dtype == "bfloat16" else None)
    prompts = [helpers.random_tokens(n, plain.cfg.vocab, 700 + i) for i, n in enumerate(PROMPT_LENS)]
    out_big, lg_big, pl_big, e_big = generate(folder, dtype, selective, None, prompts)
    out_small, lg_small, pl_small, e_small = generate(folder, dtype, selective, 14, prompts)
    assert e_big.scheduler.stats["preemptions"] == 0
    assert e_small.scheduler.stats["preemptions"] >= 2, e_small.scheduler.stats
    assert [len(o) for o in out_small] == [NEW] * 4 and set(lg_small) == set(lg_big)
    if selective:
        assert pl_small, "the case never selected anything"

    def against_plain(outs, logits, planned, what):
        for i, (p, o) in enumerate(zip(prompts, outs)):
            seq = p + o[:-1]
            sel = Selective(SEL["full_cache_layers"], SEL["subset_cache_size"], SEL["L"], 1.0, ps, len(p)) if selective else None
            forced = None
            if selective and dtype == "bfloat16":   # nearly equal page scores may order otherwise: attend to the engine's pages
                forced = {(l, q): pg for (r, l, q), pg in planned.items() if r == i}
            ref = plain.forward(seq, sel, forced=forced)
            if selective and dtype == "float32":
                want = {(i, l, q): pg for (l, q), pg in plain.last_planned.items()}
                got = {k: v for k, v in planned.items() if k[0] == i}
                assert got == want, f"{what}: request {i} chose other pages than the plain implementation"
            for pos in range(len(p) - 1, len(seq)):
                err = (logits[(i, pos)] - ref[pos]).abs()
                assert bool((err <= bound_for(ref, dtype)).all()), f"{what}: request {i} position {pos}: max error {err.max().item():.3e}"

    against_plain(out_big, lg_big, pl_big, "large pool")
    against_plain(out_small, lg_small, pl_small, "small pool")
    if dtype == "float32":
        # the same tokens, and logits that differ by rounding only, whatever the pool did to the request
        assert out_small == out_big
        worst = max((lg_small[k] - lg_big[k]).abs().max().item() for k in lg_big)
        assert worst < 2e-6, worst
        assert pl_small == pl_big


def test_preemption_with_cuda_graph_decode(model_folders):
    """The same small pool with decode steps replayed from CUDA graphs and launched ahead of the host:
    a step that was launched ahead and then overtaken by a preemption is dropped, the tokens stay."""
    folder = model_folders["B"]
    vocab = PlainYi(folder).cfg.vocab
    prompts = [helpers.random_tokens(n, vocab, 700 + i) for i, n in enumerate(PROMPT_LENS)]
    from delta_b200.engine import LMBackend
    outs = {}
    for pages, graphs in ((None, False), (14, True)):
        e = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=graphs)
        e.load_model(folder)
        e.setup_caches(max_batch_size=4, max_seq_length=128, page_size=8, num_pages=pages, max_tokens_per_step=64,
                       enable_selective_cache=True, **SEL)
        outs[graphs] = e.generate(prompts, NEW)
        if graphs:
            assert e.scheduler.stats["preemptions"] >= 2 and e.runner.graph_replays > 20
        e.runner.cache.check()
        assert all(v == 0 for v in e.runner.cache.pages_in_use().values())
    assert outs[True] == outs[False]
