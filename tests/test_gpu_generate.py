"""Generation through the Python entry point and the command line; long decoding; the
first tokens of a sequence; temperature sampling."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import helpers
from plain_yi import PlainYi, greedy, temperature_probs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def plain_greedy(plain, prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        t = greedy(plain.forward(seq)[-1])
        out.append(t)
        seq.append(t)
    return out


def backend(folder, dtype, **kw):
    from delta_b200.engine import LMBackend
    e = LMBackend(dtype=dtype, device="cuda:0")
    e.load_model(folder)
    e.setup_caches(check_kernel_errors=True, **kw)
    return e


def test_greedy_generation_matches_plain(model_folders):
    folder = model_folders["A"]
    plain = PlainYi(folder)
    prompts = [helpers.random_tokens(n, plain.cfg.vocab, 5 + i) for i, n in enumerate([5, 17, 33])]
    e = backend(folder, "float32", max_batch_size=4, max_seq_length=64, page_size=16)
    outs = e.generate(prompts, 8)
    for p, o in zip(prompts, outs):
        assert o == plain_greedy(plain, p, 8)
    res = e.get_detailed_results()
    assert [r["output_length"] for r in res] == [8, 8, 8] and all(r["status"] == "finished" for r in res)


def test_generation_with_few_pages_and_a_small_budget(model_folders):
    """More requests than slots, prompts cut into portions of at most 11 tokens, a pool that
    forces waiting; the tokens still equal the plain implementation's."""
    folder = model_folders["C"]
    plain = PlainYi(folder)
    prompts = [helpers.random_tokens(n, plain.cfg.vocab, 50 + i) for i, n in enumerate([3, 50, 75, 20, 41, 9])]
    e = backend(folder, "float32", max_batch_size=3, max_seq_length=96, page_size=32, num_pages=7, max_tokens_per_step=11)
    outs = e.generate(prompts, 6)
    for p, o in zip(prompts, outs):
        assert o == plain_greedy(plain, p, 6)
    assert e.scheduler.stats["prefill_steps"] > 6
    e.runner.cache.check()
    assert all(v == 0 for v in e.runner.cache.pages_in_use().values())


def test_long_decoding(model_folders):
    """200 tokens decoded one by one from a short prompt, against the plain implementation
    run on the whole sequence (float32 logits, and greedy tokens)."""
    from delta_b200.engine.step import RowInput
    folder = model_folders["B"]
    plain = PlainYi(folder)
    e = backend(folder, "float32", max_batch_size=1, max_seq_length=256, page_size=8)
    prompt = helpers.random_tokens(4, plain.cfg.vocab, 9)
    out = e.generate([prompt], 200)[0]
    seq = prompt + out
    ref = plain.forward(seq[:-1])
    for i, t in enumerate(out):
        assert t == greedy(ref[len(prompt) - 1 + i]), f"token {i}"


def test_first_tokens(model_folders):
    """Positions 0, 1, 2 of a sequence, fed one by one and as one portion."""
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    for which in "AB":
        folder = model_folders[which]
        plain = PlainYi(folder)
        toks = [helpers.random_tokens(3, plain.cfg.vocab, 3), helpers.random_tokens(1, plain.cfg.vocab, 4)]
        refs = [plain.forward(t) for t in toks]
        r = ModelRunner(folder, engine_config=EngineConfig(max_batch=2, max_seq_len=32, page_size=helpers.PAGE_SIZE[which], dtype="float32"))
        for steps in ([[(0, 0, 3)], [(1, 0, 1)]], [[(0, 0, 1), (1, 0, 1)], [(0, 1, 1)], [(0, 2, 1)]]):
            res = helpers.run_schedule(r, toks, steps)
            for i, t in enumerate(toks):
                assert torch.allclose(helpers.stack_positions(res, i, len(t)), refs[i], atol=2e-5, rtol=1e-4)


def test_temperature_sampling_follows_the_distribution(model_folders):
    """Each sampled token is the one whose interval of the cumulative distribution
    (vocabulary order) holds the request's uniform number for that position."""
    from delta_b200.sampling import uniform_of
    folder = model_folders["B"]
    plain = PlainYi(folder)
    prompts = [helpers.random_tokens(n, plain.cfg.vocab, 20 + i) for i, n in enumerate([1, 9, 40])]
    e = backend(folder, "float32", max_batch_size=4, max_seq_length=128, page_size=8)
    outs = e.generate(prompts, 12, temperature=0.7, seed=1234)
    again = backend(folder, "float32", max_batch_size=2, max_seq_length=128, page_size=8, max_tokens_per_step=7)
    assert again.generate(prompts, 12, temperature=0.7, seed=1234) == outs   # same seed, other batching: same tokens
    for i, (p, o) in enumerate(zip(prompts, outs)):
        seq = list(p)
        for t in o:
            probs = temperature_probs(plain.forward(seq)[-1], 0.7)
            cdf = torch.cumsum(probs, 0)
            u = uniform_of(1234 + i, len(seq))
            lo = cdf[t - 1].item() if t > 0 else 0.0
            assert lo - 1e-5 <= u <= cdf[t].item() + 1e-5, (i, len(seq), t, u, lo, cdf[t].item())
            seq.append(t)


def test_command_line(model_folders, tmp_path):
    out = tmp_path / "result.json"
    cmd = [sys.executable, "-m", "delta_b200.cli", "--model", str(model_folders["A"]), "--B", "4", "--max_len", "128",
           "--dataset", "random", "--prompt_len", "20", "--num_samples", "5", "--max_new_tokens", "6", "--dtype", "float32",
           "--enable_selective_cache", "--full_cache_layers", "0", "--subset_cache_size", "2", "--L", "1", "--out", str(out)]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    res = json.loads(out.read_text())
    assert res["summary"]["generated_tokens"] == 30 and len(res["results"]) == 5


def test_command_line_step_timings_and_tuning_file(model_folders, tmp_path):
    """--step_timings writes logs/step_timings_<time>.json with the reference's five timing names and a meta
    block; --tuning_file saves the measured kernel choices and a second run reads them back."""
    import os
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    tune = tmp_path / "tune.json"
    cmd = [sys.executable, "-m", "delta_b200.cli", "--model", str(model_folders["D"]), "--B", "3", "--max_len", "128",
           "--dataset", "random", "--prompt_len", "24", "--num_samples", "3", "--max_new_tokens", "10", "--cuda_graph_decode",
           "--step_timings", "--tuning_file", str(tune)]
    for run in range(2):
        r = subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        summary = json.loads(r.stdout.strip().splitlines()[-1])
        assert summary["generated_tokens"] == 30 and summary["graph_replays"] > 0 and summary["graph_fallbacks"] == {}
        rec = json.loads((tmp_path / summary["step_timings_file"]).read_text())
        assert {"collect_pages_ms", "plan_ms", "model_forward_ms", "postprocess_ms", "step_total_ms", "active_bsz", "total_pages"} <= set(rec["steps"][0])
        assert rec["meta"]["steps"] == len(rec["steps"]) and "summary" in rec["meta"]
        assert all(s["collect_pages_ms"] >= 0 and s["model_forward_ms"] > 0 for s in rec["steps"])
        choices = json.loads(tune.read_text())["product_kernels"]
        assert choices and all(c["kernel"] for c in choices)
        if run == 0:
            first = {(c["rows"], c["n"], c["k"], c["swiglu"]): c["kernel"] for c in choices}
        else:       # the second run took the saved choices: none differs
            assert first == {(c["rows"], c["n"], c["k"], c["swiglu"]): c["kernel"] for c in choices if (c["rows"], c["n"], c["k"], c["swiglu"]) in first}


@pytest.mark.parametrize("selective", [False, True])
def test_cuda_graph_decode_gives_the_same_tokens(model_folders, selective):
    """Decode steps replayed from a CUDA graph generate what eager steps generate, with
    batches that shrink as requests finish (one graph per batch size) and with DELTA on."""
    from delta_b200.engine import LMBackend
    folder = model_folders["B"]
    plain = PlainYi(folder)
    prompts = [helpers.random_tokens(n, plain.cfg.vocab, 80 + i) for i, n in enumerate([30, 9, 50, 17])]
    outs = {}
    for graphs in (False, True):
        e = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=graphs)
        e.load_model(folder)
        e.setup_caches(max_batch_size=4, max_seq_length=128, page_size=8, check_kernel_errors=True,
                       enable_selective_cache=selective, full_cache_layers=[1], subset_cache_size=4, L=2)
        first = len(e.scheduler.requests)
        e.add_requests(prompts, [60, 40, 90, 128], [])
        e.run_scheduler_loop()
        outs[graphs] = [r.output for r in e.scheduler.requests[first:]]
        if graphs:
            assert e.runner.graph_captures >= 2 and e.runner.graph_replays > 20
    assert outs[True] == outs[False]
    if not selective:
        assert outs[True][1] == plain_greedy(plain, prompts[1], 31)


@pytest.mark.parametrize("selective", [False, True])
def test_decode_steps_launched_ahead_give_the_same_tokens(model_folders, selective):
    """With CUDA-graph decode the engine launches step N + 1 before the host has read the tokens
    of step N (they are taken on the device).  Requests that stop at a stop token, at their
    length and at different steps, a request added while others decode, temperature sampling and
    DELTA: the tokens are those of the engine that feeds every token back through the host."""
    from delta_b200.engine import LMBackend
    folder = model_folders["B"]
    plain = PlainYi(folder)
    prompts = [helpers.random_tokens(n, plain.cfg.vocab, 90 + i) for i, n in enumerate([30, 9, 50, 17])]
    late = helpers.random_tokens(21, plain.cfg.vocab, 99)
    # a stop token that the second request really meets: taken from a run without stop tokens
    probe = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=False)
    probe.load_model(folder)
    probe.setup_caches(max_batch_size=1, max_seq_length=128, page_size=8)
    stop = probe.generate([prompts[1]], 20)[0][12]
    outs, launched = {}, {}
    for ahead in (False, True):
        e = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=True)
        e.run_ahead = ahead
        e.load_model(folder)
        e.setup_caches(max_batch_size=5, max_seq_length=128, page_size=8, check_kernel_errors=True,
                       enable_selective_cache=selective, full_cache_layers=[1], subset_cache_size=4, L=2)
        reused = 0
        first = len(e.scheduler.requests)
        e.add_requests(prompts[:1], [60], [], temperature=0.8, seed=5)
        e.add_requests(prompts[1:2], [70], [stop])
        e.add_requests(prompts[2:], [90, 128], [])
        steps = 0
        while e.scheduler.has_work():
            had = e._ahead is not None
            e.step()
            reused += int(had)
            steps += 1
            if steps == 25:
                e.add_requests([late], [64], [], temperature=0.5, seed=3)
        outs[ahead] = [r.output for r in e.scheduler.requests[first:]]
        launched[ahead] = reused
    assert outs[True] == outs[False]
    assert outs[True][1][-1] == stop and len(outs[True][1]) <= 13
    assert launched[False] == 0 and launched[True] > 40


@pytest.mark.parametrize("selective", [False, True])
def test_rounded_up_decode_batches_give_the_same_tokens(model_folders, selective):
    """Above 8 rows a captured decode step has a rounded-up batch size (12, 16, ...); its spare
    rows decode position 0 of the cache's padding slot.  Thirteen requests that end one after the
    other, so that the batch passes 13, 12, 11, ... rows: the tokens are those of the engine
    without CUDA graphs, and no page is lost."""
    from delta_b200.engine import LMBackend
    folder = model_folders["B"]
    plain = PlainYi(folder)
    prompts = [helpers.random_tokens(5 + 3 * i, plain.cfg.vocab, 300 + i) for i in range(13)]
    lengths = [len(p) + 6 + 2 * i for i, p in enumerate(prompts)]
    outs, sizes = {}, {}
    for graph in (False, True):
        e = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=graph)
        e.load_model(folder)
        e.setup_caches(max_batch_size=13, max_seq_length=96, page_size=8, check_kernel_errors=True,
                       enable_selective_cache=selective, full_cache_layers=[1], subset_cache_size=4, L=2)
        first = len(e.scheduler.requests)
        e.add_requests(prompts, lengths, [])
        while e.scheduler.has_work():
            e.step()
        outs[graph] = [r.output for r in e.scheduler.requests[first:]]
        sizes[graph] = sorted(e.runner._graphs)
        e.runner.cache.check()
        assert all(v == 0 for v in e.runner.cache.pages_in_use().values())
    assert outs[True] == outs[False]
    assert [len(o) for o in outs[True]] == [6 + 2 * i for i in range(13)]
    assert sizes[True] == [1, 2, 3, 4, 5, 6, 7, 8, 12, 13] and sizes[False] == []
    assert e.runner.graph_batch(9) == 12 and e.runner.graph_batch(13) == 13 and e.runner.graph_batch(8) == 8


def test_waves_of_requests_repeat_their_outputs(model_folders):
    """Three waves of 20 to 40 requests drawn from 12 prompts, more than the engine's 20 slots, so
    that requests wait, batches grow and shrink through the graph sizes 1..8, 12, 16, 20 and
    pages are used again: in 32-bit a prompt gives the same tokens wherever it runs, and the
    cache is empty after every wave."""
    import random
    from delta_b200.engine import LMBackend
    folder = model_folders["A"]
    vocab = PlainYi(folder).cfg.vocab
    rng = random.Random(3)
    base = [helpers.random_tokens(rng.randrange(3, 60), vocab, 400 + i) for i in range(12)]
    e = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=True)
    e.load_model(folder)
    e.setup_caches(max_batch_size=20, max_seq_length=128, page_size=16, max_tokens_per_step=96, check_kernel_errors=True)
    seen = {}
    for wave in range(3):
        idx = [rng.randrange(12) for _ in range(rng.randrange(20, 41))]
        first = len(e.scheduler.requests)
        e.add_requests([base[i] for i in idx], [len(base[i]) + 10 + 5 * (i % 5) for i in idx], [])
        while e.scheduler.has_work():
            e.step()
        for i, r in zip(idx, e.scheduler.requests[first:]):
            assert len(r.output) == 10 + 5 * (i % 5), r.finish_reason
            assert seen.setdefault(i, r.output) == r.output, f"wave {wave}: prompt {i} gave other tokens than before"
        e.runner.cache.check()
        assert all(v == 0 for v in e.runner.cache.pages_in_use().values())
    assert set(e.runner._graphs) >= {8, 12, 16, 20}


def test_a_failed_graph_recording_falls_back_to_eager_steps(model_folders, monkeypatch):
    """When recording a decode step fails, that batch size runs eagerly from then on, the reason is
    counted, and the tokens are the ones of the engine without CUDA graphs."""
    from delta_b200.engine import LMBackend
    folder = model_folders["A"]
    vocab = PlainYi(folder).cfg.vocab
    prompts = [helpers.random_tokens(n, vocab, 600 + i) for i, n in enumerate([12, 30, 7])]

    def run(graphs):
        e = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=graphs)
        e.load_model(folder)
        e.setup_caches(max_batch_size=3, max_seq_length=64, page_size=16)
        return e.generate(prompts, 12), e

    want, _ = run(False)

    class Refuses:
        def __init__(self, *a, **k):
            raise RuntimeError("recording is refused in this test")
    monkeypatch.setattr(torch.cuda, "CUDAGraph", Refuses)
    got, e = run(True)
    assert got == want
    assert e.runner.graph_captures == 0 and e.runner.graph_replays == 0
    assert sum(e.runner.graph_fallbacks.values()) >= 8 and all("capture failed" in k for k in e.runner.graph_fallbacks)
    assert "refused" in e.runner._graphs[3]["error"]


def test_garbage_of_an_earlier_engine_does_not_spoil_a_recording(model_folders):
    """An engine that is no longer used, with its CUDA graphs, may lie in a reference cycle until Python's
    garbage collector meets it.  If that happens while a later engine records a decode step, freeing the
    old graphs is a call that CUDA does not allow during a recording, and the recording is lost.  Here the
    old engine becomes garbage in the middle of the second engine's recording and a collection follows at
    once if the collector is enabled at that moment (which is when an automatic collection could run; when
    one really runs depends on Python's counts of objects); the second engine must still record."""
    import gc
    from delta_b200.engine import LMBackend
    folder = model_folders["A"]
    vocab = PlainYi(folder).cfg.vocab
    prompts = [helpers.random_tokens(n, vocab, 650 + i) for i, n in enumerate([12, 30, 7])]

    def engine():
        e = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=True)
        e.load_model(folder)
        e.setup_caches(max_batch_size=3, max_seq_length=64, page_size=16)
        return e

    old = engine()
    want = old.generate(prompts, 12)
    assert old.runner.graph_captures >= 1
    cycle = [old]
    cycle.append(cycle)
    box = {"old": cycle}
    del old, cycle
    e = engine()
    forward = e.runner.model.forward
    dropped = []

    def forward_that_drops_the_old_engine(ctx):
        if box and torch.cuda.is_current_stream_capturing():
            box.clear()                   # from here on only the collector can free the old engine
            dropped.append(gc.isenabled())
            if gc.isenabled():
                gc.collect()
        return forward(ctx)
    e.runner.model.forward = forward_that_drops_the_old_engine
    got = e.generate(prompts, 12)
    assert not e.runner.graph_fallbacks and e.runner.graph_captures >= 1
    assert dropped == [False] and got == want
