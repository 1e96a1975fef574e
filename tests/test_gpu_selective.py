"""DELTA's selective cache on the GPU against the plain implementation that attends
to the same chosen pages: logits, page scores and the chosen pages themselves."""
import pytest
import torch

import helpers
from plain_yi import PlainYi, Selective
from test_gpu_model import compare

pytestmark = pytest.mark.gpu

CASES = [
    # which, full_cache_layers, k, L, ratio, count_page_ahead
    ("B", (1,), 4, 8, 1.0, False),      # layer 0 reads the last 4 pages, layer 1 plans, layer 2 reads the chosen pages
    ("B", (0,), 3, 1, 1.0, False),
    ("A", (0,), 2, 1, 1.5, False),      # selection starts only when pages / k > 1.5
    ("C", (0,), 2, 1, 1.0, False),      # layer 0 plans for layer 2; the windowed layers 1 and 3 take no selection
    ("B", (0, 1), 2, 2, 1.0, False),    # two full layers, the second one plans
    ("D", (0,), 3, 2, 1.0, False),      # head size 64: the tensor-core decode kernel dumps, scores and reads chosen pages
    ("B", (1,), 4, 2, 1.0, True),       # pages counted as the reference counts them: an empty one once the newest is full
    ("D", (0,), 3, 3, 1.0, True),
    ("A", (0,), 2, 2, 1.5, True),
]


def plain_logits(plain, toks, prompt_lens, sel, ps, forced=None):
    refs, planned = [], {}
    for i, (t, pl) in enumerate(zip(toks, prompt_lens)):
        f = None if forced is None else {(l, p): pg for (r, l, p), pg in forced.items() if r == i}
        refs.append(plain.forward(t, Selective(list(sel.full_cache_layers), sel.subset_cache_size, sel.L,
                                               sel.compression_ratio, ps, pl, trailing_empty_page=sel.count_page_ahead), forced=f))
        # (the empty page that the reference's count adds can be among the chosen; nothing is read from it,
        # and the engine leaves it out of its list)
        planned.update({(i, l, p): [j for j in pg if j * ps <= p] for (l, p), pg in plain.last_planned.items()})
    return refs, planned


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which, full, k, L, ratio, ahead", CASES)
def test_selective_cache(model_folders, which, full, k, L, ratio, ahead, dtype):
    """In 32 bit the engine chooses the pages the plain implementation chooses, and the logits
    agree.  In bfloat16 two nearly equal page scores may come out in the other order, so there
    the plain implementation attends to the pages the engine chose (and the two choices must
    still agree almost everywhere)."""
    from delta_b200.config import EngineConfig, SelectiveCacheConfig
    from delta_b200.engine.step import ModelRunner
    folder = model_folders[which]
    ps = helpers.PAGE_SIZE[which]
    sel = SelectiveCacheConfig(full_cache_layers=full, subset_cache_size=k, L=L, compression_ratio=ratio, count_page_ahead=ahead)
    lengths = [30, 70, 110, 150]
    prompt_lens = [9, 20, 35, 40]
    plain = PlainYi(folder, rounding="bfloat16" if dtype == "bfloat16" else None)
    toks = [helpers.random_tokens(n, plain.cfg.vocab, 40 + i) for i, n in enumerate(lengths)]
    refs, want = plain_logits(plain, toks, prompt_lens, sel, ps)
    assert want, "the case never selected anything"

    def runner(num_pages):
        cfg = EngineConfig(max_batch=4, max_seq_len=256, page_size=ps, num_pages=num_pages, dtype=dtype, options=dict(selective_cache=sel))
        return ModelRunner(folder, engine_config=cfg)

    def check(res, got, what):
        assert set(got) == set(want), f"{what}: the engine planned at other (request, layer, position) places"
        if dtype == "float32":
            assert got == want, f"{what}: the engine chose other pages"
            compare(res, refs, lengths, dtype, what)
        else:
            same = sum(got[key] == want[key] for key in want)
            assert same >= 0.9 * len(want), f"{what}: only {same} of {len(want)} choices agree"
            forced_refs, _ = plain_logits(plain, toks, prompt_lens, sel, ps, forced=got)
            compare(res, forced_refs, lengths, dtype, what)

    # each request alone: the prompt in one step, then token by token
    steps = []
    for i, (n, pl) in enumerate(zip(lengths, prompt_lens)):
        steps.append([(i, 0, pl)])
        steps.extend([[(i, p, 1)] for p in range(pl, n)])
    got = {}
    res = helpers.run_schedule(runner(4 * (256 // ps)), toks, steps, prompt_lens=prompt_lens, planned=got)
    check(res, got, "alone")

    # prompts in portions, decode tokens of several requests in one step, few pages
    sched, ends = helpers.mixed(lengths, prompt_lens, seed=5)
    got = {}
    res = helpers.run_schedule(runner(helpers.peak_pages(sched, ends, ps)), toks, sched, ends, prompt_lens=prompt_lens,
                               planned=got)
    check(res, got, "mixed")


def test_chosen_pages_equal_the_plain_ones(model_folders):
    """One request, float32: after every decode step the state slot holds exactly the
    pages that the plain implementation chose for that position."""
    from delta_b200.config import EngineConfig, SelectiveCacheConfig
    from delta_b200.engine.step import ModelRunner, RowInput
    from delta_b200.parts.attention import SELECTED_COUNT, SELECTED_PAGES
    folder, ps, k = model_folders["B"], helpers.PAGE_SIZE["B"], 4
    sel = SelectiveCacheConfig(full_cache_layers=(1,), subset_cache_size=k, L=2)
    plain = PlainYi(folder)
    n, pl = 120, 16
    toks = helpers.random_tokens(n, plain.cfg.vocab, 77)
    plain.forward(toks, Selective([1], k, 2, 1.0, ps, pl))
    want = plain.last_selection
    r = ModelRunner(folder, engine_config=EngineConfig(max_batch=2, max_seq_len=128, page_size=ps, dtype="float32", options=dict(selective_cache=sel)))
    slot = r.cache.acquire_slot()
    r.run_rows([RowInput(slot, toks[:pl], 0, [])])
    checked = 0
    for p in range(pl, n):
        r.run_rows([RowInput(slot, toks[p:p + 1], p, [0], flags=1)])
        count = int(r.cache.states[SELECTED_COUNT][slot])
        if (2, p) in want:
            assert count == k
            assert r.cache.states[SELECTED_PAGES][slot, :count].tolist() == want[(2, p)], f"position {p}"
            checked += 1
        else:
            assert count == -1
    assert checked > 50


# ---- the engine beside stored outputs of the reference itself ------------------------------------

def golden_model(tmp_path_factory, name):
    import sys
    from pathlib import Path
    golden = Path(__file__).parent / "golden"
    sys.path.insert(0, str(golden))
    from make_reference_model_golden import checksum
    from plain_yi import read_safetensors_plain
    from delta_b200.weights import write_random_model
    M = torch.load(golden / name)
    folder = write_random_model(tmp_path_factory.mktemp("golden") / "hf", M["config"], M["seed"], torch.float32)
    if checksum(read_safetensors_plain(folder / "model.safetensors")) != M["weights_sha256"]:
        pytest.skip("this torch draws other random weights from the seed than the one the stored logits were made with")
    return M, folder


def worst_against(ref, got):
    scale = ref.abs().max().item()
    err = (got - ref).abs().amax(dim=-1) / scale
    return err.max().item(), int(err.argmax())


@pytest.mark.parametrize("graphs", [False, True])
def test_the_engine_follows_the_reference_with_delta_on(tmp_path_factory, graphs):
    """The reference ran one request with DELTA on (layer 0 the newest pages, layer 1 plans, layer 2 the chosen
    pages) on this kind of GPU; its logits at all 119 positions are stored.  The engine, in bfloat16 with the
    pages counted as the reference counts them, is fed the same tokens: every position agrees to the rounding
    of bfloat16 (the bound is that of the plain implementation's comparison with the same file, 1.5 % of the
    largest logit).  With the engine's own count the positions where a page has just filled differ, by far more."""
    from delta_b200.config import EngineConfig, SelectiveCacheConfig
    from delta_b200.engine.step import ModelRunner, RowInput
    M, folder = golden_model(tmp_path_factory, "reference_selective_logits.pt")
    s, prompt, out = M["selective"], M["prompt"], M["output"]
    ref = M["logits"].float()
    seq = prompt + out[:-1]
    worst = {}
    for ahead in (True, False):
        sel = SelectiveCacheConfig(full_cache_layers=tuple(s["full_cache_layers"]), subset_cache_size=s["subset_cache_size"],
                                   L=s["L"], compression_ratio=s["compression_ratio"], count_page_ahead=ahead)
        r = ModelRunner(folder, engine_config=EngineConfig(max_batch=2, max_seq_len=128, page_size=M["page_size"], dtype="bfloat16",
                                                           cuda_graph_decode=graphs, options=dict(selective_cache=sel)))
        slot = r.cache.acquire_slot()
        rows = [r.run_rows([RowInput(slot, prompt, 0, list(range(len(prompt))))]).float().cpu()]
        for p in range(len(prompt), len(seq)):
            row = RowInput(slot, seq[p:p + 1], p, [0], flags=1)
            if graphs:          # the way generation runs its decode steps: sampled, and replayed from a CUDA graph
                r.cache.grow(slot, p + 1)
                rows.append(r.step_and_sample([row])[0].float().cpu())
                r.cache.advance(slot, p + 1)
            else:
                rows.append(r.run_rows([row]).float().cpu())
        r.check_errors()
        worst[ahead] = worst_against(ref, torch.cat(rows))
        if graphs and ahead:
            assert r.graph_replays > 50
    print(f"worst difference / largest logit: counted as the reference {worst[True]}, the engine's own count {worst[False]}")
    assert worst[True][0] <= 0.015, f"position {worst[True][1]} differs by {worst[True][0]:.4f} of the largest logit"
    assert worst[False][0] > 0.05 and (worst[False][1] + 1) % M["page_size"] == 0


def test_the_engine_follows_the_reference_without_selection(tmp_path_factory):
    """The stored logits of the reference's plain path (three requests of 40, 23 and 1 prompt tokens, 24 decoded
    tokens each), against the engine in bfloat16 fed the same tokens as one batch."""
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner, RowInput
    M, folder = golden_model(tmp_path_factory, "reference_model_logits.pt")
    r = ModelRunner(folder, engine_config=EngineConfig(max_batch=4, max_seq_len=128, page_size=16, dtype="bfloat16"))
    seqs = [p + o[:-1] for p, o in zip(M["prompts"], M["outputs"])]
    slots = [r.cache.acquire_slot() for _ in seqs]
    got = [[] for _ in seqs]
    res = r.run_rows([RowInput(sl, p, 0, list(range(len(p)))) for sl, p in zip(slots, M["prompts"])]).float().cpu()
    at = 0
    for i, p in enumerate(M["prompts"]):
        got[i].append(res[at:at + len(p)])
        at += len(p)
    for j in range(len(M["outputs"][0]) - 1):
        res = r.run_rows([RowInput(sl, [s[len(p) + j]], len(p) + j, [0], flags=1) for sl, s, p in zip(slots, seqs, M["prompts"])]).float().cpu()
        for i in range(len(seqs)):
            got[i].append(res[i:i + 1])
    for i in range(len(seqs)):
        w, at = worst_against(M["logits"][i].float(), torch.cat(got[i]))
        assert w <= 0.015, f"request {i}: position {at} differs by {w:.4f} of the largest logit"
