"""What only runs in bfloat16, recorded into CUDA graphs: the decode kernel that also rotates and
appends, its variant that fetches runs of pages by TMA (with the padding slot's spare page in the
rounded-up batches), the product kernels the tuner chose, DELTA's planner inside the graph, and
steps launched ahead of the host.  Every variant of the engine is compared, logits and all, with
the plain implementation run on the tokens that variant generated; the run-ahead engine must give
exactly the tokens of the same engine without run-ahead (the same recorded steps on the same data)."""
import pytest
import torch

import helpers
from plain_yi import PlainYi, Selective
from test_gpu_model import bound_for
from test_gpu_odd_sizes import ODD

pytestmark = pytest.mark.gpu

SEL = dict(full_cache_layers=[0], subset_cache_size=3, L=2)     # layer 0 plans, layer 1 reads the chosen pages
PS = 16
N_REQ = 13


@pytest.fixture(scope="module")
def folders(tmp_path_factory, model_folders):
    from delta_b200.weights import write_random_model
    root = tmp_path_factory.mktemp("graph_models")
    return {"D": model_folders["D"], "hd128g3": write_random_model(root / "hd128g3", ODD["hd128g3"], seed=11, dtype=torch.float32)}


def run(folder, prompts, lengths, *, graphs, ahead, hook, selective, shuffle):
    from delta_b200.engine import LMBackend
    from delta_b200.parts.attention import SELECTED_COUNT, SELECTED_PAGES
    e = LMBackend(dtype="bfloat16", device="cuda:0", cuda_graph_decode=graphs)
    e.run_ahead = ahead
    e.load_model(folder)
    e.setup_caches(max_batch_size=N_REQ, max_seq_length=192, page_size=PS, enable_selective_cache=selective,
                   shuffle_pages=7 if shuffle else None, **SEL)
    logits, planned = {}, {}

    def keep(plan, lg):
        rows = [x for x in plan if x.samples]
        for x, row in zip(rows, lg.float().cpu()):
            logits[(x.request.id, x.start + x.count - 1)] = row
        if selective:
            # one planner (layer 0): after the step its choice for each decode row is the row's state
            pages, counts = e.runner.cache.states[SELECTED_PAGES].cpu(), e.runner.cache.states[SELECTED_COUNT].cpu()
            for x in plan:
                n = int(counts[x.request.slot])
                if x.decode and n >= 0:
                    planned[(x.request.id, 0, x.start)] = pages[x.request.slot, :n].tolist()
    if hook:
        e.on_step_logits = keep
    e.add_requests(prompts, lengths, [])
    steps_ahead = 0
    while e.scheduler.has_work():
        steps_ahead += int(e._ahead is not None)
        e.step()
    e.runner.cache.check()
    assert all(v == 0 for v in e.runner.cache.pages_in_use().values())
    outs = [list(r.output) for r in e.scheduler.requests]
    return outs, logits, planned, e, steps_ahead


def against_plain(plain, prompts, outs, logits, planned, selective, what):
    worst = 0.0
    for i, (p, o) in enumerate(zip(prompts, outs)):
        seq = p + o[:-1]
        sel = Selective(SEL["full_cache_layers"], SEL["subset_cache_size"], SEL["L"], 1.0, PS, len(p)) if selective else None
        forced = {(l, q): pg for (r, l, q), pg in planned.items() if r == i} if selective else None
        if selective:
            # nearly equal page scores may order otherwise in bfloat16: the choices must agree almost everywhere,
            # and the logits are compared with the plain implementation attending to the engine's pages
            plain.forward(seq, sel)
            own = dict(plain.last_planned)
            same = sum(planned.get((i, l, q)) == pg for (l, q), pg in own.items())
            assert same >= 0.9 * len(own), f"{what}: request {i}: only {same} of {len(own)} page choices agree with the plain ones"
        ref = plain.forward(seq, sel, forced=forced)
        for pos in range(len(p) - 1, len(seq)):
            err = (logits[(i, pos)] - ref[pos]).abs()
            assert bool((err <= bound_for(ref, "bfloat16")).all()), f"{what}: request {i} position {pos}: max error {err.max().item():.3e}"
            worst = max(worst, err.max().item())
    return worst


@pytest.mark.parametrize("shuffle", [False, True])
@pytest.mark.parametrize("selective", [False, True])
@pytest.mark.parametrize("which", ["D", "hd128g3"])
def test_bfloat16_decode_from_graphs(folders, monkeypatch, which, selective, shuffle):
    from delta_b200.parts import attention_kernels
    monkeypatch.setattr(attention_kernels, "TMA_MIN_TILES", 1)   # short blocks too take the variant that fetches runs by TMA
    folder = folders[which]
    plain = PlainYi(folder, rounding="bfloat16")
    prompts = [helpers.random_tokens(20 + 7 * i, plain.cfg.vocab, 900 + i) for i in range(N_REQ)]
    lengths = [len(p) + 8 + 6 * i for i, p in enumerate(prompts)]        # they end one after the other: 13, 12, ... rows
    kw = dict(selective=selective, shuffle=shuffle)

    outs, lg, pl, e, _ = run(folder, prompts, lengths, graphs=False, ahead=False, hook=True, **kw)
    assert e.runner.graph_replays == 0
    w_eager = against_plain(plain, prompts, outs, lg, pl, selective, f"{which} eager")
    if selective:
        assert pl, "the case never selected anything"

    outs_g, lg, pl, e, _ = run(folder, prompts, lengths, graphs=True, ahead=False, hook=True, **kw)
    assert e.runner.graph_replays > 30 and not e.runner.graph_fallbacks
    assert {12, 13} <= set(e.runner._graphs) and all(g["graph"] is not None for b, g in e.runner._graphs.items() if b in (12, 8, 4))
    w_graph = against_plain(plain, prompts, outs_g, lg, pl, selective, f"{which} graphs")
    print(f"\nworst bfloat16 logit error {which} selective={selective} shuffle={shuffle}: eager {w_eager:.2e}, graphs {w_graph:.2e}")

    # steps launched ahead of the host replay the same recorded steps on the same data: the same tokens, exactly
    outs_n, _, _, e, n0 = run(folder, prompts, lengths, graphs=True, ahead=False, hook=False, **kw)
    outs_a, _, _, e, n1 = run(folder, prompts, lengths, graphs=True, ahead=True, hook=False, **kw)
    assert n0 == 0 and n1 > 20
    assert outs_a == outs_n == outs_g


def test_scratch_addresses_stay_when_graphs_of_other_sizes_are_recorded(folders):
    """Working buffers whose addresses recorded steps hold are made once, large enough for every
    batch size: recording 1, 2 and 8 rows in turn moves none of them, and the first graph still
    gives what an eager step gives."""
    from delta_b200.config import EngineConfig
    from delta_b200.config.selective_cache import SelectiveCacheConfig
    from delta_b200.engine.step import ModelRunner, RowInput
    sel = SelectiveCacheConfig(full_cache_layers=(0,), subset_cache_size=3, L=2)
    # (2,048 tokens at most: then a request is split more than five ways, which go through the buffer of partial
    # results and the merge kernel; up to five splits merge inside a cluster and need no buffer)
    cfg = EngineConfig(max_batch=8, max_seq_len=2048, page_size=PS, dtype="bfloat16", cuda_graph_decode=True,
                       options=dict(selective_cache=sel))
    r = ModelRunner(folders["hd128g3"], engine_config=cfg)
    vocab = ODD["hd128g3"]["vocab_size"]
    slots = [r.cache.acquire_slot() for _ in range(8)]
    lens = [200 + 9 * i for i in range(8)]
    for s, n in zip(slots, lens):
        r.run_rows([RowInput(s, helpers.random_tokens(n, vocab, 50 + s), 0, [])])

    def decode(batch):
        rows = [RowInput(s, [5 + s], lens[i], [0], flags=1) for i, s in enumerate(slots[:batch])]
        for row in rows:
            r.cache.grow(row.slot, row.start_pos + 1)
        logits, _ = r.step_and_sample(rows)
        return logits.clone()

    seen = {}
    for batch in (1, 2, 8, 1):
        for _ in range(3):          # two eager runs, then the recording and a replay
            out = decode(batch)
        assert r._graphs[batch]["graph"] is not None
        ptrs = {k: v.data_ptr() for k, v in r._scratch.items() if isinstance(v, torch.Tensor)}
        for k, p in seen.items():
            assert ptrs[k] == p, f"working buffer '{k}' moved after a step of {batch} rows was recorded"
        seen.update(ptrs)
    assert "__retired__" not in r._scratch
    assert {"attention.decode_partials", "delta.dump", "delta.lse", "delta.page_scores"} <= set(seen)
    # the graph of one row, recorded first, after all the others: equal to the same step run eagerly
    replayed = decode(1)
    eager = ModelRunner(folders["hd128g3"], engine_config=EngineConfig(max_batch=8, max_seq_len=512, page_size=PS, dtype="bfloat16",
                                                                        options=dict(selective_cache=sel)))
    s0 = eager.cache.acquire_slot()
    eager.run_rows([RowInput(s0, helpers.random_tokens(lens[0], vocab, 50 + slots[0]), 0, [])])
    eager.cache.grow(s0, lens[0] + 1)
    want, _ = eager.step_and_sample([RowInput(s0, [5 + slots[0]], lens[0], [0], flags=1)])
    r.check_errors()
    assert (replayed[0] - want[0]).abs().max().item() <= bound_for(want[0], "bfloat16")
