"""bin/trace_run: the replay program drives the engine's own step function; its logits
equal the plain implementation's under several ways of cutting, in both precisions."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
from plain_yi import PlainYi, Selective
from test_gpu_model import bound_for

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def replay(folder, dtype, steps_json, out_dir, max_tokens, extra=()):
    cmd = [str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
           "--max-tokens", str(max_tokens), *map(str, extra)]
    r = subprocess.run(cmd, input="\n".join(json.dumps(s) for s in steps_json) + "\n", capture_output=True, text=True,
                       cwd=ROOT, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps_json]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run(model_folders, tmp_path, dtype):
    folder = model_folders["A"]
    plain = PlainYi(folder, rounding="bfloat16" if dtype == "bfloat16" else None)
    V = plain.cfg.vocab
    lengths = [40, 70, 33, 64, 50]
    prompt_lens = [20, 30, 33, 10, 25]
    toks = [helpers.random_tokens(n, V, 60 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(t) for t in toks]
    sched, ends = helpers.mixed(lengths, prompt_lens, seed=11)
    steps_json, wanted = [], []
    for k, (step, end) in enumerate(zip(sched, ends)):
        entries = []
        for (i, start, count) in step:
            want = list(range(count)) if (k % 3) else [count - 1]
            entries.append(dict(id=f"r{i}", tokens=toks[i][start:start + count], want=want))
            wanted.extend((k, i, start + w) for w in want)
        steps_json.append(dict(step=k, entries=entries, end=[f"r{i}" for i in end]))
    # each live request counts rounded up to 64 tokens: four live requests of up to 70 tokens
    out = tmp_path / "logits"
    replay(folder, dtype, steps_json, out, max_tokens=4 * 128)
    by_step = {}
    for (k, i, p) in wanted:
        by_step.setdefault(k, []).append((i, p))
    for k, items in by_step.items():
        got = torch.from_numpy(np.fromfile(out / f"{k}.f32", dtype="<f4").reshape(len(items), V))
        for row, (i, p) in zip(got, items):
            assert (row - refs[i][p]).abs().max().item() <= bound_for(refs[i], dtype), f"step {k}, request {i}, position {p}"


def schedules(lengths, prompt_lens):
    """The four ways of cutting, with every position from the prompt's end on fed alone: {name: (steps, ends)}."""
    alone = []
    for i, (n, pl) in enumerate(zip(lengths, prompt_lens)):
        alone.append([(i, 0, pl)])
        alone.extend([[(i, p, 1)] for p in range(pl, n)])
    tail = []
    for i, (n, pl) in enumerate(zip(lengths, prompt_lens)):
        head = min(pl, max(1, n - 32))
        tail.append([(i, 0, head)])
        tail.extend([[(i, p, 1)] for p in range(head, n)])
    portions = []
    sizes = (7, 2, 13, 2, 5, 3, 16, 2, 9)
    for i, (n, pl) in enumerate(zip(lengths, prompt_lens)):
        p, j = 0, i
        while p < pl:
            c = min(sizes[j % len(sizes)], pl - p)
            portions.append([(i, p, c)])
            p, j = p + c, j + 1
        portions.extend([[(i, q, 1)] for q in range(pl, n)])

    def ends_of(steps):
        last = {}
        for k, st in enumerate(steps):
            for (i, _, _) in st:
                last[i] = k
        return [[i for i, kk in last.items() if kk == k] for k in range(len(steps))]
    mixed, mixed_ends = helpers.mixed(lengths, prompt_lens, seed=5)
    return {"alone": (alone, ends_of(alone)), "last 32 one by one": (tail, ends_of(tail)),
            "portions": (portions, ends_of(portions)), "mixed": (mixed, mixed_ends)}


@pytest.mark.parametrize("dtype, ahead", [("float32", False), ("bfloat16", False), ("float32", True)])
def test_trace_run_with_the_selective_cache(model_folders, tmp_path, dtype, ahead):
    """Configuration B with full_cache_layers=[1] and 4 pages through the program itself, in the four
    ways of cutting: logits and the pages each planner chose against the plain implementation.  The
    mixed replay runs with so few pages that they are used again, handed out in a shuffled order."""
    folder, ps, k = model_folders["B"], helpers.PAGE_SIZE["B"], 4
    plain = PlainYi(folder, rounding="bfloat16" if dtype == "bfloat16" else None)
    V = plain.cfg.vocab
    lengths, prompt_lens = [60, 100, 45, 130, 80], [9, 40, 20, 35, 1]
    toks = [helpers.random_tokens(n, V, 160 + i) for i, n in enumerate(lengths)]
    # ``ahead``: pages counted as the reference's scheduler counts them (--count_page_ahead); the empty page it adds
    # can be among the chosen, nothing is read from it, and the program leaves it out of what it writes
    sel = [Selective([1], k, 8, 1.0, ps, pl, trailing_empty_page=ahead) for pl in prompt_lens]
    refs, want_pages = [], {}
    for i, t in enumerate(toks):
        refs.append(plain.forward(t, sel[i]))
        want_pages.update({(i, l, p): [j for j in pg if j * ps <= p] for (l, p), pg in plain.last_planned.items()})
    assert want_pages
    opts = ["--enable_selective_cache", "--full_cache_layers", 1, "--subset_cache_size", k, "--L", 8, "--page-size", ps,
            "--dump-selected"] + (["--count_page_ahead"] if ahead else [])
    for name, (steps, ends) in schedules(lengths, prompt_lens).items():
        steps_json = []
        for n, (step, end) in enumerate(zip(steps, ends)):
            entries = [dict(id=f"r{i}", tokens=toks[i][a:a + c], want=list(range(c)),
                            **({"decode": True} if (c == 1 and a >= prompt_lens[i]) else {})) for (i, a, c) in step]
            steps_json.append(dict(step=n, entries=entries, end=[f"r{i}" for i in end]))
        out = tmp_path / f"{dtype}_{name.replace(' ', '_')}"
        extra = list(opts)
        if name == "mixed":
            extra += ["--num-pages", helpers.peak_pages(steps, ends, ps), "--shuffle-pages", 3]
        replay(folder, dtype, steps_json, out, max_tokens=4 * 192, extra=extra)
        got_pages = {}
        for f in out.glob("*.selected.json"):
            for item in json.loads(f.read_text()):
                got_pages[(int(item["id"][1:]), int(item["part"].split(".")[2]), item["position"])] = item["pages"]
        assert set(got_pages) == set(want_pages), f"{name}: planned at other places"
        use = refs
        if dtype == "float32":
            assert got_pages == want_pages, f"{name}: other pages were chosen"
        else:
            same = sum(got_pages[key] == want_pages[key] for key in want_pages)
            assert same >= 0.9 * len(want_pages), f"{name}: only {same} of {len(want_pages)} choices agree"
            use = [plain.forward(t, sel[i], forced={(l, p): pg for (r, l, p), pg in got_pages.items() if r == i}) for i, t in enumerate(toks)]
        for n, step in enumerate(steps):
            rows = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, V))
            at = 0
            for (i, a, c) in step:
                for p in range(a, a + c):
                    assert (rows[at] - use[i][p]).abs().max().item() <= bound_for(use[i], dtype), f"{name}: step {n}, request {i}, position {p}"
                    at += 1
            assert at == rows.shape[0]


def test_trace_run_decodes_from_cuda_graphs(model_folders, tmp_path):
    """--cuda_graph_decode: steps of single tokens go through the recorded decode step (bfloat16, head
    size 64: the fused decode kernel inside the graph), more than four requests live (--max-live)."""
    folder = model_folders["D"]
    plain = PlainYi(folder, rounding="bfloat16")
    V = plain.cfg.vocab
    lengths = [50, 64, 33, 47, 58, 40]
    toks = [helpers.random_tokens(n, V, 260 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(t) for t in toks]
    steps_json = [dict(step=0, entries=[dict(id=f"r{i}", tokens=t[:20], want=[19]) for i, t in enumerate(toks)], end=[])]
    for p in range(20, max(lengths)):
        live = [i for i, n in enumerate(lengths) if p < n]
        steps_json.append(dict(step=len(steps_json), entries=[dict(id=f"r{i}", tokens=[toks[i][p]], want=[0], decode=True) for i in live],
                               end=[f"r{i}" for i in live if p == lengths[i] - 1]))
    out = tmp_path / "graphs"
    replay(folder, "bfloat16", steps_json, out, max_tokens=6 * 64, extra=["--cuda_graph_decode", "--max-live", 6])
    for n, st in enumerate(steps_json):
        rows = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(st["entries"]), V))
        for row, e in zip(rows, st["entries"]):
            i = int(e["id"][1:])
            p = 19 if n == 0 else 20 + n - 1
            assert (row - refs[i][p]).abs().max().item() <= bound_for(refs[i], "bfloat16"), f"step {n}, request {i}"
