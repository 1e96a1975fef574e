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
from plain_yi import PlainYi

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def replay(folder, dtype, steps_json, out_dir, max_tokens):
    cmd = [str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
           "--max-tokens", str(max_tokens)]
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
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=2.5e-2, rtol=2e-2)
    by_step = {}
    for (k, i, p) in wanted:
        by_step.setdefault(k, []).append((i, p))
    for k, items in by_step.items():
        got = torch.from_numpy(np.fromfile(out / f"{k}.f32", dtype="<f4").reshape(len(items), V))
        for row, (i, p) in zip(got, items):
            assert torch.allclose(row, refs[i][p], **tol), f"step {k}, request {i}, position {p}"
