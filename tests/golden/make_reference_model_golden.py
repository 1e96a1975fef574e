"""Makes tests/golden/reference_model_logits.pt: logits of hoenza/DELTA's own model code on a tiny
random model, for the parts of it that need a GPU (rotary positions, the cache append, attention,
the whole forward pass).  Run on a machine with a CUDA device, the reference on the path:

    PYTHONPATH=/path/to/hoenza-DELTA python tests/golden/make_reference_model_golden.py OUT.pt
    PYTHONPATH=/path/to/hoenza-DELTA python tests/golden/make_reference_model_golden.py --selective OUT2.pt

The reference's stock path is driven (tests/reasoni.py:320-342, 449-455): ``LMBackend`` ->
``load_model`` (a ``model.pth`` whose folder names the configuration; the tiny configuration is added
to its table of configurations at run time, DELTA/Engine/DELTA/model.py:72-97) -> ``setup_caches`` ->
``add_requests`` -> ``run_scheduler_loop``.  Its model returns only the argmax (model.py:320-323), so
a forward hook on its output matrix keeps the logits of every row of every step.

The weights are the tiny model folder's that ``delta_b200.weights.write_random_model`` writes from
(configuration, seed), renamed to the reference's names; the rows of every head of q_proj and
k_proj are reordered (j, j + head/2) -> (2j, 2j + 1), which is what the reference's missing
converter does for its neighbour-pair rotation (model.py:165-175, ``interleave=True``).  If the
plain implementation, which reads the unconverted folder and rotates pairs (j, j + head/2), gives
the reference's logits, then half-split rotation on unconverted rows, the exponent of theta, the
mapping of query heads to key-value heads, the placement of the norms and the untied output matrix
are all what the reference computes.

With ``--selective`` a second file is made, tests/golden/reference_selective_logits.pt: one request through
the reference with DELTA on (three layers, ``full_cache_layers=[1]``: layer 0 reads the most recent pages,
layer 1 plans, layer 2 reads the chosen pages; 4 pages of 16 tokens, the last 2 always kept), a prompt of 20
tokens (fewer pages than the subset, so that the reference's prompt step reads everything, as the engine's
always does) and 100 decoded tokens.

tests/test_plain_against_reference.py compares the plain implementation with the stored logits.
"""
import hashlib
import json
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

NAME = "tiny-golden-yi"
CONFIG = dict(architectures=["LlamaForCausalLM"], hidden_act="silu", tie_word_embeddings=False, model_type="llama",
              hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=320,
              vocab_size=192, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=256, torch_dtype="float32")
SEED = 21
PROMPT_LENS = [40, 23, 1]
MAX_LEN = 128       # the reference wants a multiple of 128
NEW_TOKENS = [24, 24, 24]


def checksum(tensors) -> str:
    h = hashlib.sha256()
    for k in sorted(tensors):
        h.update(k.encode())
        h.update(tensors[k].to(torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


def to_reference_names(w, cfg):
    """The state dict the reference loads (module names: model.py:134-137, 333-336, 369-370, 498-500)."""
    H, KV = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg["hidden_size"] // H

    def pairs(t, heads):    # rows (j, j + hd/2) of each head become neighbours (2j, 2j + 1)
        t = t.view(heads, 2, hd // 2, -1).transpose(1, 2).reshape(heads * hd, -1)
        return t.contiguous()
    sd = {"tok_embeddings.weight": w["model.embed_tokens.weight"], "norm.weight": w["model.norm.weight"],
          "output.weight": w["lm_head.weight"]}
    for i in range(cfg["num_hidden_layers"]):
        p, q = f"model.layers.{i}.", f"layers.{i}."
        sd[q + "attention.wq.weight"] = pairs(w[p + "self_attn.q_proj.weight"], H)
        sd[q + "attention.wk.weight"] = pairs(w[p + "self_attn.k_proj.weight"], KV)
        sd[q + "attention.wv.weight"] = w[p + "self_attn.v_proj.weight"]
        sd[q + "attention.wo.weight"] = w[p + "self_attn.o_proj.weight"]
        sd[q + "feed_forward.w1.weight"] = w[p + "mlp.gate_proj.weight"]
        sd[q + "feed_forward.w3.weight"] = w[p + "mlp.up_proj.weight"]
        sd[q + "feed_forward.w2.weight"] = w[p + "mlp.down_proj.weight"]
        sd[q + "attention_norm.weight"] = w[p + "input_layernorm.weight"]
        sd[q + "ffn_norm.weight"] = w[p + "post_attention_layernorm.weight"]
    return {k: v.to(torch.bfloat16) for k, v in sd.items()}


SEL_CONFIG = dict(CONFIG, num_hidden_layers=3)
SEL = dict(full_cache_layers=[1], subset_cache_size=4, L=2, compression_ratio=1.0)
SEL_PROMPT, SEL_NEW = 20, 100


def main_selective(out_path):
    import helpers
    import plain_yi
    from delta_b200.weights import write_random_model
    import delta_b200.models  # noqa: F401
    from DELTA.Engine.DELTA import model as ref_model
    from DELTA.Engine.DELTA.backend import LMBackend
    from DELTA.Engine.DELTA.public_config import FINAL_PUBLIC_DELTA_BACKEND_CONFIG

    work = Path(tempfile.mkdtemp(prefix="golden_sel_"))
    c = SEL_CONFIG
    folder = write_random_model(work / "hf", c, SEED + 1, torch.float32)
    w = plain_yi.read_safetensors_plain(folder / "model.safetensors")
    name = NAME + "-selective"
    ref_model.transformer_configs[name] = dict(block_size=c["max_position_embeddings"], n_layer=c["num_hidden_layers"],
                                               n_head=c["num_attention_heads"], n_local_heads=c["num_key_value_heads"],
                                               dim=c["hidden_size"], intermediate_size=c["intermediate_size"],
                                               vocab_size=c["vocab_size"], rope_base=c["rope_theta"], norm_eps=c["rms_norm_eps"])
    (work / name).mkdir()
    torch.save(to_reference_names(w, c), str(work / name / "model.pth"))
    eng = LMBackend(dtype=torch.bfloat16, device="cuda:0", cuda_graph_decode=False, **dict(FINAL_PUBLIC_DELTA_BACKEND_CONFIG))
    eng.is_main_process = True
    eng.load_model(work / name / "model.pth", use_tp=False, rank_group=[0], group=None)
    cfg = eng.model.config                      # as tests/reasoni.py:327-335 sets them
    cfg.enable_selective_cache = True
    cfg.page_selector_version = FINAL_PUBLIC_DELTA_BACKEND_CONFIG["page_selector_version"]
    cfg.page_selector_v2 = True
    cfg.full_cache_layers = list(SEL["full_cache_layers"])
    cfg.subset_cache_ratio = 0.5
    cfg.compression_ratio = SEL["compression_ratio"]
    cfg.subset_cache_size = SEL["subset_cache_size"]
    cfg.L = SEL["L"]
    eng.setup_caches(max_batch_size=1, max_seq_length=MAX_LEN)
    steps = []
    eng.model.output.register_forward_hook(lambda mod, inp, out: steps.append(out.detach().float().cpu().reshape(-1, out.shape[-1])))
    prompt = torch.tensor(helpers.random_tokens(SEL_PROMPT, c["vocab_size"], 600))
    eng.add_requests([prompt], [SEL_PROMPT + SEL_NEW], [])
    eng.run_scheduler_loop()
    out = list(map(int, eng.scheduler.request_queue[0].output_ids))
    assert len(out) == SEL_NEW and steps[0].shape[0] == SEL_PROMPT and len(steps) == SEL_NEW
    logits = torch.cat([steps[0]] + [s[:1] for s in steps[1:]])
    assert logits.shape[0] == SEL_PROMPT + SEL_NEW - 1
    assert out == [int(logits[SEL_PROMPT - 1 + j].argmax()) for j in range(SEL_NEW)]
    golden = dict(config=c, seed=SEED + 1, weights_sha256=checksum(w), selective=SEL, page_size=16, prompt=prompt.tolist(),
                  output=out, logits=logits.to(torch.bfloat16),
                  made_with=dict(torch=str(torch.__version__), device=torch.cuda.get_device_name(0)))
    torch.save(golden, out_path)
    print(json.dumps(dict(written=str(out_path), output=out)))


def main(out_path):
    import helpers
    import plain_yi
    from delta_b200.weights import write_random_model
    import delta_b200.models  # noqa: F401
    from DELTA.Engine.DELTA import model as ref_model
    from DELTA.Engine.DELTA.backend import LMBackend
    from DELTA.Engine.DELTA.public_config import FINAL_PUBLIC_DELTA_BACKEND_CONFIG

    work = Path(tempfile.mkdtemp(prefix="golden_"))
    folder = write_random_model(work / "hf", CONFIG, SEED, torch.float32)
    w = plain_yi.read_safetensors_plain(folder / "model.safetensors")
    c = CONFIG
    ref_model.transformer_configs[NAME] = dict(block_size=c["max_position_embeddings"], n_layer=c["num_hidden_layers"],
                                               n_head=c["num_attention_heads"], n_local_heads=c["num_key_value_heads"],
                                               dim=c["hidden_size"], intermediate_size=c["intermediate_size"],
                                               vocab_size=c["vocab_size"], rope_base=c["rope_theta"], norm_eps=c["rms_norm_eps"])
    (work / NAME).mkdir()
    torch.save(to_reference_names(w, c), str(work / NAME / "model.pth"))

    eng = LMBackend(dtype=torch.bfloat16, device="cuda:0", cuda_graph_decode=False, **dict(FINAL_PUBLIC_DELTA_BACKEND_CONFIG))
    eng.is_main_process = True
    eng.load_model(work / NAME / "model.pth", use_tp=False, rank_group=[0], group=None)
    eng.model.config.enable_selective_cache = False
    eng.setup_caches(max_batch_size=len(PROMPT_LENS), max_seq_length=MAX_LEN)
    steps = []
    eng.model.output.register_forward_hook(lambda mod, inp, out: steps.append(out.detach().float().cpu().reshape(-1, out.shape[-1])))
    prompts = [torch.tensor(helpers.random_tokens(n, c["vocab_size"], 500 + i)) for i, n in enumerate(PROMPT_LENS)]
    eng.add_requests(prompts, [n + k for n, k in zip(PROMPT_LENS, NEW_TOKENS)], [])
    eng.run_scheduler_loop()
    outputs = [list(map(int, r.output_ids)) for r in eng.scheduler.request_queue]

    # rows of a step are the slots' tokens in slot order: the first step holds the whole prompts, every later one a token each
    logits = [[None] * (n + k - 1) for n, k in zip(PROMPT_LENS, NEW_TOKENS)]
    off = 0
    for i, n in enumerate(PROMPT_LENS):
        for p in range(n):
            logits[i][p] = steps[0][off + p]
        off += n
    assert off == steps[0].shape[0]
    for s, rows in enumerate(steps[1:], start=1):
        live = [i for i, (n, k) in enumerate(zip(PROMPT_LENS, NEW_TOKENS)) if s < k]
        assert rows.shape[0] == len(live), (s, rows.shape, live)
        for row, i in zip(rows, live):
            logits[i][PROMPT_LENS[i] + s - 1] = row
    for i, (n, k) in enumerate(zip(PROMPT_LENS, NEW_TOKENS)):
        assert len(outputs[i]) == k and all(x is not None for x in logits[i])
        assert outputs[i] == [int(logits[i][n - 1 + j].argmax()) for j in range(k)]
    golden = dict(config=CONFIG, seed=SEED, weights_sha256=checksum(w), prompts=[p.tolist() for p in prompts], outputs=outputs,
                  logits=[torch.stack(l).to(torch.bfloat16) for l in logits],
                  made_with=dict(torch=str(torch.__version__), device=torch.cuda.get_device_name(0)))
    torch.save(golden, out_path)
    print(json.dumps(dict(written=str(out_path), outputs=outputs)))


if __name__ == "__main__":
    if sys.argv[1] == "--selective":
        main_selective(sys.argv[2])
    else:
        main(sys.argv[1])
