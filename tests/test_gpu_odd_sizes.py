"""Configurations with awkward sizes through the whole engine, in both precisions: head sizes in
steps of 16 (including 80, 112 and 256), numbers of heads and groups that are odd or prime, widths
and vocabularies that are no multiple of 8, one layer and five layers, a window with the head size of the
tensor-core kernels."""
import pytest
import torch

import helpers
from plain_yi import PlainYi
from test_gpu_model import compare

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["LlamaForCausalLM"], hidden_act="silu", tie_word_embeddings=False, model_type="llama")
ODD = {
    "hd80": dict(BASE, hidden_size=100, num_hidden_layers=1, num_attention_heads=5, num_key_value_heads=5, head_dim=80,
                 intermediate_size=130, vocab_size=1003, rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=256),
    "hd112": dict(BASE, hidden_size=224, num_hidden_layers=2, num_attention_heads=7, num_key_value_heads=1, head_dim=112,
                  intermediate_size=296, vocab_size=520, rope_theta=750000.0, rms_norm_eps=2e-5, max_position_embeddings=256),
    "hd256": dict(BASE, hidden_size=96, num_hidden_layers=1, num_attention_heads=3, num_key_value_heads=3, head_dim=256,
                  intermediate_size=64, vocab_size=301, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=256),
    "hd64g9": dict(BASE, hidden_size=144, num_hidden_layers=5, num_attention_heads=18, num_key_value_heads=2, head_dim=64,
                   intermediate_size=112, vocab_size=777, rope_theta=5000000.0, rms_norm_eps=1e-5, max_position_embeddings=256),
    # head size 64 with a window in every second layer: the tensor-core attention kernels mask by window,
    # and the windowed group gives pages back while the requests run
    "hd64win": dict(BASE, hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                    intermediate_size=144, vocab_size=600, rope_theta=1000000.0, rms_norm_eps=1e-5, max_position_embeddings=256,
                    sliding_window=40, layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"]),
    "hd128g3": dict(BASE, hidden_size=160, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=128,
                    intermediate_size=208, vocab_size=1000, rope_theta=5000000.0, rms_norm_eps=1e-5, max_position_embeddings=256),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ODD))
def test_odd_sizes(tmp_path, name, dtype):
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    from delta_b200.weights import write_random_model
    folder = write_random_model(tmp_path / name, ODD[name], seed=11, dtype=torch.float32)
    plain = PlainYi(folder, rounding="bfloat16" if dtype == "bfloat16" else None)
    lengths = [3, 41, 70, 130]
    toks = [helpers.random_tokens(n, plain.cfg.vocab, 300 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(t) for t in toks]
    r = ModelRunner(folder, engine_config=EngineConfig(max_batch=4, max_seq_len=192, page_size=16, num_pages=48, dtype=dtype))
    res = helpers.run_schedule(r, toks, helpers.last_one_by_one(lengths, tail=20))
    compare(res, refs, lengths, dtype, f"{name}: last 20 one by one")
    steps, ends = helpers.mixed(lengths, [n // 2 for n in lengths], seed=8)
    res = helpers.run_schedule(r, toks, steps, ends)
    compare(res, refs, lengths, dtype, f"{name}: mixed")
