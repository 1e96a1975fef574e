"""Configuration, registry and weight loading (no GPU)."""
import json

import pytest
import torch

import helpers
import delta_b200.models  # noqa: F401
from delta_b200.config import ConfigError, EngineConfig, SelectiveCacheConfig, YiConfig, read_config
from delta_b200.models import Model, yi_spec
from delta_b200.weights import WeightError, load_tensors, write_random_model, write_safetensors, SafetensorsFile
from plain_yi import read_safetensors_plain


def test_config_reads_every_size_from_config_json():
    for which in "ABC":
        c = helpers.tiny_config(which)
        cfg = YiConfig.from_dict(c)
        assert cfg.hidden_size == c["hidden_size"] and cfg.num_hidden_layers == c["num_hidden_layers"]
        assert cfg.num_key_value_heads == c["num_key_value_heads"] and cfg.vocab_size == c["vocab_size"]
        assert cfg.rms_norm_eps == c["rms_norm_eps"] and cfg.rope_theta == c["rope_theta"]
        assert cfg.head_dim == c.get("head_dim", c["hidden_size"] // c["num_attention_heads"])
    assert YiConfig.from_dict(helpers.tiny_config("C")).window_of_layer(1) == 24
    assert YiConfig.from_dict(helpers.tiny_config("C")).window_of_layer(0) is None


@pytest.mark.parametrize("change, text", [
    (dict(tie_word_embeddings=True), "tie_word_embeddings"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "bias"),
    (dict(rope_scaling={"type": "linear", "factor": 2}), "rope_scaling"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(architectures=["NoSuchModel"]), "unknown architecture"),
    (dict(layer_types=["sliding_attention", "full_attention"]), "sliding_window"),
])
def test_config_errors(tmp_path, change, text):
    c = dict(helpers.tiny_config("A"), **change)
    (tmp_path / "config.json").write_text(json.dumps(c))
    with pytest.raises(ConfigError, match=text):
        read_config(tmp_path)


def test_missing_key_is_named():
    c = helpers.tiny_config("A")
    del c["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        YiConfig.from_dict(c)


def test_selective_roles():
    s = SelectiveCacheConfig(full_cache_layers=(2, 0, 1, 5), subset_cache_size=4, L=8)
    assert s.full_cache_layers == (0, 1, 2, 5) and s.keep_last == 4
    assert [s.role(i, 8) for i in range(8)] == ["full", "full", "planner", "subset", "subset", "planner", "subset", "subset"]
    assert SelectiveCacheConfig(full_cache_layers=(7,), subset_cache_size=2).role(7, 8) == "full"  # the last layer
    assert SelectiveCacheConfig().role(3, 8) == "full"
    with pytest.raises(ValueError):
        SelectiveCacheConfig(full_cache_layers=(0,), subset_cache_size=0)


def test_random_model_folder_round_trip(tmp_path):
    folder = helpers.make_model_folder(tmp_path, "B", torch.bfloat16)
    assert (folder / "config.json").is_file() and (folder / "model.safetensors").is_file()
    arch, cfg = read_config(folder)
    model = Model(arch.build_spec(cfg, None))
    t = load_tensors(folder, model.tensor_specs(), torch.bfloat16, "cpu")
    assert t["model.layers.2.mlp.down_proj.weight"].shape == (128, 344)
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    # the same seed gives the same folder; another seed another one
    again = write_random_model(tmp_path / "again", helpers.tiny_config("B"), helpers.SEED["B"], torch.bfloat16)
    other = write_random_model(tmp_path / "other", helpers.tiny_config("B"), 99, torch.bfloat16)
    a = read_safetensors_plain(folder / "model.safetensors")
    b = read_safetensors_plain(again / "model.safetensors")
    c = read_safetensors_plain(other / "model.safetensors")
    assert all(torch.equal(a[k], b[k]) for k in a) and not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    # the engine's reader and the plain reader agree
    f = SafetensorsFile(folder / "model.safetensors")
    assert torch.equal(f.tensor("lm_head.weight").float(), a["lm_head.weight"])
    # norm weights 1 + U(-0.1, 0.1), matrices N(0, 0.02)
    nw = a["model.norm.weight"]
    assert 0.89 < nw.min() and nw.max() < 1.11
    assert abs(a["lm_head.weight"].std().item() - 0.02) < 2e-3


def test_dtype_policy(tmp_path):
    folder = helpers.make_model_folder(tmp_path, "A", torch.float32)
    arch, cfg = read_config(folder)
    specs = Model(arch.build_spec(cfg, None)).tensor_specs()
    t = load_tensors(folder, specs, torch.bfloat16, "cpu")
    # operands of products are kept in bfloat16; a vector stored in 32 bit stays in 32 bit
    assert t["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert t["model.norm.weight"].dtype == torch.float32
    t32 = load_tensors(folder, specs, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = helpers.make_model_folder(tmp_path, "A", torch.float32)
    tensors = read_safetensors_plain(folder / "model.safetensors")
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["lm_head.weight"] = torch.zeros(511, 64)
    write_safetensors(folder / "model.safetensors", tensors)
    arch, cfg = read_config(folder)
    specs = Model(arch.build_spec(cfg, None)).tensor_specs()
    with pytest.raises(WeightError) as e:
        load_tensors(folder, specs, torch.float32, "cpu")
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "rotary_emb.inv_freq" in msg
    assert "lm_head.weight is [511, 64], expected [512, 64]" in msg
    assert e.value.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"] or set(e.value.missing) == {
        "model.layers.1.mlp.up_proj.weight", "model.norm.weight"}


def test_names_the_architecture_calls_ignorable_may_be_in_the_folder(tmp_path):
    """Older exports store ``rotary_emb.inv_freq`` buffers beside the weights: the Yi specification
    names them ignorable, so such a folder loads; any other name nobody asked for is still an error."""
    folder = helpers.make_model_folder(tmp_path, "A", torch.float32)
    tensors = read_safetensors_plain(folder / "model.safetensors")
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    write_safetensors(folder / "model.safetensors", tensors)
    arch, cfg = read_config(folder)
    spec = arch.build_spec(cfg, None)
    specs = Model(spec).tensor_specs()
    assert spec.ignorable_tensors
    t = load_tensors(folder, specs, torch.float32, "cpu", ignorable=spec.ignorable_tensors)
    assert "model.layers.0.self_attn.rotary_emb.inv_freq" not in t and len(t) == len(specs)
    tensors["model.layers.0.self_attn.something_else"] = torch.zeros(8)
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_tensors(folder, specs, torch.float32, "cpu", ignorable=spec.ignorable_tensors)
    assert e.value.unexpected == ["model.layers.0.self_attn.something_else"]


def test_engine_config_checks():
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(page_size=24)
    assert EngineConfig(max_batch=3, max_seq_len=100, page_size=16).pool_pages == 21


def test_spec_follows_config_layer_by_layer():
    cfg = YiConfig.from_dict(helpers.tiny_config("C"))
    sel = SelectiveCacheConfig(full_cache_layers=(0,), subset_cache_size=3)
    spec = yi_spec(cfg, EngineConfig(options=dict(selective_cache=sel)))
    roles = [l.parts["mixer"].params.get("role", "full") for l in spec.layers]
    windows = [l.parts["mixer"].params["window"] for l in spec.layers]
    assert windows == [None, 24, None, 24]
    assert roles == ["planner", "full", "subset", "full"]   # windowed layers take no page selection
    m = Model(spec)
    groups = {}
    for cid, cs in m.cache_specs().items():
        groups.setdefault(cs, []).append(cid)
    assert sorted(groups.values()) == [[0, 2], [1, 3]]


def test_the_page_counted_ahead_needs_two_places():
    from delta_b200.config import SelectiveCacheConfig
    SelectiveCacheConfig(full_cache_layers=(0,), subset_cache_size=2, L=2, count_page_ahead=True)
    for k, L in ((1, 2), (4, 1)):
        with pytest.raises(ValueError, match="count_page_ahead"):
            SelectiveCacheConfig(full_cache_layers=(0,), subset_cache_size=k, L=L, count_page_ahead=True)
