"""Yi (Llama-layout dense decoder) as a ``ModelSpec``.

Every layer: RMSNorm, grouped-query attention with rotary positions, RMSNorm,
SwiGLU, in the pre-norm arrangement (reference: DELTA/Engine/DELTA/model.py:130-137,
330-341; the Yi sizes at model.py:87-88).  Tensor names are the ones of the model
folder (``model.layers.N.self_attn.q_proj.weight`` and so on); the reference's
own names (``layers.N.attention.wq.weight`` ...) belong to a converted
checkpoint whose converter it does not ship.

Options of the engine configuration that this builder reads: ``selective_cache`` (a
``SelectiveCacheConfig``: each layer gets its DELTA role from ``full_cache_layers``,
model.py:177-194) and ``rope_interleaved`` (the reference's pairing of rotary
positions, for converted checkpoints).  Older exports store ``rotary_emb.inv_freq``
buffers beside the weights; the loader is told that they may be there.
"""
from __future__ import annotations

from typing import Optional

from ..config.engine_config import EngineConfig
from ..config.selective_cache import SelectiveCacheConfig
from ..config.model_config import YiConfig
from ..parts.base import PartSpec, TensorSpec
from .spec import LayerSpec, ModelSpec, RunEntry


def yi_spec(cfg: YiConfig, engine: Optional[EngineConfig] = None) -> ModelSpec:
    engine = engine or EngineConfig()
    sel: Optional[SelectiveCacheConfig] = engine.option("selective_cache")
    d, hd = cfg.hidden_size, cfg.head_dim
    max_pos = max(cfg.max_position_embeddings, engine.max_seq_len)
    position = PartSpec("rotary", dict(head_dim=hd, theta=cfg.rope_theta, max_positions=max_pos,
                                       interleaved=bool(engine.option("rope_interleaved", False))), "position")
    layers = []
    for i in range(cfg.num_hidden_layers):
        pre = f"model.layers.{i}."
        window = cfg.window_of_layer(i)
        mixer = dict(prefix=pre + "self_attn.", width=d, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
                     head_dim=hd, position=position, window=window)
        if sel is not None and window is None:
            role = sel.role(i, cfg.num_hidden_layers)
            if role != "full":
                mixer.update(role=role, subset_cache_size=sel.subset_cache_size, keep_last=sel.keep_last,
                             compression_ratio=sel.compression_ratio, position_bias=sel.position_bias,
                             count_page_ahead=sel.count_page_ahead)
        layers.append(LayerSpec(dict(
            norm1=PartSpec("rms_norm", dict(name=pre + "input_layernorm.weight", width=d, eps=cfg.rms_norm_eps), "norm"),
            mixer=PartSpec("gqa_attention", mixer, "mixer"),
            norm2=PartSpec("rms_norm", dict(name=pre + "post_attention_layernorm.weight", width=d, eps=cfg.rms_norm_eps), "norm"),
            feed_forward=PartSpec("swiglu", dict(prefix=pre + "mlp.", width=d, intermediate=cfg.intermediate_size), "feed_forward"))))
    return ModelSpec(
        vocab_size=cfg.vocab_size, width=d, layers=tuple(layers),
        order=tuple(RunEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", dict(name="model.norm.weight", width=d, eps=cfg.rms_norm_eps), "norm"),
        embedding=TensorSpec("model.embed_tokens.weight", (cfg.vocab_size, d), kind="table"),
        lm_head=TensorSpec("lm_head.weight", (cfg.vocab_size, d), kind="matrix"),
        max_positions=max_pos, ignorable_tensors=("*.rotary_emb.inv_freq",))
