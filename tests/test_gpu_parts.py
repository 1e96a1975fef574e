"""Each part of a layer alone against the plain functions, and toy parts that are defined
here: a mixer with state of its own, a mixer whose cache holds one vector per token, a
feed-forward with routing, another position encoding, a block with a norm more than the
pre-norm block has, a run order that names a layer twice and lets a run read another run's
cache.  The toy parts are registered, built from a config.json and stepped without a change
to the package."""
import json
import math
from dataclasses import dataclass

import pytest
import torch

import helpers
import plain_yi as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runner_for(folder, which, dtype="float32", **kw):
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    return ModelRunner(folder, engine_config=EngineConfig(max_batch=4, max_seq_len=128, page_size=helpers.PAGE_SIZE[which],
                                                          dtype=dtype, **kw))


# ---------------------------------------------------------------- parts of the engine, alone

@pytest.mark.parametrize("which", ["A", "C"])
def test_norm_feed_forward_mixer_and_block_alone(model_folders, which):
    """A real step context, then one part at a time on inputs of our own."""
    from delta_b200.engine.step import RowInput
    folder = model_folders[which]
    plain = P.PlainYi(folder)
    c, w = plain.cfg, plain.w
    r = runner_for(folder, which)
    lens = [19, 40]
    slots = [r.cache.acquire_slot() for _ in lens]
    rows = [RowInput(s, [1] * n, 0, []) for s, n in zip(slots, lens)]
    for row in rows:
        r.cache.grow(row.slot, len(row.tokens))
    ctx = r.build_context(rows)
    T = sum(lens)
    torch.manual_seed(0)
    x = torch.randn(T, c.hidden, device=DEV)
    add = torch.randn(T, c.hidden, device=DEV) * 0.1
    layer = 1                      # in C this is a layer with a window
    block = r.model.blocks[layer]
    pre = f"model.layers.{layer}."

    # norm, with the fused residual add and with a row choice
    xs = x.clone()
    got = block.norm1.forward(ctx, xs, add=add)
    want = P.rms_norm((x + add).cpu(), w[pre + "input_layernorm.weight"], c.eps)
    assert torch.allclose(xs, x + add) and torch.allclose(got.cpu(), want, atol=1e-5, rtol=1e-5)
    pick = torch.tensor([3, 0, T - 1], dtype=torch.int32, device=DEV)
    got = block.norm2.forward(ctx, x.clone(), rows=pick)
    want = P.rms_norm(x.cpu()[[3, 0, T - 1]], w[pre + "post_attention_layernorm.weight"], c.eps)
    assert torch.allclose(got.cpu(), want, atol=1e-5, rtol=1e-5)

    # feed-forward
    got = block.feed_forward.forward(ctx, x)
    want = P.swiglu(x.cpu(), w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"], w[pre + "mlp.down_proj.weight"])
    assert torch.allclose(got.cpu(), want, atol=2e-5, rtol=1e-4)

    # mixer: projections, rotary positions, append, attention (with the layer's window), output projection
    got = block.mixer.forward(ctx, x.clone(), ctx.cache_view(layer, True)).cpu()
    off = 0
    for n in lens:
        a = x.cpu()[off:off + n]
        pos = torch.arange(n)
        q = (a @ w[pre + "self_attn.q_proj.weight"].T).view(n, c.heads, c.head_dim)
        k = (a @ w[pre + "self_attn.k_proj.weight"].T).view(n, c.kv_heads, c.head_dim)
        v = (a @ w[pre + "self_attn.v_proj.weight"].T).view(n, c.kv_heads, c.head_dim)
        y, _ = P.attention(P.rope(q, pos, c.theta, False), P.rope(k, pos, c.theta, False), v, P.causal_mask(n, c.windows[layer]))
        want = y.reshape(n, -1) @ w[pre + "self_attn.o_proj.weight"].T
        assert torch.allclose(got[off:off + n], want, atol=2e-5, rtol=1e-4)
        off += n

    # the block: stream and pending update in, stream and pending update out
    xs = x.clone()
    out_x, pending = block.forward(ctx, xs, add.clone(), ctx.cache_view(layer, True))
    off = 0
    for n in lens:
        full, _, _ = plain.layer(layer, (x + add).cpu()[off:off + n], torch.arange(n), P.causal_mask(n, c.windows[layer]))
        assert torch.allclose((out_x + pending).cpu()[off:off + n], full, atol=3e-5, rtol=1e-4)
        off += n


def test_rotary_table_and_both_pairings():
    from delta_b200.parts.rope import RotaryPositions
    for theta, hd in ((10000.0, 16), (5000000.0, 128), (250000.0, 48)):
        t = RotaryPositions(hd, theta, 300).table_cpu()
        pos = torch.tensor([0, 1, 17, 299])
        x = torch.randn(4, 2, hd)
        for inter in (False, True):
            want = P.rope(x, pos, theta, inter)
            c, s = t[pos, :, 0][:, None, :], t[pos, :, 1][:, None, :]
            if inter:
                a, b = x[..., 0::2], x[..., 1::2]
                got = torch.empty_like(x)
                got[..., 0::2], got[..., 1::2] = a * c - b * s, a * s + b * c
            else:
                a, b = x[..., :hd // 2], x[..., hd // 2:]
                got = torch.cat([a * c - b * s, a * s + b * c], -1)
            assert torch.allclose(got, want, atol=1e-6)


# ---------------------------------------------------------------- toy parts, defined here

def register_toys():
    from delta_b200.config.registry import register_architecture
    from delta_b200.models.spec import LayerSpec, ModelSpec, RunEntry
    from delta_b200.parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, PAGE, POSITION_ENCODINGS, Block, CacheSpec, FeedForward,
                                       Mixer, PartSpec, PositionEncoding, StateSpec, TensorSpec)

    if "toy_running_mean" not in MIXERS:
        @MIXERS.register("toy_running_mean")
        class RunningMean(Mixer):
            """s <- a * s + x_t per request, y_t = s Wo^T: no cache, a state vector per request."""

            def __init__(self, prefix, width):
                self.prefix, self.width = prefix, width

            def tensor_specs(self):
                return [TensorSpec(self.prefix + "decay", (self.width,), kind="vector", init="norm"),
                        TensorSpec(self.prefix + "out.weight", (self.width, self.width))]

            def bind(self, tensors):
                self.decay = tensors[self.prefix + "decay"].float() * 0.5
                self.w_out = tensors[self.prefix + "out.weight"]

            def state_specs(self):
                return {self.prefix + "state": StateSpec((self.width,), torch.float32, 0.0)}

            def forward(self, ctx, x, cache):
                assert cache is None
                state = ctx.state(self.prefix + "state")
                ys = torch.empty_like(x, dtype=torch.float32)
                for row, q0, n in zip(ctx.host["rows"], ctx.host["q_start"], ctx.host["q_lens"]):
                    s = state[row.slot].clone()
                    for i in range(n):
                        s = self.decay * s + x[q0 + i].float()
                        ys[q0 + i] = s
                    state[row.slot] = s
                return (ys @ self.w_out.float().T).to(x.dtype)

    if "toy_latent_memory" not in MIXERS:
        @MIXERS.register("toy_latent_memory")
        class LatentMemory(Mixer):
            """Keeps one latent vector per token in its pages, c_t = x_t Wc^T, and gives
            y_t = mean(c_0 .. c_t) Wo^T.  Its page layout has no heads and no key/value pair."""

            def __init__(self, prefix, width, latent):
                self.prefix, self.width, self.latent = prefix, width, latent

            def tensor_specs(self):
                return [TensorSpec(self.prefix + "down.weight", (self.latent, self.width)),
                        TensorSpec(self.prefix + "up.weight", (self.width, self.latent))]

            def bind(self, tensors):
                self.w_down, self.w_up = tensors[self.prefix + "down.weight"], tensors[self.prefix + "up.weight"]

            def cache_spec(self):
                return CacheSpec((PAGE, self.latent))

            def forward(self, ctx, x, cache):
                assert tuple(cache.pages.shape[1:]) == (cache.page_size, self.latent)
                c = x.float() @ self.w_down.float().T
                ys = torch.empty((x.shape[0], self.latent), dtype=torch.float32, device=x.device)
                ps = cache.page_size
                for b, (row, q0, n) in enumerate(zip(ctx.host["rows"], ctx.host["q_start"], ctx.host["q_lens"])):
                    table = cache.block_table[b]
                    for i in range(n):
                        pos = row.start_pos + i
                        cache.pages[table[pos // ps], pos % ps] = c[q0 + i].to(cache.pages.dtype)
                    held = torch.cat([cache.pages[table[j]] for j in range((row.start_pos + n + ps - 1) // ps)]).float()
                    sums = held[:row.start_pos + n].cumsum(0)
                    for i in range(n):
                        pos = row.start_pos + i
                        ys[q0 + i] = sums[pos] / (pos + 1)
                return (ys @ self.w_up.float().T).to(x.dtype)

    if "toy_sandwich" not in BLOCKS:
        @BLOCKS.register("toy_sandwich")
        class Sandwich(Block):
            """h = x + post_norm(mixer(norm1(x))); out = h + feed_forward(norm2(h)): one norm more
            than the pre-norm block."""
            roles = ("norm1", "mixer", "post_norm", "norm2", "feed_forward")

            def forward(self, ctx, x, pending, cache):
                a = self.norm1.forward(ctx, x, add=pending)
                y = self.post_norm.forward(ctx, self.mixer.forward(ctx, a, cache))
                f = self.norm2.forward(ctx, x, add=y)
                return x, self.feed_forward.forward(ctx, f)

    if "toy_routed" not in FEED_FORWARDS:
        @FEED_FORWARDS.register("toy_routed")
        class Routed(FeedForward):
            """Top-1 of E experts per token, each a two-matrix GELU block."""

            def __init__(self, prefix, width, intermediate, experts):
                self.prefix, self.width, self.inter, self.experts = prefix, width, intermediate, experts

            def tensor_specs(self):
                specs = [TensorSpec(self.prefix + "router.weight", (self.experts, self.width))]
                for e in range(self.experts):
                    specs += [TensorSpec(f"{self.prefix}experts.{e}.up.weight", (self.inter, self.width)),
                              TensorSpec(f"{self.prefix}experts.{e}.down.weight", (self.width, self.inter))]
                return specs

            def bind(self, tensors):
                self.t = {k: v for k, v in tensors.items() if k.startswith(self.prefix)}

            def forward(self, ctx, x):
                logits = x.float() @ self.t[self.prefix + "router.weight"].float().T
                pick = logits.argmax(-1)
                out = torch.zeros_like(x, dtype=torch.float32)
                for e in range(self.experts):
                    m = pick == e
                    h = torch.nn.functional.gelu(x[m].float() @ self.t[f"{self.prefix}experts.{e}.up.weight"].float().T)
                    out[m] = h @ self.t[f"{self.prefix}experts.{e}.down.weight"].float().T
                return out.to(x.dtype)

    if "toy_partial_rotary" not in POSITION_ENCODINGS:
        @POSITION_ENCODINGS.register("toy_partial_rotary")
        class PartialRotary(PositionEncoding):
            """Rotates only the first half of the pairs; the others keep angle zero."""
            interleaved = False

            def __init__(self, head_dim, theta, max_positions):
                self.head_dim, self.theta, self.max_positions = head_dim, theta, max_positions
                self._t = None

            def table_cpu(self):
                half = self.head_dim // 2
                j = torch.arange(half, dtype=torch.float64)
                inv = self.theta ** (-2.0 * j / self.head_dim)
                inv[half // 2:] = 0.0
                ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None]
                return torch.stack([torch.cos(ang), torch.sin(ang)], -1).float().contiguous()

            def table(self, device):
                if self._t is None:
                    self._t = self.table_cpu().to(device)
                return self._t

    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int
        heads: int
        kv_heads: int
        head_dim: int
        intermediate_size: int
        vocab_size: int
        eps: float
        theta: float
        experts: int
        max_position_embeddings: int
        latent: int

        @staticmethod
        def from_dict(c):
            return ToyConfig(c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                             c["intermediate_size"], c["vocab_size"], c["rms_norm_eps"], c["rope_theta"], c["experts"],
                             c["max_position_embeddings"], c["latent"])

    def toy_spec(cfg, engine):
        d = cfg.hidden_size

        def norm(name):
            return PartSpec("rms_norm", dict(name=name, width=d, eps=cfg.eps), "norm")
        pos = PartSpec("toy_partial_rotary", dict(head_dim=cfg.head_dim, theta=cfg.theta, max_positions=cfg.max_position_embeddings),
                       "position")
        l0 = LayerSpec(dict(norm1=norm("toy.0.n1"),
                            mixer=PartSpec("gqa_attention", dict(prefix="toy.0.attn.", width=d, heads=cfg.heads, kv_heads=cfg.kv_heads,
                                                                 head_dim=cfg.head_dim, position=pos), "mixer"),
                            norm2=norm("toy.0.n2"),
                            feed_forward=PartSpec("swiglu", dict(prefix="toy.0.mlp.", width=d, intermediate=cfg.intermediate_size),
                                                  "feed_forward")))
        l1 = LayerSpec(dict(norm1=norm("toy.1.n1"), mixer=PartSpec("toy_running_mean", dict(prefix="toy.1.mean.", width=d), "mixer"),
                            norm2=norm("toy.1.n2"),
                            feed_forward=PartSpec("toy_routed", dict(prefix="toy.1.ff.", width=d, intermediate=cfg.intermediate_size,
                                                                     experts=cfg.experts), "feed_forward")))
        l2 = LayerSpec(dict(norm1=norm("toy.2.n1"),
                            mixer=PartSpec("toy_latent_memory", dict(prefix="toy.2.mem.", width=d, latent=cfg.latent), "mixer"),
                            post_norm=norm("toy.2.post"), norm2=norm("toy.2.n2"),
                            feed_forward=PartSpec("swiglu", dict(prefix="toy.2.mlp.", width=d, intermediate=cfg.intermediate_size),
                                                  "feed_forward")), block="toy_sandwich")
        # layer 0 runs three times: with its own cache, again with another cache, and reading the first run's cache
        order = (RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(0, cache=0, writes_cache=False), RunEntry(2))
        return ModelSpec(vocab_size=cfg.vocab_size, width=d, layers=(l0, l1, l2), order=order, final_norm=norm("toy.norm"),
                         embedding=TensorSpec("toy.embed", (cfg.vocab_size, d), kind="table"),
                         lm_head=TensorSpec("toy.head", (cfg.vocab_size, d)), max_positions=cfg.max_position_embeddings)

    register_architecture("ToyForCausalLM", ToyConfig.from_dict, toy_spec)


TOY = dict(architectures=["ToyForCausalLM"], hidden_size=48, num_attention_heads=3, num_key_value_heads=1, head_dim=16,
           intermediate_size=80, vocab_size=100, rms_norm_eps=1e-5, rope_theta=10000.0, experts=3,
           max_position_embeddings=128, latent=24)


def toy_plain(folder, tokens):
    """Whole-sequence float32 forward of the toy model, written from its definition above."""
    w = P.read_safetensors_plain(folder / "model.safetensors")
    w = {k: v.float() for k, v in w.items()}
    c = TOY
    T, hd, H, KV = len(tokens), c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"]
    half = hd // 2
    j = torch.arange(half, dtype=torch.float64)
    inv = c["rope_theta"] ** (-2.0 * j / hd)
    inv[half // 2:] = 0.0
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = torch.cos(ang).float()[:, None, :], torch.sin(ang).float()[:, None, :]

    def rot(t):
        a, b = t[..., :half], t[..., half:]
        return torch.cat([a * cos - b * sin, a * sin + b * cos], -1)

    def attn_layer(x, kv_from=None):
        a = P.rms_norm(x, w["toy.0.n1"], c["rms_norm_eps"])
        q = rot((a @ w["toy.0.attn.q_proj.weight"].T).view(T, H, hd))
        k = rot((a @ w["toy.0.attn.k_proj.weight"].T).view(T, KV, hd))
        v = (a @ w["toy.0.attn.v_proj.weight"].T).view(T, KV, hd)
        if kv_from is not None:
            k, v = kv_from
        y, _ = P.attention(q, k, v, P.causal_mask(T))
        h = x + y.reshape(T, -1) @ w["toy.0.attn.o_proj.weight"].T
        f = P.rms_norm(h, w["toy.0.n2"], c["rms_norm_eps"])
        return h + P.swiglu(f, w["toy.0.mlp.gate_proj.weight"], w["toy.0.mlp.up_proj.weight"], w["toy.0.mlp.down_proj.weight"]), (k, v)

    def mean_layer(x):
        a = P.rms_norm(x, w["toy.1.n1"], c["rms_norm_eps"])
        s = torch.zeros(c["hidden_size"])
        ys = []
        for t in range(T):
            s = w["toy.1.mean.decay"] * 0.5 * s + a[t]
            ys.append(s)
        h = x + torch.stack(ys) @ w["toy.1.mean.out.weight"].T
        f = P.rms_norm(h, w["toy.1.n2"], c["rms_norm_eps"])
        pick = (f @ w["toy.1.ff.router.weight"].T).argmax(-1)
        out = torch.zeros_like(f)
        for e in range(c["experts"]):
            m = pick == e
            out[m] = torch.nn.functional.gelu(f[m] @ w[f"toy.1.ff.experts.{e}.up.weight"].T) @ w[f"toy.1.ff.experts.{e}.down.weight"].T
        return h + out

    def memory_layer(x):
        a = P.rms_norm(x, w["toy.2.n1"], c["rms_norm_eps"])
        lat = a @ w["toy.2.mem.down.weight"].T
        means = lat.cumsum(0) / torch.arange(1, T + 1)[:, None]
        h = x + P.rms_norm(means @ w["toy.2.mem.up.weight"].T, w["toy.2.post"], c["rms_norm_eps"])
        f = P.rms_norm(h, w["toy.2.n2"], c["rms_norm_eps"])
        return h + P.swiglu(f, w["toy.2.mlp.gate_proj.weight"], w["toy.2.mlp.up_proj.weight"], w["toy.2.mlp.down_proj.weight"])

    x = w["toy.embed"][torch.tensor(tokens)]
    x, kv0 = attn_layer(x)
    x = mean_layer(x)
    x, _ = attn_layer(x)
    x, _ = attn_layer(x, kv_from=kv0)
    x = memory_layer(x)
    return P.rms_norm(x, w["toy.norm"], c["rms_norm_eps"]) @ w["toy.head"].T


def test_toy_parts_are_registered_built_and_stepped(tmp_path):
    """A mixer with state of its own, one whose pages hold a latent vector per token, a routed
    feed-forward, another position encoding, a block with an extra norm and a run order with a
    repeated layer and a shared cache: built from a model folder and stepped whole, token by
    token, in portions and mixed, with the same logits every time."""
    from delta_b200.config import EngineConfig
    from delta_b200.config.registry import unregister_architecture
    from delta_b200.engine.step import ModelRunner
    from delta_b200.weights import write_random_model
    register_toys()
    try:
        folder = write_random_model(tmp_path / "toy", TOY, seed=5, dtype=torch.float32)
        lengths = [33, 7, 50, 21]
        toks = [helpers.random_tokens(n, TOY["vocab_size"], 200 + i) for i, n in enumerate(lengths)]
        refs = [toy_plain(folder, t) for t in toks]
        r = ModelRunner(folder, engine_config=EngineConfig(max_batch=4, max_seq_len=64, page_size=8, num_pages=40, dtype="float32"))
        assert set(r.cache.groups) == {"2x1xPx16", "Px24"} and r.cache.groups["2x1xPx16"].cache_ids == [0, 2]
        assert r.cache.groups["Px24"].cache_ids == [4] and r.cache.groups["Px24"].pages.shape == (1, 40 + 1, 8, 24)
        assert [type(b).__name__ for b in r.model.blocks] == ["PreNormBlock", "PreNormBlock", "Sandwich"]
        assert r.cache.states["toy.1.mean.state"].shape == (4 + 1, 48)     # four requests and the padding slot
        prompt_lens = [n // 2 for n in lengths]
        mixed, ends = helpers.mixed(lengths, prompt_lens, seed=2)
        for what, steps, e in (("whole", helpers.whole(lengths), None), ("one by one", helpers.last_one_by_one(lengths), None),
                               ("portions", helpers.changing_portions(lengths), None), ("mixed", mixed, ends)):
            res = helpers.run_schedule(r, toks, steps, e)
            for i, n in enumerate(lengths):
                got = helpers.stack_positions(res, i, n)
                assert torch.allclose(got, refs[i], atol=5e-5, rtol=2e-4), f"{what}: request {i}"
    finally:
        unregister_architecture("ToyForCausalLM")
