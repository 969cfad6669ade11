"""The parts of a layer, each alone against its plain formula, and the ways they are put
together: different mixers in different layers, a run order that names a layer twice and
lets a layer read another layer's cache, and a toy mixer with state of its own that is
defined here, registered, built, loaded and stepped without touching the package; likewise a
feed-forward with routing, other position encodings (one with two axes), a mixer that caches
keys and values of different widths, and an architecture with an embedding multiplier, capped
logits and an ignored buffer (GPU)."""
import json
import math
import os
import random
from dataclasses import dataclass

import pytest
import torch

import helpers
from helpers import TINY, TOL
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def _runner(model, page=4, pages=64, max_requests=4):
    from pulsar_b200.cache import CacheManager
    from pulsar_b200.engine.runner import ModelRunner
    cache = CacheManager(model.cache_needs(), page, pages, max_requests, model.dtype, "cuda:0")
    return ModelRunner(model, cache, "cuda:0")


def _tiny_model(tmp_path, name, dtype):
    from pulsar_b200.engine import load_model
    raw, seed, page = TINY[name]
    folder = helpers.make_folder(tmp_path, raw, seed)
    cfg, weights = helpers.read_folder(folder)
    _, model = load_model(folder, dtype, "cuda:0")
    return cfg, weights, model


def _close(got, ref, tol):
    err = helpers.rel_err(got.detach().float().cpu(), ref)
    assert err < tol, f"relative error {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_each_part_alone(tmp_path, name, dtype):
    from pulsar_b200.engine.runner import StepEntry
    cfg, weights, model = _tiny_model(tmp_path, name, dtype)
    tdt = model.dtype
    w = {k: v.double() for k, v in (helpers.as_bf16_matrices(weights) if dtype == "bfloat16" else weights).items()}
    runner = _runner(model)
    rng = random.Random(0)
    n = 21
    tokens = helpers.random_tokens(rng, n, cfg["vocab_size"])
    ctx = runner.prepare([StepEntry("a", tokens, [n - 1])])
    g = torch.Generator().manual_seed(3)
    d = cfg["hidden_size"]
    h = torch.randn(n, d, generator=g)
    h_dev = h.to(tdt).cuda()
    hd = h_dev.double().cpu()                      # what the part really saw
    layer = cfg["num_hidden_layers"] - 1           # in C this layer has a window
    blk = model.blocks[layer]
    p = f"model.layers.{layer}."
    tol = TOL[dtype]

    # norm (with the residual add it is fused with)
    res = torch.randn(n, d, generator=g)
    res_dev = res.cuda()
    out = blk.mixer_norm.forward(ctx, res_dev, h_dev)
    x = res.double() + hd
    _close(out, plain.rmsnorm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"]), tol)
    _close(res_dev, x, 1e-6)

    # position encoding
    cos, sin = blk.mixer.position.tables(ctx)
    ang = plain.rope_angles(torch.arange(n), cfg["head_dim"], cfg["rope_theta"])
    assert float((cos.cpu().double() - torch.cos(ang)).abs().max()) < 1e-6
    assert float((sin.cpu().double() - torch.sin(ang)).abs().max()) < 1e-6

    # mixer
    out = blk.mixer.forward(ctx, h_dev, ctx.cache(layer))
    ref = plain.attention_block(hd, torch.arange(n), w, p + "self_attn.", cfg, layer)
    _close(out, ref, tol)

    # feed-forward
    out = blk.feed_forward.forward(ctx, h_dev)
    ref = plain.swiglu_mlp(hd, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    _close(out, ref, tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_arrangement(tmp_path, dtype):
    from pulsar_b200.engine.runner import StepEntry
    cfg, weights, model = _tiny_model(tmp_path, "B", dtype)
    w = {k: v.double() for k, v in (helpers.as_bf16_matrices(weights) if dtype == "bfloat16" else weights).items()}
    runner = _runner(model)
    n = 13
    ctx = runner.prepare([StepEntry("a", list(range(n)), [])])
    g = torch.Generator().manual_seed(4)
    x = torch.randn(n, cfg["hidden_size"], generator=g)
    res = x.clone().cuda()
    delta = model.blocks[1].forward(ctx, res, None, ctx.cache(1))
    ref = plain.block(x.double(), torch.arange(n), w, 1, cfg)
    _close(res.double().cpu() + delta.double().cpu(), ref, TOL[dtype])


# ------------------------------------------------------------------ run order as data
def _shared_cache_spec(raw):
    """Three calls over two blocks: block 0, block 1 (no k/v of its own, reads block 0's
    cache entry), block 0 again on a second cache entry."""
    import dataclasses
    from pulsar_b200.config import LayerCall, config_from_dict
    spec = config_from_dict(dict(raw, num_hidden_layers=2)).model_spec()
    b0, b1 = spec.blocks
    b1 = dataclasses.replace(b1, mixer=dataclasses.replace(b1.mixer, own_kv=False))
    return dataclasses.replace(spec, blocks=(b0, b1), run_order=(LayerCall(0, 0), LayerCall(1, 0), LayerCall(0, 1)))


def _plain_shared(cfg, w, tokens):
    t = len(tokens)
    pos = torch.arange(t)
    hq, hkv, d, eps, theta = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                              cfg["rms_norm_eps"], cfg["rope_theta"])
    x = plain.embedding(torch.tensor(tokens), w["model.embed_tokens.weight"])
    kept = {}

    def layer(x, i, share_from=None):
        p = f"model.layers.{i}."
        h = plain.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        q = plain.rope(plain.rmsnorm((h @ w[p + "self_attn.q_proj.weight"].T).view(t, hq, d), w[p + "self_attn.q_norm.weight"], eps), pos, theta)
        if share_from is None:
            k = plain.rope(plain.rmsnorm((h @ w[p + "self_attn.k_proj.weight"].T).view(t, hkv, d), w[p + "self_attn.k_norm.weight"], eps), pos, theta)
            v = (h @ w[p + "self_attn.v_proj.weight"].T).view(t, hkv, d)
            kept[i] = (k, v)
        else:
            k, v = kept[share_from]
        o = plain.attention(q, k, v, 1 / math.sqrt(d))
        x = x + o.reshape(t, hq * d) @ w[p + "self_attn.o_proj.weight"].T
        h2 = plain.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        return x + plain.swiglu_mlp(h2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x = layer(x, 0)
    x = layer(x, 1, share_from=0)
    x = layer(x, 0)
    return plain.head(x, w, cfg)


def test_run_order_names_a_layer_twice_and_shares_a_cache(tmp_path):
    from pulsar_b200.engine.runner import StepEntry
    from pulsar_b200.models.decoder import DecoderModel
    from pulsar_b200.weights import load_weights, random_tensors, write_safetensors
    raw, seed, page = TINY["B"]
    spec = _shared_cache_spec(raw)
    model = DecoderModel(spec, torch.float32)
    names = [s.name for s in model.weight_specs()]
    assert "model.layers.1.self_attn.k_proj.weight" not in names and "model.layers.1.self_attn.q_proj.weight" in names
    assert len(model.cache_needs()) == 2
    tensors = dict(random_tensors(model, 5, 0.05))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    load_weights(model, str(tmp_path), "cuda:0")
    runner = _runner(model, page=page)
    rng = random.Random(1)
    tokens = helpers.random_tokens(rng, 29, raw["vocab_size"])
    cfg = dict(raw, num_hidden_layers=2)
    ref = _plain_shared(cfg, {k: v.double() for k, v in tensors.items()}, tokens)
    # whole, then in portions and single tokens: the shared entry is written once per step
    got = runner.step([StepEntry("w", tokens, range(len(tokens)))]).cpu()
    runner.finish("w")
    assert helpers.rel_err(got, ref) < TOL["float32"]
    rows, at = [], 0
    for n in [5, 2, 9, 1, 1, 7, 4]:
        rows.append(runner.step([StepEntry("p", tokens[at:at + n], range(n))]).cpu())
        at += n
    assert at == len(tokens) and helpers.rel_err(torch.cat(rows), ref) < TOL["float32"]

    with pytest.raises(ValueError, match="written by two"):
        import dataclasses
        from pulsar_b200.config import LayerCall
        DecoderModel(dataclasses.replace(spec, run_order=(LayerCall(0, 0), LayerCall(0, 0))), torch.float32)


# ------------------------------------------------------------------ a toy mixer with state
def _register_toy():
    """A recurrent toy mixer (state s <- a*s + W_in h_t, output W_out s) and a toy architecture
    whose layers alternate between it and attention.  Everything lives in this test file."""
    from pulsar_b200.cache import CacheNeed
    from pulsar_b200.config import (ARCHITECTURES, MIXERS, BlockSpec, FeedForwardSpec, LayerCall, MixerSpec, ModelSpec,
                                    NormSpec, PositionSpec)
    from pulsar_b200.parts.base import Mixer, WeightSpec

    class ToyRecurrent(Mixer):
        graph_safe = False              # loops over the step's requests on the host

        def __init__(self, spec, prefix, dtype):
            self.spec, self.prefix, self.dtype = spec, prefix, dtype
            self.width = spec.option("state_width")
            self.decay = spec.option("decay")

        def weight_specs(self):
            return [WeightSpec(self.prefix + "in_proj.weight", (self.width, self.spec.hidden)),
                    WeightSpec(self.prefix + "out_proj.weight", (self.spec.hidden, self.width))]

        def load(self, tensors):
            self.w_in, self.w_out = tensors[self.prefix + "in_proj.weight"], tensors[self.prefix + "out_proj.weight"]

        def cache_need(self):
            return CacheNeed.state((self.width,), torch.float32)

        def forward(self, ctx, h, cache):
            u = (h.float() @ self.w_in.float().T)                       # [N, width]
            out = torch.empty_like(u)
            row = 0
            for i, (n, start) in enumerate(zip(ctx.host.q_lens, ctx.host.starts)):
                slot = ctx.host.state_slots[i]
                s = cache.state[slot] if start > 0 else torch.zeros_like(cache.state[slot])   # fresh request: fresh state
                for t in range(n):                                      # a portion's tokens in order
                    s = self.decay * s + u[row]
                    out[row] = s
                    row += 1
                cache.state[slot] = s
            return (out @ self.w_out.float().T).to(h.dtype)

    @dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        hidden_size: int
        num_hidden_layers: int
        state_width: int
        decay: float
        eps: float

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"], raw["num_hidden_layers"], raw["state_width"], raw["decay"],
                       raw["eps"])

        def to_dict(self):
            return dict(architectures=["ToyRecurrentForCausalLM"], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                        num_hidden_layers=self.num_hidden_layers, state_width=self.state_width, decay=self.decay, eps=self.eps)

        def model_spec(self):
            norm = NormSpec("rmsnorm", self.hidden_size, self.eps)
            blocks = []
            for i in range(self.num_hidden_layers):
                if i % 2 == 0:
                    mixer = MixerSpec("toy_recurrent", self.hidden_size,
                                      extra=(("state_width", self.state_width), ("decay", self.decay)))
                    sub = "recurrent."
                else:
                    mixer = MixerSpec("attention", self.hidden_size, n_heads=2, n_kv_heads=1, head_dim=16, scale=0.25,
                                      qk_norm_eps=None, position=PositionSpec("rope", 16, 8, 1e4))   # partial rotary, no q/k norm
                    sub = "attn."
                blocks.append(BlockSpec("prenorm", mixer, FeedForwardSpec("swiglu", self.hidden_size, 2 * self.hidden_size),
                                        norm, norm, f"toy.layers.{i}.",
                                        (("mixer", sub), ("feed_forward", "ffn."), ("mixer_norm", "norm1."),
                                         ("feed_forward_norm", "norm2."))))
            return ModelSpec("ToyRecurrentForCausalLM", self.vocab_size, self.hidden_size, tuple(blocks),
                             tuple(LayerCall(i, i) for i in range(self.num_hidden_layers)), norm,
                             embed_name="toy.embed.weight", final_norm_name="toy.norm.weight", head_name=None,
                             init_std=0.08)

    MIXERS.register("toy_recurrent", ToyRecurrent, replace=True)
    ARCHITECTURES.register("ToyRecurrentForCausalLM", ToyConfig.from_dict, replace=True)
    return ToyConfig


def _plain_toy(raw, w, tokens):
    t = len(tokens)
    x = w["toy.embed.weight"][torch.tensor(tokens)]
    pos = torch.arange(t)
    for i in range(raw["num_hidden_layers"]):
        p = f"toy.layers.{i}."
        h = plain.rmsnorm(x, w[p + "norm1.weight"], raw["eps"])
        if i % 2 == 0:
            u = h @ w[p + "recurrent.in_proj.weight"].T
            s = torch.zeros(raw["state_width"], dtype=torch.float64)
            rows = []
            for j in range(t):
                s = raw["decay"] * s + u[j]
                rows.append(s)
            x = x + torch.stack(rows) @ w[p + "recurrent.out_proj.weight"].T
        else:
            q = (h @ w[p + "attn.q_proj.weight"].T).view(t, 2, 16)
            k = (h @ w[p + "attn.k_proj.weight"].T).view(t, 1, 16)
            v = (h @ w[p + "attn.v_proj.weight"].T).view(t, 1, 16)

            def partial_rope(z):
                return torch.cat([plain.rope(z[..., :8], pos, 1e4), z[..., 8:]], dim=-1)
            o = plain.attention(partial_rope(q), partial_rope(k), v, 0.25)
            x = x + o.reshape(t, 32) @ w[p + "attn.o_proj.weight"].T
        h2 = plain.rmsnorm(x, w[p + "norm2.weight"], raw["eps"])
        x = x + plain.swiglu_mlp(h2, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
    return plain.rmsnorm(x, w["toy.norm.weight"], raw["eps"]) @ w["toy.embed.weight"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from pulsar_b200.config import ARCHITECTURES, MIXERS, config_from_dict
    from pulsar_b200.replay import Replay
    from pulsar_b200.weights import write_model_folder
    _register_toy()
    try:
        raw = dict(architectures=["ToyRecurrentForCausalLM"], vocab_size=97, hidden_size=48, num_hidden_layers=3,
                   state_width=24, decay=0.9, eps=1e-5)
        folder = write_model_folder(config_from_dict(raw), str(tmp_path), 7)
        _, weights = helpers.read_folder(folder)
        w = {k: v.double() for k, v in weights.items()}
        rng = random.Random(2)
        reqs = {f"r{i}": helpers.random_tokens(rng, n, 97) for i, n in enumerate([19, 33, 8, 26, 14])}
        ref = {rid: _plain_toy(raw, w, toks) for rid, toks in reqs.items()}
        rp = Replay(folder, "float32", 3 * 64, page_size=4, max_running=3)
        kinds = [n.kind for n in rp.cache.needs]
        assert kinds == ["state", "paged_kv", "state"]                  # different mixers in different layers
        trace = helpers.trace_mixed(reqs, rng, max_live=3, portion=(2, 7), decode_tail=4)
        got = {}
        for rec, rows in zip(trace.records, trace.rows):
            logits = rp.run_step(rec)
            for i, key in enumerate(rows):
                got[key] = logits[i]
        assert len(got) == sum(len(t) for t in reqs.values())
        for (rid, pos), row in got.items():
            err = helpers.rel_err(row, ref[rid][pos])
            assert err < TOL["float32"], f"{rid} position {pos}: {err:.2e}"     # state slots are reused by later requests
        rp.cache.check_consistency()
    finally:
        MIXERS.unregister("toy_recurrent")
        ARCHITECTURES.unregister("ToyRecurrentForCausalLM")


# ------------------------------------------------------------------ a toy routed feed-forward and another position encoding
def _register_routed():
    """A feed-forward that routes each token to one of several small experts (float32 router
    logits, top-1) and a rotary encoding with linearly scaled positions, both defined here."""
    from pulsar_b200.config import (ARCHITECTURES, FEED_FORWARDS, POSITIONS, BlockSpec, FeedForwardSpec, LayerCall,
                                    MixerSpec, ModelSpec, NormSpec, PositionSpec)
    from pulsar_b200.parts.base import FeedForward, PositionEncoding, WeightSpec

    class ToyRouted(FeedForward):
        graph_safe = False              # picks its rows on the host

        def __init__(self, spec, prefix, dtype):
            self.spec, self.prefix, self.dtype = spec, prefix, dtype
            self.n_experts = spec.option("n_experts")

        def weight_specs(self):
            s, p = self.spec, self.prefix
            out = [WeightSpec(p + "router.weight", (self.n_experts, s.hidden))]
            for e in range(self.n_experts):
                out += [WeightSpec(p + f"experts.{e}.up.weight", (s.intermediate, s.hidden)),
                        WeightSpec(p + f"experts.{e}.down.weight", (s.hidden, s.intermediate))]
            return out

        def load(self, tensors):
            p = self.prefix
            self.router = tensors[p + "router.weight"].float()
            self.up = [tensors[p + f"experts.{e}.up.weight"] for e in range(self.n_experts)]
            self.down = [tensors[p + f"experts.{e}.down.weight"] for e in range(self.n_experts)]

        def forward(self, ctx, h):
            logits = h.float() @ self.router.T                        # router logits in float32
            choice = logits.argmax(-1)
            out = torch.zeros_like(h)
            for e in range(self.n_experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    x = h[rows]
                    out[rows] = (torch.relu(x @ self.up[e].T) @ self.down[e].T).to(h.dtype)
            return out

    class ScaledRope(PositionEncoding):
        """cos/sin of (position / 4) * theta^(-2j/d): what the attention kernels consume, computed here."""

        def __init__(self, spec):
            self.spec = spec

        def tables(self, ctx):
            key = ("scaled", self.spec)
            if key not in ctx.shared:
                half = self.spec.rotary_dim // 2
                inv = torch.tensor([self.spec.theta ** (-2.0 * j / self.spec.rotary_dim) for j in range(half)],
                                   dtype=torch.float64, device=ctx.device)
                ang = (ctx.positions.double() / 4.0)[:, None] * inv[None, :]
                ctx.shared[key] = (torch.cos(ang).float().contiguous(), torch.sin(ang).float().contiguous())
            return ctx.shared[key]

    @dataclass(frozen=True)
    class RoutedConfig:
        vocab_size: int
        hidden_size: int
        n_experts: int

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"], raw["n_experts"])

        def to_dict(self):
            return dict(architectures=["ToyRoutedForCausalLM"], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                        n_experts=self.n_experts)

        def model_spec(self):
            norm = NormSpec("rmsnorm", self.hidden_size, 1e-5)
            mixer = MixerSpec("attention", self.hidden_size, n_heads=4, n_kv_heads=4, head_dim=16, scale=0.25,
                              qk_norm_eps=None, position=PositionSpec("toy_scaled_rope", 16, 16, 100.0))
            ffn = FeedForwardSpec("toy_routed", self.hidden_size, 40, extra=(("n_experts", self.n_experts),))
            blocks = tuple(BlockSpec("prenorm", mixer, ffn, norm, norm, f"m.{i}.",
                                     (("mixer", "attn."), ("feed_forward", "moe."), ("mixer_norm", "n1."),
                                      ("feed_forward_norm", "n2."))) for i in range(2))
            return ModelSpec("ToyRoutedForCausalLM", self.vocab_size, self.hidden_size, blocks,
                             (LayerCall(0, 0), LayerCall(1, 1)), norm, embed_name="m.embed.weight",
                             final_norm_name="m.norm.weight", head_name=None, init_std=0.3)

    FEED_FORWARDS.register("toy_routed", ToyRouted, replace=True)
    POSITIONS.register("toy_scaled_rope", ScaledRope, replace=True)
    ARCHITECTURES.register("ToyRoutedForCausalLM", RoutedConfig.from_dict, replace=True)


def _plain_routed(raw, w, tokens):
    t = len(tokens)
    x = w["m.embed.weight"][torch.tensor(tokens)]
    inv = torch.tensor([100.0 ** (-2.0 * j / 16) for j in range(8)], dtype=torch.float64)
    ang = (torch.arange(t).double() / 4.0)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rot(z):
        a, b = z[..., :8], z[..., 8:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    for i in range(2):
        p = f"m.{i}."
        h = plain.rmsnorm(x, w[p + "n1.weight"], 1e-5)
        q = (h @ w[p + "attn.q_proj.weight"].T).view(t, 4, 16)
        k = (h @ w[p + "attn.k_proj.weight"].T).view(t, 4, 16)
        v = (h @ w[p + "attn.v_proj.weight"].T).view(t, 4, 16)
        x = x + plain.attention(rot(q), rot(k), v, 0.25).reshape(t, 64) @ w[p + "attn.o_proj.weight"].T
        h2 = plain.rmsnorm(x, w[p + "n2.weight"], 1e-5)
        choice = (h2 @ w[p + "moe.router.weight"].T).argmax(-1)
        y = torch.zeros_like(h2)
        for j in range(t):
            e = int(choice[j])
            y[j] = torch.relu(h2[j] @ w[p + f"moe.experts.{e}.up.weight"].T) @ w[p + f"moe.experts.{e}.down.weight"].T
        x = x + y
    return plain.rmsnorm(x, w["m.norm.weight"], 1e-5) @ w["m.embed.weight"].T


def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    from pulsar_b200.config import ARCHITECTURES, FEED_FORWARDS, POSITIONS, config_from_dict
    from pulsar_b200.replay import Replay
    from pulsar_b200.weights import write_model_folder
    _register_routed()
    try:
        raw = dict(architectures=["ToyRoutedForCausalLM"], vocab_size=83, hidden_size=64, n_experts=3)
        folder = write_model_folder(config_from_dict(raw), str(tmp_path), 11)
        _, weights = helpers.read_folder(folder)
        w = {k: v.double() for k, v in weights.items()}
        rng = random.Random(8)
        toks = helpers.random_tokens(rng, 45, 83)
        ref = _plain_routed(raw, w, toks)
        rp = Replay(folder, "float32", 64, page_size=8)
        trace = helpers.trace_portions(toks, [9, 2, 1, 14, 3])
        rows = []
        for rec in trace.records:
            rows.append(rp.run_step(rec))
        got = torch.cat(rows)
        # a token whose two best router logits nearly tie could pick another expert in float32: none does here
        assert helpers.rel_err(got, ref) < TOL["float32"]
    finally:
        FEED_FORWARDS.unregister("toy_routed")
        POSITIONS.unregister("toy_scaled_rope")
        ARCHITECTURES.unregister("ToyRoutedForCausalLM")


# ------------------------------------------------------------------ a mixer that caches keys and values of different widths,
# in an architecture with an embedding multiplier, capped logits and a buffer in its checkpoints that nobody reads
def _register_asymmetric():
    """Attention without position encoding whose keys are 48 wide and whose values are 32 wide: two cached tensors
    of different shapes, declared by the mixer, in pools of their own.  The toy reads and writes its pages with
    plain tensor operations (it is a test of the cache's interface, not a kernel)."""
    from pulsar_b200.cache import CachedTensor, CacheNeed
    from pulsar_b200.config import (ARCHITECTURES, MIXERS, BlockSpec, FeedForwardSpec, LayerCall, MixerSpec, ModelSpec,
                                    NormSpec)
    from pulsar_b200.parts.base import Mixer, WeightSpec

    class ToyAsymmetric(Mixer):
        KEY, VALUE = 48, 32
        graph_safe = False              # loops over the step's requests on the host

        def __init__(self, spec, prefix, dtype):
            self.spec, self.prefix, self.dtype = spec, prefix, dtype

        def weight_specs(self):
            s, p = self.spec, self.prefix
            return [WeightSpec(p + "q.weight", (s.n_heads * self.KEY, s.hidden)),
                    WeightSpec(p + "k.weight", (s.n_kv_heads * self.KEY, s.hidden)),
                    WeightSpec(p + "v.weight", (s.n_kv_heads * self.VALUE, s.hidden)),
                    WeightSpec(p + "o.weight", (s.hidden, s.n_heads * self.VALUE))]

        def load(self, tensors):
            self.w = {n: tensors[self.prefix + n + ".weight"].float() for n in "qkvo"}

        def cache_need(self):
            return CacheNeed.paged((CachedTensor("key", self.spec.n_kv_heads, self.KEY),
                                    CachedTensor("value", self.spec.n_kv_heads, self.VALUE)))

        def forward(self, ctx, h, cache):
            s, n, ps = self.spec, ctx.n_tokens, cache.page_size
            x = h.float()
            q = (x @ self.w["q"].T).view(n, s.n_heads, self.KEY)
            k = (x @ self.w["k"].T).view(n, s.n_kv_heads, self.KEY)
            v = (x @ self.w["v"].T).view(n, s.n_kv_heads, self.VALUE)
            keys, values = cache.pools["key"], cache.pools["value"]            # [pages, heads, page, width]
            assert keys.shape[1:] == (s.n_kv_heads, ps, self.KEY) and values.shape[1:] == (s.n_kv_heads, ps, self.VALUE)
            slots = cache.slots.long()
            keys[slots // ps, :, slots % ps] = k.to(keys.dtype)
            values[slots // ps, :, slots % ps] = v.to(values.dtype)
            out = torch.empty(n, s.n_heads, self.VALUE, dtype=torch.float32, device=h.device)
            row, group = 0, s.n_heads // s.n_kv_heads
            for i, (n_q, kv_len) in enumerate(zip(ctx.host.q_lens, ctx.host.kv_lens)):
                pages = cache.block_table[i, :-(-kv_len // ps)].long()
                kk = keys[pages].permute(0, 2, 1, 3).reshape(-1, s.n_kv_heads, self.KEY)[:kv_len].float()
                vv = values[pages].permute(0, 2, 1, 3).reshape(-1, s.n_kv_heads, self.VALUE)[:kv_len].float()
                for t in range(n_q):
                    p = kv_len - n_q + t
                    for hd in range(s.n_heads):
                        sc = (kk[:p + 1, hd // group] @ q[row, hd]) * s.scale
                        out[row, hd] = torch.softmax(sc, 0) @ vv[:p + 1, hd // group]
                    row += 1
            return (out.view(n, -1) @ self.w["o"].T).to(h.dtype)

    @dataclass(frozen=True)
    class AsymConfig:
        vocab_size: int
        hidden_size: int
        embedding_multiplier: float
        logit_scale: float
        logit_softcap: float
        ignore: tuple

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"], raw["embedding_multiplier"], raw["logit_scale"],
                       raw["logit_softcap"], tuple(raw.get("ignore", ())))

        def to_dict(self):
            return dict(architectures=["ToyAsymmetricForCausalLM"], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                        embedding_multiplier=self.embedding_multiplier, logit_scale=self.logit_scale,
                        logit_softcap=self.logit_softcap, ignore=list(self.ignore))

        def model_spec(self):
            norm = NormSpec("rmsnorm", self.hidden_size, 1e-5)
            mixer = MixerSpec("toy_asymmetric", self.hidden_size, n_heads=4, n_kv_heads=2, scale=0.2)
            ffn = FeedForwardSpec("swiglu", self.hidden_size, 72)
            blocks = tuple(BlockSpec("prenorm", mixer, ffn, norm, norm, f"a.{i}.",
                                     (("mixer", "mix."), ("feed_forward", "ffn."), ("mixer_norm", "n1."),
                                      ("feed_forward_norm", "n2."))) for i in range(2))
            return ModelSpec("ToyAsymmetricForCausalLM", self.vocab_size, self.hidden_size, blocks,
                             (LayerCall(0, 0), LayerCall(1, 1)), norm, embed_name="a.embed.weight",
                             final_norm_name="a.norm.weight", head_name=None, init_std=0.15,
                             embedding_multiplier=self.embedding_multiplier, logit_scale=self.logit_scale,
                             logit_softcap=self.logit_softcap, ignore=self.ignore)

    MIXERS.register("toy_asymmetric", ToyAsymmetric, replace=True)
    ARCHITECTURES.register("ToyAsymmetricForCausalLM", AsymConfig.from_dict, replace=True)


def _plain_asymmetric(raw, w, tokens):
    t = len(tokens)
    x = w["a.embed.weight"][torch.tensor(tokens)] * raw["embedding_multiplier"]
    causal = torch.tril(torch.ones(t, t, dtype=torch.bool))
    for i in range(2):
        p = f"a.{i}."
        h = plain.rmsnorm(x, w[p + "n1.weight"], 1e-5)
        q = (h @ w[p + "mix.q.weight"].T).view(t, 4, 48)
        k = (h @ w[p + "mix.k.weight"].T).view(t, 2, 48)
        v = (h @ w[p + "mix.v.weight"].T).view(t, 2, 32)
        o = torch.empty(t, 4, 32, dtype=torch.float64)
        for hd in range(4):
            sc = (q[:, hd] @ k[:, hd // 2].T * 0.2).masked_fill(~causal, float("-inf"))
            o[:, hd] = torch.softmax(sc, -1) @ v[:, hd // 2]
        x = x + o.reshape(t, 128) @ w[p + "mix.o.weight"].T
        h2 = plain.rmsnorm(x, w[p + "n2.weight"], 1e-5)
        x = x + plain.swiglu_mlp(h2, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
    logits = plain.rmsnorm(x, w["a.norm.weight"], 1e-5) @ w["a.embed.weight"].T * raw["logit_scale"]
    return raw["logit_softcap"] * torch.tanh(logits / raw["logit_softcap"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cached_tensors_of_different_widths_an_ignored_buffer_and_what_sits_around_the_blocks(tmp_path, dtype):
    from safetensors.torch import load_file, save_file
    from pulsar_b200.config import ARCHITECTURES, MIXERS, config_from_dict
    from pulsar_b200.replay import Replay
    from pulsar_b200.weights import WeightError, write_model_folder
    _register_asymmetric()
    try:
        raw = dict(architectures=["ToyAsymmetricForCausalLM"], vocab_size=91, hidden_size=56, embedding_multiplier=3.5,
                   logit_scale=0.4, logit_softcap=2.5, ignore=["a.*.mix.rotary.inv_freq", "a.position_ids"])
        folder = write_model_folder(config_from_dict(raw), str(tmp_path / "m"), 21)
        path = os.path.join(folder, "model.safetensors")
        tensors = load_file(path)
        tensors["a.0.mix.rotary.inv_freq"] = torch.arange(8, dtype=torch.float32)      # what checkpoints carry along
        tensors["a.position_ids"] = torch.arange(16, dtype=torch.int64)
        save_file(tensors, path)
        _, weights = helpers.read_folder(folder)
        w = {k: v.double() for k, v in weights.items()}
        if dtype == "bfloat16":
            w = {k: v.double() for k, v in helpers.as_bf16_matrices(weights).items()}
        rng = random.Random(5)
        reqs = {f"r{i}": helpers.random_tokens(rng, n, 91) for i, n in enumerate([21, 9, 30, 13])}
        ref = {rid: _plain_asymmetric(raw, w, toks) for rid, toks in reqs.items()}
        rp = Replay(folder, dtype, 2 * 64, page_size=4, max_running=2)        # room for two requests: pages are used again
        group = rp.cache.groups[0]
        assert {n: tuple(p.shape[2:]) for n, p in group.pools.items()} == {"key": (2, 4, 48), "value": (2, 4, 32)}
        trace = helpers.trace_mixed(reqs, rng, max_live=2, portion=(2, 6), decode_tail=3)
        got = {}
        for rec, rows in zip(trace.records, trace.rows):
            logits = rp.run_step(rec)
            for i, key in enumerate(rows):
                got[key] = logits[i]
        assert len(got) == sum(len(t) for t in reqs.values())
        worst = max(helpers.rel_err(row, ref[rid][pos]) for (rid, pos), row in got.items())
        helpers.report("asymmetric_cache", worst, dtype)
        assert worst < TOL[dtype]
        assert float(torch.stack(list(got.values())).abs().max()) <= 2.5 + 1e-6         # the cap holds
        rp.cache.check_consistency()
        # without the patterns the same folder is refused, and the message names the buffers
        with pytest.raises(WeightError) as info:
            Replay(write_config(folder, dict(raw, ignore=[])), dtype, 64, page_size=4)
        assert sorted(info.value.unexpected) == ["a.0.mix.rotary.inv_freq", "a.position_ids"] and not info.value.missing
    finally:
        MIXERS.unregister("toy_asymmetric")
        ARCHITECTURES.unregister("ToyAsymmetricForCausalLM")


def write_config(folder, raw):
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    return folder


def test_a_preempted_request_of_the_recurrent_toy_mixer_starts_from_fresh_state(tmp_path):
    """So few pages that the scheduler preempts a request and computes it again from its tokens: the state slot it
    gets then starts at zero, and the tokens that come out are the plain implementation's."""
    from pulsar_b200.config import ARCHITECTURES, MIXERS, config_from_dict
    from pulsar_b200.engine.engine import Engine
    from pulsar_b200.weights import write_model_folder
    _register_toy()
    try:
        raw = dict(architectures=["ToyRecurrentForCausalLM"], vocab_size=97, hidden_size=48, num_hidden_layers=3,
                   state_width=24, decay=0.9, eps=1e-5)
        folder = write_model_folder(config_from_dict(raw), str(tmp_path), 7)
        _, weights = helpers.read_folder(folder)
        w = {k: v.double() for k, v in weights.items()}
        rng = random.Random(3)
        prompts = [helpers.random_tokens(rng, n, 97) for n in (14, 9, 12)]
        new = 22

        def plain_generate(prompt):
            seq, out = list(prompt), []
            for _ in range(new):
                tok = int(torch.argmax(_plain_toy(raw, w, seq)[-1]))
                out.append(tok)
                seq.append(tok)
            return out
        want = [plain_generate(p) for p in prompts]
        eng = Engine(folder, dict(dtype="float32", page_size=4, num_pages=20, max_sessions=4, max_running=3,
                                  max_chunk_size=16, eos_id=-1))            # 80 tokens of cache for 101 needed
        got = eng.generate(prompts, new)
        assert eng.scheduler.n_preemptions >= 1
        assert got == want
        eng.cache.check_consistency()
    finally:
        MIXERS.unregister("toy_recurrent")
        ARCHITECTURES.unregister("ToyRecurrentForCausalLM")


# ------------------------------------------------------------------ positions with two axes
def _register_two_axes():
    """A rotary encoding whose lower frequencies turn with a second axis of the position (as encodings for
    images and video have it), and an architecture that declares two axes."""
    from pulsar_b200.config import (ARCHITECTURES, POSITIONS, BlockSpec, FeedForwardSpec, LayerCall, MixerSpec, ModelSpec,
                                    NormSpec, PositionSpec)
    from pulsar_b200.parts.base import PositionEncoding

    class TwoAxisRope(PositionEncoding):
        def __init__(self, spec):
            self.spec = spec

        def tables(self, ctx):
            key = ("two_axes", self.spec)
            if key not in ctx.shared:
                half = self.spec.rotary_dim // 2
                inv = torch.tensor([self.spec.theta ** (-2.0 * j / self.spec.rotary_dim) for j in range(half)],
                                   dtype=torch.float64, device=ctx.device)
                axes = ctx.position_axes.double()                       # [2, N]
                which = (torch.arange(half, device=ctx.device) >= half // 2).long()      # upper half of the pairs: axis 1
                ang = axes[which].T * inv[None, :]                      # [N, half]
                ctx.shared[key] = (torch.cos(ang).float().contiguous(), torch.sin(ang).float().contiguous())
            return ctx.shared[key]

    @dataclass(frozen=True)
    class AxesConfig:
        vocab_size: int
        hidden_size: int

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"])

        def to_dict(self):
            return dict(architectures=["ToyAxesForCausalLM"], vocab_size=self.vocab_size, hidden_size=self.hidden_size)

        def model_spec(self):
            norm = NormSpec("rmsnorm", self.hidden_size, 1e-5)
            mixer = MixerSpec("attention", self.hidden_size, n_heads=4, n_kv_heads=2, head_dim=16, scale=0.25,
                              qk_norm_eps=1e-5, position=PositionSpec("toy_two_axis_rope", 16, 16, 50.0))
            blocks = (BlockSpec("prenorm", mixer, FeedForwardSpec("swiglu", self.hidden_size, 80), norm, norm, "x.0.",
                                (("mixer", "attn."), ("feed_forward", "ffn."), ("mixer_norm", "n1."),
                                 ("feed_forward_norm", "n2."))),)
            return ModelSpec("ToyAxesForCausalLM", self.vocab_size, self.hidden_size, blocks, (LayerCall(0, 0),), norm,
                             embed_name="x.embed.weight", final_norm_name="x.norm.weight", head_name=None, init_std=0.2,
                             position_axes=2)

    POSITIONS.register("toy_two_axis_rope", TwoAxisRope, replace=True)
    ARCHITECTURES.register("ToyAxesForCausalLM", AxesConfig.from_dict, replace=True)


def _plain_two_axes(w, tokens, second_axis):
    t = len(tokens)
    x = w["x.embed.weight"][torch.tensor(tokens)]
    inv = torch.tensor([50.0 ** (-2.0 * j / 16) for j in range(8)], dtype=torch.float64)
    pos = torch.stack([torch.arange(t).double(), torch.tensor(second_axis).double()])
    ang = pos[(torch.arange(8) >= 4).long()].T * inv[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rot(z):
        a, b = z[..., :8], z[..., 8:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    h = plain.rmsnorm(x, w["x.0.n1.weight"], 1e-5)
    q = plain.rmsnorm((h @ w["x.0.attn.q_proj.weight"].T).view(t, 4, 16), w["x.0.attn.q_norm.weight"], 1e-5)
    k = plain.rmsnorm((h @ w["x.0.attn.k_proj.weight"].T).view(t, 2, 16), w["x.0.attn.k_norm.weight"], 1e-5)
    v = (h @ w["x.0.attn.v_proj.weight"].T).view(t, 2, 16)
    x = x + plain.attention(rot(q), rot(k), v, 0.25).reshape(t, 64) @ w["x.0.attn.o_proj.weight"].T
    h2 = plain.rmsnorm(x, w["x.0.n2.weight"], 1e-5)
    x = x + plain.swiglu_mlp(h2, w["x.0.ffn.gate_proj.weight"], w["x.0.ffn.up_proj.weight"], w["x.0.ffn.down_proj.weight"])
    return plain.rmsnorm(x, w["x.norm.weight"], 1e-5) @ w["x.embed.weight"].T


def test_positions_with_two_axes_reach_a_position_encoding_defined_here(tmp_path):
    from pulsar_b200.config import ARCHITECTURES, POSITIONS, config_from_dict
    from pulsar_b200.engine.runner import StepEntry, StepError
    from pulsar_b200.replay import Replay
    from pulsar_b200.weights import write_model_folder
    _register_two_axes()
    try:
        raw = dict(architectures=["ToyAxesForCausalLM"], vocab_size=77, hidden_size=40)
        folder = write_model_folder(config_from_dict(raw), str(tmp_path), 31)
        _, weights = helpers.read_folder(folder)
        w = {k: v.double() for k, v in weights.items()}
        rng = random.Random(13)
        toks = helpers.random_tokens(rng, 26, 77)
        second = [rng.randrange(0, 9) for _ in toks]                    # a second axis that does not follow the first
        ref = _plain_two_axes(w, toks, second)
        rp = Replay(folder, "float32", 64, page_size=8)
        rows, at = [], 0
        for n in (7, 2, 1, 1, 9, 6):                                    # portions and single tokens
            rows.append(rp.runner.step([StepEntry("a", toks[at:at + n], list(range(n)), positions=[second[at:at + n]])]).cpu())
            at += n
        assert at == len(toks)
        err = helpers.rel_err(torch.cat(rows), ref)
        helpers.report("two_axes", err, "float32")
        assert err < TOL["float32"]
        # an axis that is not given repeats the index in the sequence
        rp.runner.finish("a")
        same = rp.runner.step([StepEntry("b", toks, list(range(len(toks))))]).cpu()
        assert helpers.rel_err(same, _plain_two_axes(w, toks, list(range(len(toks))))) < TOL["float32"]
        with pytest.raises(StepError, match="axes"):
            rp.runner.step([StepEntry("c", toks[:3], [2], positions=[[1, 2]])])
    finally:
        POSITIONS.unregister("toy_two_axis_rope")
        ARCHITECTURES.unregister("ToyAxesForCausalLM")
