"""The parts of a layer, each alone against its plain formula, and the ways they are put
together: different mixers in different layers, a run order that names a layer twice and
lets a layer read another layer's cache, and a toy mixer with state of its own that is
defined here, registered, built, loaded and stepped without touching the package (GPU)."""
import math
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
