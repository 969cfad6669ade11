"""The plain implementation itself (no GPU): against golden logits made by the reference's own
model code, and against properties each part must have."""
import json
import math
import os

import pytest
import torch

import helpers
from helpers import TINY
from plain import qwen3_plain as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_references_model_code(name, tmp_path):
    """tests/golden/make_golden.py ran the reference's Qwen3Model::forward on these weights."""
    with open(os.path.join(GOLDEN, f"tiny_{name}.json")) as f:
        gold = json.load(f)
    raw, seed, _ = TINY[name]
    assert gold["seed"] == seed
    folder = helpers.make_folder(tmp_path, raw, seed)
    cfg, weights = helpers.read_folder(folder)
    logits = plain.forward(cfg, weights, gold["tokens"], torch.float64)
    for p, row in zip(gold["positions"], gold["logits"]):
        ref = torch.tensor(row, dtype=torch.float64)
        err = float((logits[p] - ref).abs().max() / ref.abs().max())
        assert err < 2e-5, f"position {p}: {err:.2e}"            # the reference ran in float32


def test_rmsnorm_zero_row_and_scale_invariance():
    w = torch.tensor([1.0, 2.0, 0.5, 1.5], dtype=torch.float64)
    x = torch.tensor([[3.0, -4.0, 0.0, 0.0], [0.0, 0.0, 0.0, 0.0]], dtype=torch.float64)
    y = plain.rmsnorm(x, w, 1e-6)
    assert torch.isfinite(y).all() and float(y[1].abs().max()) == 0.0
    rms = math.sqrt((9 + 16) / 4 + 1e-6)
    assert torch.allclose(y[0], x[0] / rms * w)
    assert torch.allclose(plain.rmsnorm(x * 1000, w, 1e-6)[0], y[0], atol=1e-6)


def test_rope_is_a_rotation_and_scores_depend_on_distance_only():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 32, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, 32, generator=g, dtype=torch.float64)
    for theta in (1e4, 1e6):
        def score(pq, pk):
            a = plain.rope(q, torch.tensor([pq]), theta)
            b = plain.rope(k, torch.tensor([pk]), theta)
            return float((a * b).sum())
        assert abs(score(5, 3) - score(1005, 1003)) < 1e-9 and abs(score(7, 7) - float((q * k).sum())) < 1e-9
        r = plain.rope(q, torch.tensor([12345]), theta)
        assert abs(float(r.norm()) - float(q.norm())) < 1e-9
    assert torch.equal(plain.rope(q, torch.tensor([0]), 1e4), q)
    # rotate_half pairs (j, j + D/2), frequency theta^(-2j/D)
    x = torch.zeros(1, 1, 4, dtype=torch.float64)
    x[0, 0, 1] = 1.0
    y = plain.rope(x, torch.tensor([3]), 100.0)
    ang = 3 * 100.0 ** (-2 * 1 / 4)
    assert torch.allclose(y[0, 0], torch.tensor([0.0, math.cos(ang), 0.0, math.sin(ang)], dtype=torch.float64))


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    t, hq, hkv, d = 9, 4, 2, 8
    q = torch.randn(t, hq, d, generator=g, dtype=torch.float64)
    k = torch.randn(t, hkv, d, generator=g, dtype=torch.float64)
    v = torch.randn(t, hkv, d, generator=g, dtype=torch.float64)
    o = plain.attention(q, k, v, 0.3)
    assert torch.allclose(o[0], v[0].repeat_interleave(2, dim=0))          # the first token sees itself only
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 7.0, -3.0
    assert torch.allclose(plain.attention(q, k2, v2, 0.3)[:5], o[:5])      # the future does not leak
    # head h reads kv head h // group
    v3 = v.clone()
    v3[:, 1] += 100.0
    o3 = plain.attention(q, k, v3, 0.3)
    assert torch.allclose(o3[:, :2], o[:, :2]) and torch.allclose(o3[:, 2:], o[:, 2:] + 100.0)
    # all-zero q and k: exactly uniform over the visible keys (pulsar-core/tests/kernels/test_ops.cpp:63-68)
    z = torch.zeros_like(q)
    u = plain.attention(z, torch.zeros_like(k), v, 1.0)
    assert torch.allclose(u[3, 0], v[:4, 0].mean(0))
    w = plain.attention(z, torch.zeros_like(k), v, 1.0, window=3)
    assert torch.allclose(w[6, 0], v[4:7, 0].mean(0)) and torch.allclose(w[1, 0], v[:2, 0].mean(0))


def test_swiglu_and_head_tying():
    g = torch.Generator().manual_seed(2)
    h = torch.randn(3, 6, generator=g, dtype=torch.float64)
    wg, wu, wd = (torch.randn(10, 6, generator=g, dtype=torch.float64), torch.randn(10, 6, generator=g, dtype=torch.float64),
                  torch.randn(6, 10, generator=g, dtype=torch.float64))
    gate = h @ wg.T
    assert torch.allclose(plain.swiglu_mlp(h, wg, wu, wd), (torch.nn.functional.silu(gate) * (h @ wu.T)) @ wd.T)
    cfg = {"rms_norm_eps": 1e-6}
    w = {"model.norm.weight": torch.ones(6, dtype=torch.float64), "model.embed_tokens.weight": wg[:, :6]}
    tied = plain.head(h, w, cfg)
    w["lm_head.weight"] = wu
    assert tied.shape == (3, 10) and not torch.allclose(plain.head(h, w, cfg), tied)


def test_greedy_generation_stops_at_eos(tmp_path):
    raw, seed, _ = TINY["A"]
    cfg, weights = helpers.read_folder(helpers.make_folder(tmp_path, raw, seed))
    out = plain.greedy_generate(cfg, weights, [1, 2, 3], 5)
    assert len(out) == 5
    eos = out[-1]
    assert plain.greedy_generate(cfg, weights, [1, 2, 3], 5, eos_id=eos) == out[:out.index(eos) + 1]


def test_sample_filter_keeps_the_crossing_token():
    probs = torch.tensor([0.5, 0.3, 0.15, 0.05], dtype=torch.float64)
    logits = torch.log(probs)
    sp, si = plain.sample_filter(logits, 1.0, 0, 0.7)                      # 0.5, then 0.3 crosses 0.7 and stays
    assert si.tolist() == [0, 1]
    sp, si = plain.sample_filter(logits, 1.0, 3, 1.0)
    assert si.tolist() == [0, 1, 2]
    sp, si = plain.sample_filter(logits, 1.0, 1, 0.99)
    assert si.tolist() == [0]


# ---------------------------------------------------------------- the reference's own CUDA kernels
def _reference_kernel_cases():
    """tests/golden/make_reference_kernel_golden.py ran the reference's kernels, compiled unchanged, on a B200:
    rmsnorm, rope, write_kv + the scalar attention ops (and the tensor-core ones on one bfloat16 case)."""
    from safetensors import safe_open
    path = os.path.join(GOLDEN, "reference_kernels.safetensors")
    with safe_open(path, "pt") as f:
        cases = json.loads(f.metadata()["cases"])
        tensors = {name: f.get_tensor(name).clone() for name in f.keys()}
    return cases, tensors


def test_plain_rmsnorm_matches_the_references_kernel():
    cases, t = _reference_kernel_cases()
    assert len(cases["rmsnorm"]) >= 3
    for c in cases["rmsnorm"]:
        x, w, ref = (t[c[k]].to(torch.float64) for k in ("x", "weight", "out"))
        got = plain.rmsnorm(x, w, c["eps"])
        assert float(ref[-1].abs().max()) == 0.0 and float(got[-1].abs().max()) == 0.0       # the all-zero row
        err = float((got - ref).abs().max() / ref.abs().max())
        assert err < 1e-6, f"rmsnorm width {c['width']}: {err:.2e}"                            # the kernel ran in float32


def test_plain_rope_matches_the_references_kernel():
    cases, t = _reference_kernel_cases()
    assert len(cases["rope"]) >= 3
    for c in cases["rope"]:
        x, ref = t[c["x"]].to(torch.float64), t[c["out"]].to(torch.float64)                # [heads, seq, D]
        got = plain.rope(x.transpose(0, 1).contiguous(), torch.tensor(c["positions"]), c["theta"]).transpose(0, 1)
        err = float((got - ref).abs().max())
        assert err < 1e-6, f"rope head_dim {c['head_dim']} theta {c['theta']}: {err:.2e}"     # up to position 1,000,003


def test_plain_attention_matches_the_references_kernels():
    """The reference's ops hold unrotated keys and rotate key j to position j while reading it
    (pulsar-core/inc/pulsar/ops.hpp:34-43); the plain implementation rotates each key once, at its
    position, before plain attention.  Queries are taken as given (already rotated)."""
    cases, t = _reference_kernel_cases()
    assert sum(c["op"].endswith("_scalar") for c in cases["attention"]) >= 4
    for c in cases["attention"]:
        q_all, k_all, v_all, ref_all = (t[c[k]].to(torch.float64) for k in ("q", "k_unrotated", "v", "out"))
        bar = 5e-6 if c["dtype"] == "float32" else 1e-2      # seen: 4.5e-7 (scalar, float32), 2.7e-3 (tensor cores, bfloat16)
        q_at = k_at = 0
        for n_q, ctx in c["seqs"]:
            q, ref = q_all[q_at:q_at + n_q], ref_all[q_at:q_at + n_q]
            k, v = k_all[k_at:k_at + ctx], v_all[k_at:k_at + ctx]
            q_at, k_at = q_at + n_q, k_at + ctx
            k_rot = plain.rope(k, torch.arange(ctx), c["theta"])
            # the n_q queries sit at the last n_q positions of the context: run the whole context and keep those rows
            q_full = torch.zeros(ctx, *q.shape[1:], dtype=torch.float64)
            q_full[ctx - n_q:] = q
            got = plain.attention(q_full, k_rot, v, c["scale"])[ctx - n_q:]
            err = float((got - ref).abs().max() / ref.abs().max())
            assert err < bar, f"{c['op']} {c['dtype']} D={c['head_dim']} ({n_q}, {ctx}): {err:.2e}"
