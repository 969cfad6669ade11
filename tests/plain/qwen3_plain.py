"""Plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the product
package: it reads a ``config.json`` dictionary and a ``{name: tensor}`` mapping and
evaluates the formulas that cosmonomic/pulsar's Qwen3 model evaluates, in the order in
which it evaluates them.  Every function cites the place in the reference that fixes
its formula (paths are relative to the reference project's root).

All arithmetic runs on the CPU in one dtype (float64 by default), so that the
engine's float32 and bfloat16 paths can both be compared against something more
exact than either.

One extension beyond the reference: a sliding attention window (the architecture's
``sliding_window`` / ``use_sliding_window`` / ``max_window_layers`` keys, which the
reference does not read).  A query at position p sees key j iff ``p - window < j <= p``.
"""
from __future__ import annotations

import math

import torch


def embedding(token_ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x[t] = E[token[t]]  (pulsar-core/src/model/paged_forward.cpp:89)."""
    return table[token_ids.long()]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis
    (pulsar-core/src/kernels/rmsnorm.cu:29-49)."""
    mean_sq = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(mean_sq + eps) * weight


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """a[t, j] = p_t * theta^(-2j/D), j < D/2, formed in float64
    (pulsar-core/inc/pulsar/rope.hpp:52-56, 95-100)."""
    j = torch.arange(head_dim // 2, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * j / head_dim)
    return positions.to(torch.float64)[:, None] * inv_freq[None, :]


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """rotate_half over the full head_dim; x is [T, H, D]
    (pulsar-core/src/kernels/rope.cu:42-50; pulsar-core/inc/pulsar/rope.hpp:95-104)."""
    d = x.shape[-1]
    ang = rope_angles(positions, d, theta)
    cos = torch.cos(ang).to(x.dtype)[:, None, :]
    sin = torch.sin(ang).to(x.dtype)[:, None, :]
    first, second = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([first * cos - second * sin, second * cos + first * sin], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: int | None = None) -> torch.Tensor:
    """Causal grouped-query attention over one whole sequence.

    q [T, Hq, D], k/v [T, Hkv, D]; q head h reads kv head h // (Hq/Hkv); the query at
    index p attends keys [0, p]; s = scale * q.k; softmax over keys; o = sum p*v
    (pulsar-core/src/kernels/paged_common.cu:85-123; pulsar-core/inc/pulsar/ops.hpp:106-111).
    ``window`` (not in the reference) hides keys j <= p - window.
    """
    t, hq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    out = torch.empty_like(q)
    idx = torch.arange(t)
    visible = idx[None, :] <= idx[:, None]
    if window is not None:
        visible &= idx[None, :] > idx[:, None] - window
    for h in range(hq):
        g = h // group
        scores = (q[:, h, :] @ k[:, g, :].T) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ v[:, g, :]
    return out


def swiglu_mlp(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """(silu(h Wg^T) * (h Wu^T)) Wd^T, silu(z) = z * sigmoid(z)
    (pulsar-core/src/model/qwen3.cpp:117-119)."""
    gate = h @ w_gate.T
    up = h @ w_up.T
    return ((gate * torch.sigmoid(gate)) * up) @ w_down.T


def layer_window(cfg: dict, layer: int) -> int | None:
    """Window of a layer by the architecture's own keys: a ``layer_types`` list decides where it is
    given; else layers with index >= max_window_layers slide when use_sliding_window is set (keys the
    reference ignores, pulsar/src/pulsar/checkpoint.py:36-51 reads none of them)."""
    if cfg.get("layer_types") is not None:
        return int(cfg["sliding_window"]) if cfg["layer_types"][layer] == "sliding_attention" else None
    if not cfg.get("use_sliding_window", False) or cfg.get("sliding_window") is None:
        return None
    return int(cfg["sliding_window"]) if layer >= int(cfg.get("max_window_layers", 0)) else None


def attention_block(x: torch.Tensor, positions: torch.Tensor, w: dict, prefix: str, cfg: dict,
                    layer: int) -> torch.Tensor:
    """q/k/v projections without bias, per-head q/k RMSNorm with the layer eps before
    RoPE, RoPE on q and k, attention with scale 1/sqrt(D), output projection
    (pulsar-core/src/model/qwen3.cpp:81-114, :47 for the scale)."""
    t = x.shape[0]
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // hq
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    q = (x @ w[prefix + "q_proj.weight"].T).view(t, hq, d)
    k = (x @ w[prefix + "k_proj.weight"].T).view(t, hkv, d)
    v = (x @ w[prefix + "v_proj.weight"].T).view(t, hkv, d)
    q = rmsnorm(q, w[prefix + "q_norm.weight"], eps)
    k = rmsnorm(k, w[prefix + "k_norm.weight"], eps)
    q = rope(q, positions, theta)
    k = rope(k, positions, theta)
    o = attention(q, k, v, 1.0 / math.sqrt(d), layer_window(cfg, layer))
    return o.reshape(t, hq * d) @ w[prefix + "o_proj.weight"].T


def block(x: torch.Tensor, positions: torch.Tensor, w: dict, layer: int, cfg: dict) -> torch.Tensor:
    """x += attn(norm(x)); x += mlp(norm(x))  (pulsar-core/src/model/qwen3.cpp:77-121)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = rmsnorm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(h, positions, w, p + "self_attn.", cfg, layer)
    h2 = rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu_mlp(h2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return x


def head(x: torch.Tensor, w: dict, cfg: dict) -> torch.Tensor:
    """Final RMSNorm, then logits = x W^T with W = lm_head.weight when that tensor
    exists, else the token embedding (pulsar-core/src/model/qwen3.cpp:51-53, 123-129)."""
    x = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    table = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return x @ table.T


def forward(cfg: dict, weights: dict, token_ids, dtype: torch.dtype = torch.float64,
            return_hidden: bool = False) -> torch.Tensor:
    """Logits [T, V] of one whole sequence at positions 0..T-1
    (pulsar-core/src/model/paged_forward.cpp:82-94)."""
    w = {name: t.to(dtype) for name, t in weights.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    x = embedding(ids, w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        x = block(x, positions, w, layer, cfg)
    if return_hidden:
        return x
    return head(x, w, cfg)


def greedy_generate(cfg: dict, weights: dict, prompt, max_new_tokens: int, eos_id: int = -1,
                    dtype: torch.dtype = torch.float64) -> list[int]:
    """argmax of the raw last-row logits, one token at a time, by re-running the
    whole sequence (pulsar-core/src/runtime/sampler.cpp:13-15;
    pulsar-core/src/runtime/engine.cpp:727-729 for the stop rule)."""
    seq = list(prompt)
    out: list[int] = []
    for _ in range(max_new_tokens):
        logits = forward(cfg, weights, seq, dtype)
        token = int(torch.argmax(logits[-1]))
        out.append(token)
        seq.append(token)
        if token == eos_id:
            break
    return out


def sample_filter(logits_row: torch.Tensor, temperature: float, top_k: int, top_p: float):
    """Surviving (probabilities, token ids) of one row, sorted by descending
    probability: softmax(logits / T); top_k > 0 keeps ranks < k; top_p in (0,1) keeps a
    token when the mass strictly before it is <= top_p; both -> the intersection
    (pulsar-core/src/runtime/sampler.cpp:18-42)."""
    probs = torch.softmax(logits_row.to(torch.float64) / temperature, dim=-1)
    sp, si = torch.sort(probs, descending=True, stable=True)
    keep = torch.ones_like(sp, dtype=torch.bool)
    if top_k > 0:
        keep &= torch.arange(sp.numel()) < top_k
    if 0.0 < top_p < 1.0:
        keep &= (torch.cumsum(sp, 0) - sp) <= top_p
    return sp[keep], si[keep]
