"""Shared by the tests: tiny configurations, model folders in temporary places, the
plain implementation's view of a folder, and trace builders.

Nothing here is imported by the product package.
"""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from plain import qwen3_plain as plain

# Tiny configurations of the architecture that differ in every size and option.
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64, intermediate_size=128,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, rope_theta=10000.0,
    rms_norm_eps=1e-6, tie_word_embeddings=True, use_sliding_window=False, sliding_window=None,
    max_window_layers=2, hidden_act="silu", attention_bias=False, initializer_range=0.02, eos_token_id=7)
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=512, hidden_size=96, intermediate_size=320,
    num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=32, rope_theta=1000000.0,
    rms_norm_eps=1e-5, tie_word_embeddings=False, use_sliding_window=False, sliding_window=None,
    max_window_layers=3, hidden_act="silu", attention_bias=False, initializer_range=0.05, eos_token_id=11)
# Sizes that are no power of two, MHA-like group of 2, a window on the upper layers.
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=300, hidden_size=80, intermediate_size=176,
    num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3, head_dim=48, rope_theta=500000.0,
    rms_norm_eps=3e-6, tie_word_embeddings=False, use_sliding_window=True, sliding_window=12,
    max_window_layers=2, hidden_act="silu", attention_bias=False, initializer_range=0.04, eos_token_id=5)

# Head size 64: the sizes at which the bfloat16 path runs its tensor-core attention kernels.
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=320, hidden_size=128, intermediate_size=192,
    num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64, rope_theta=100000.0,
    rms_norm_eps=2e-6, tie_word_embeddings=True, use_sliding_window=True, sliding_window=40,
    max_window_layers=1, hidden_act="silu", attention_bias=False, initializer_range=0.03, eos_token_id=3)

# Head size 128: the size at which prompt portions run the tcgen05 attention kernel (pages of 8 or more).
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=272, hidden_size=96, intermediate_size=160,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128, rope_theta=250000.0,
    rms_norm_eps=4e-6, tie_word_embeddings=False, use_sliding_window=True, sliding_window=150,
    max_window_layers=1, hidden_act="silu", attention_bias=False, initializer_range=0.03, eos_token_id=9)

# Eight key/value heads: a few dozen sequences make more (sequence, kv head) pairs than a decode attention grid
# has block slots, so the blocks run in rounds and the split rule for that case applies.
TINY_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=336, hidden_size=192, intermediate_size=224,
    num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=8, head_dim=64, rope_theta=200000.0,
    rms_norm_eps=5e-6, tie_word_embeddings=False, use_sliding_window=False, sliding_window=None,
    max_window_layers=2, hidden_act="silu", attention_bias=False, initializer_range=0.03, eos_token_id=13)

TINY = {"A": (TINY_A, 0, 16), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 4), "D": (TINY_D, 3, 16),
        "E": (TINY_E, 4, 8), "F": (TINY_F, 6, 16)}     # config, seed, page size


def make_folder(tmpdir: str, raw: dict, seed: int, store_dtype=torch.float32, std: Optional[float] = None) -> str:
    """Write a random model folder with the product's random-weights mode."""
    from pulsar_b200.config import config_from_dict
    from pulsar_b200.weights import write_model_folder
    cfg = config_from_dict(raw)
    return write_model_folder(cfg, str(tmpdir), seed, std=std, store_dtype=store_dtype)


def read_folder(folder: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    """config.json and tensors, read with the ``safetensors`` package (not the product's reader)."""
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).clone()     # never alias the mapped file
    return cfg, weights


def as_bf16_matrices(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """What the bfloat16 engine holds: matrices rounded to bfloat16, vectors untouched."""
    return {n: (t.to(torch.bfloat16).to(torch.float32) if t.dim() >= 2 else t) for n, t in weights.items()}


def plain_logits(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    return plain.forward(cfg, weights, list(tokens), torch.float64)


def random_tokens(rng: random.Random, n: int, vocab: int) -> List[int]:
    return [rng.randrange(vocab) for _ in range(n)]


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max |ref|: error relative to the scale of the logits."""
    ref = ref.to(torch.float64)
    return float((got.to(torch.float64) - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


# Error bars relative to the logits' scale.  float32: about ten times the worst error that the replay and engine
# tests of the tiny models see (1.7e-6; every such test prints its worst error), so that a slip of the size of one
# bfloat16 rounding (4e-3) inside the float32 path cannot pass; the reference's own bar for float32 is 1e-4.
# bfloat16: the reference's bar for its bfloat16 kernels (pulsar/tests/test_paged_attention.py:50-55: 2e-2); the
# tests see up to 1.5e-2.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
# Models with the real layer sizes add up 4,096 to 25,600 terms per product: seen 9.2e-6 in float32.
TOL_LARGE = {"float32": 1e-4, "bfloat16": 2e-2}

WORST = {}      # test name -> worst relative error it saw (printed by ``report``; pytest -s or -rP shows it)


def report(test: str, worst: float, dtype: str = "") -> float:
    """Print the worst error a comparison saw, so that the distance to the bar is on record."""
    WORST[test] = max(WORST.get(test, 0.0), worst)
    print(f"[worst error] {test} {dtype}: {worst:.3e} (bar {TOL.get(dtype, float('nan')):.1e})")
    return worst


class Trace:
    """Builds step records for the replay program and remembers which (request,
    position) each wanted row belongs to."""

    def __init__(self):
        self.records: List[dict] = []
        self.fed: Dict[str, int] = {}
        self.rows: List[List[Tuple[str, int]]] = []      # per record: (request, absolute position) per wanted row

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], end: Sequence[str] = ()) -> None:
        rec = {"step": len(self.records), "entries": [], "end": list(end)}
        rows = []
        for rid, tokens, want in entries:
            start = self.fed.get(rid, 0)
            rec["entries"].append({"id": rid, "tokens": list(tokens), "want": list(want)})
            rows.extend((rid, start + w) for w in want)
            self.fed[rid] = start + len(tokens)
        for rid in end:
            self.fed.pop(rid, None)
        self.records.append(rec)
        self.rows.append(rows)

    def lines(self) -> str:
        return "".join(json.dumps(r) + "\n" for r in self.records)


def trace_whole(tokens: Sequence[int], rid: str = "a") -> Trace:
    """The request alone and whole, every position wanted."""
    t = Trace()
    t.step([(rid, tokens, range(len(tokens)))], end=[rid])
    return t


def trace_tail(tokens: Sequence[int], tail: int = 32, rid: str = "a") -> Trace:
    """Most of it in one step, the last ``tail`` tokens one by one; all of the tail wanted."""
    t = Trace()
    head = len(tokens) - tail
    assert head >= 1
    t.step([(rid, tokens[:head], [head - 1])])
    for i in range(head, len(tokens)):
        t.step([(rid, tokens[i:i + 1], [0])], end=[rid] if i == len(tokens) - 1 else [])
    return t


def trace_portions(tokens: Sequence[int], sizes: Sequence[int], rid: str = "a") -> Trace:
    """Portions of changing size (cycled), every position wanted."""
    t = Trace()
    at, i = 0, 0
    while at < len(tokens):
        n = min(sizes[i % len(sizes)], len(tokens) - at)
        if len(tokens) - at - n == 1:       # never leave a single token behind a portion: portions go down to two
            n += 1
        t.step([(rid, tokens[at:at + n], range(n))], end=[rid] if at + n == len(tokens) else [])
        at += n
        i += 1
    return t


def trace_mixed(requests: Dict[str, Sequence[int]], rng: random.Random, max_live: int = 4,
                portion: Tuple[int, int] = (2, 9), decode_tail: int = 6) -> Trace:
    """Up to ``max_live`` requests at a time: prompt portions of random size beside
    single tokens of requests that are in their tail; a request is sometimes left out of
    a step; a finished request ends and the next one starts on its pages."""
    t = Trace()
    waiting = list(requests)
    live: List[str] = []
    at: Dict[str, int] = {}
    while waiting or live:
        while waiting and len(live) < max_live:
            rid = waiting.pop(0)
            live.append(rid)
            at[rid] = 0
        entries, end = [], []
        for rid in list(live):
            toks = requests[rid]
            left = len(toks) - at[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            if left <= decode_tail:
                n = 1
            else:
                n = min(rng.randint(*portion), left - decode_tail)
            entries.append((rid, toks[at[rid]:at[rid] + n], range(n)))
            at[rid] += n
            if at[rid] == len(toks):
                end.append(rid)
                live.remove(rid)
        if entries:
            t.step(entries, end=end)
    return t
