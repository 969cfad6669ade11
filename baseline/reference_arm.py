"""The reference arm of ``bench.py``: the unmodified reference, driven through its own public API.

The reference's Python-facing engine is the TorchBind class ``torch.classes.pulsar.Engine``
(pulsar/ext/engine.cpp:419-449; pulsar/src/pulsar/core/engine.py:9): constructed from a
dictionary of named weights, a flat configuration dictionary and a dtype, and driven with
``create_session`` / ``feed`` / ``set_decode_budget`` / ``step(n)`` / ``release``.  That surface
is what this file calls; the forward pass, the cache, the scheduler, the sampler and every
kernel behind it are the reference's (built unchanged by ``baseline/build_reference.py``).
Nothing of ``pulsar_b200`` is imported here.  The asyncio layer above the class
(pulsar/src/pulsar/rt) needs Python 3.13 (``asyncio.Queue.shutdown``) and is not used.

Same metric, configuration and protocol as the other arm: Qwen3-8B layer sizes, random bfloat16
weights N(0, 0.02), batch 8, the timed decode steps are the last K before the context reaches
4,096, prefill of 2,048 tokens, points at batch 1 and 64.  ``value`` is device-timed (CUDA events
around the K calls of ``step``), ``e2e`` is the wall clock around the same calls: the reference
reads every sampled token back to the host inside ``step`` (pulsar-core/src/runtime/sampler.cpp:14),
so each call already contains its host-to-device copies and its device-to-host reads.
"""
from __future__ import annotations

import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
PAGE = 16


def available():
    """None when the reference can be loaded, else the reason in one line."""
    lib = os.path.join(REF, "pulsar", "pulsar_core.so")
    if not os.path.isfile(lib):
        return ("baseline/_ref/pulsar/pulsar_core.so is not built: run `python baseline/build_reference.py --src <checkout>` "
                "where the reference's sources are (its own build needs xmake, hatchling, Python 3.13 and torch 2.14)")
    import torch
    if not torch.cuda.is_available():
        return "no CUDA device here: the reference's engine runs on a GPU only"
    return None


def load_engine_class():
    import torch
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import pulsar.core  # noqa: F401  (loads pulsar_core.so: registers the class and the ops)
    return torch.classes.pulsar.Engine


def random_weights(raw: dict, n_layers: int, device: str):
    """Tensors under the names the reference resolves (pulsar-core/src/model/qwen3.cpp:48-72), all bfloat16."""
    import torch
    gen = torch.Generator(device=device).manual_seed(0)
    d, hq, hkv, hd, inter, v = (raw["hidden_size"], raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"],
                                raw["intermediate_size"], raw["vocab_size"])

    def matrix(rows, cols):
        return (torch.randn(rows, cols, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    def vector(n):
        return (1.0 + 0.1 * torch.randn(n, generator=gen, device=device, dtype=torch.float32)).to(torch.bfloat16)

    w = {"model.embed_tokens.weight": matrix(v, d), "model.norm.weight": vector(d), "lm_head.weight": matrix(v, d)}
    for i in range(n_layers):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = vector(d)
        w[p + "post_attention_layernorm.weight"] = vector(d)
        w[p + "self_attn.q_proj.weight"] = matrix(hq * hd, d)
        w[p + "self_attn.k_proj.weight"] = matrix(hkv * hd, d)
        w[p + "self_attn.v_proj.weight"] = matrix(hkv * hd, d)
        w[p + "self_attn.o_proj.weight"] = matrix(d, hq * hd)
        w[p + "self_attn.q_norm.weight"] = vector(hd)
        w[p + "self_attn.k_norm.weight"] = vector(hd)
        w[p + "mlp.gate_proj.weight"] = matrix(inter, d)
        w[p + "mlp.up_proj.weight"] = matrix(inter, d)
        w[p + "mlp.down_proj.weight"] = matrix(d, inter)
    return w


def build_engine(raw: dict, n_layers: int, sessions: int, context: int, max_chunk: int):
    import torch
    Engine = load_engine_class()
    weights = random_weights(raw, n_layers, "cuda:0")
    window = -(-(context + 4 * PAGE) // PAGE) * PAGE
    config = {
        "model": "qwen3-8b", "max_sessions": sessions, "n_layers": n_layers, "n_heads": raw["num_attention_heads"],
        "n_kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"], "hidden": raw["hidden_size"],
        "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"], "rope_theta": float(raw["rope_theta"]),
        "rms_eps": float(raw["rms_norm_eps"]), "active_buffer_size": window, "page_size": PAGE, "device": "cuda:0",
        "max_running": sessions, "max_chunk_size": max_chunk, "eos_id": -1, "temperature": 0.0, "top_p": 1.0, "top_k": 0,
        "seed": -1,
    }
    return Engine(weights, config, torch.bfloat16), weights


def _open(engine, prompt):
    """A session that is scheduled: ``create_session`` registers the first tokens, the first ``feed`` schedules
    (pulsar-core/src/runtime/engine.cpp:312-375, 392-412)."""
    sid = engine.create_session(prompt[:-1], {})
    engine.feed(sid, prompt[-1:])
    return sid


def time_decode(engine, vocab: int, batch: int, context: int, steps: int, warmup: int, sampler=None):
    """K calls of ``step(batch)`` with ``batch`` sequences decoding, the last of which brings the contexts to
    ``context``.  Returns (device seconds, wall seconds, clocks)."""
    import torch
    # Prompts are prefilled in portions of the token budget, so the first ones decode a few tokens while the
    # others still prefill: leave room for that (as the other arm's end-to-end measurement does).
    slack = 3 * batch + 8
    prompt_len = context - steps - warmup - 1 - slack
    gen = torch.Generator().manual_seed(3)
    prompts = torch.randint(0, vocab, (batch, prompt_len), generator=gen).tolist()
    sids = [_open(engine, p) for p in prompts]
    started = set()
    while len(started) < batch:
        ids, _, _ = engine.step(1)
        started.update(ids)
    for _ in range(warmup):
        engine.step(batch)
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    t0.record()
    got = 0
    for _ in range(steps):
        ids, _, _ = engine.step(batch)
        got += len(ids)
    t1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop() if sampler is not None else None
    assert got == batch * steps, (got, batch, steps)
    for sid in sids:
        engine.release(sid)
    return t0.elapsed_time(t1) / 1e3, wall, clocks


def time_prefill(engine, vocab: int, tokens: int, reps: int = 5):
    """One step that runs a whole prompt of ``tokens`` tokens and samples its first token."""
    import torch
    gen = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
    times = []
    for i in range(reps + 2):
        sid = _open(engine, prompt)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record()
        engine.step(1)
        t1.record()
        torch.cuda.synchronize()
        engine.release(sid)
        if i >= 2:
            times.append(t0.elapsed_time(t1) / 1e3)
    return sorted(times)[len(times) // 2]


def run(args, shape: dict, name: str, pk: dict, prefill_flops, decode_bytes, ClockSampler) -> dict:
    """The bench line of the reference arm (same keys as the other arm's)."""
    warmup = max(3, args.warmup)
    layers = args.layers if args.layers is not None else shape["num_hidden_layers"]
    raw = dict(shape, num_hidden_layers=layers)
    big = 64 if not args.no_points else args.batch
    engine, weights = build_engine(raw, layers, max(big, args.batch), args.context, 2048)
    vocab = raw["vocab_size"]
    p_seconds = time_prefill(engine, vocab, 2048)
    device_s, wall_s, clocks = time_decode(engine, vocab, args.batch, args.context, args.steps, warmup, ClockSampler())
    points = {}
    if not args.no_points:
        for b in (1, 64):
            s, _, _ = time_decode(engine, vocab, b, args.context, args.steps, warmup)
            points[f"decode_b{b}"] = b * args.steps / s
    value = args.batch * args.steps / device_s
    achieved = decode_bytes(raw, args.batch, args.context - args.steps / 2.0) / (device_s / args.steps) / 1e9
    # index arrays the reference's scheduler copies per decode step (pulsar-core/src/runtime/scheduler.cpp:172-220:
    # context lengths, page tables, slot mapping; token ids and positions from engine.cpp:654-702), and the ids it reads back
    table_width = -(-args.context // PAGE)
    h2d = args.batch * 4 * (1 + table_width + 1) + args.batch * 16
    return {
        "metric": f"decode tok/s at batch {args.batch} ({name}, context {args.context}); prefill and batch 1/64 alongside",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": device_s / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids, prompts prefilled by the engine",
        "impl": "reference",
        "config": {"model": name, "global_batch": args.batch, "seq_len": args.context, "parallelism": "single GPU",
                   "layers": layers, "layers_of_configuration": shape["num_hidden_layers"], "hidden": shape["hidden_size"],
                   "q_heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
                   "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
                   "page_size": PAGE, "prompt_tokens": 2048, "l2": "inputs larger than L2 (weights)", "peaks": pk["source"],
                   "api": "torch.classes.pulsar.Engine create_session/feed/step"},
        "e2e": {"value": args.batch * args.steps / wall_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": args.batch * 8},
        "gpu_launches": None, "clocks": clocks,
        "prefill": {"value": 2048 / p_seconds, "tokens": 2048, "ms": p_seconds * 1e3,
                    "frac": prefill_flops(raw, 2048) / p_seconds / (pk["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
        "points": points,
    }
