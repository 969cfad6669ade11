#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 8b|14b|32b] [--layers L] [--batch B] [--context C] [--no-points] [--no-e2e]

A step is one decode step.  The default run has the layer sizes of the Qwen3-8B
configuration (36 layers, hidden 4096, 32/8 heads of 128, intermediate 12288, vocabulary
151936, bfloat16, page 16) with random weights, a batch of 8 and a context of 4,096: the
timed steps are the last K steps before the context reaches 4,096.  It prints one JSON
line:

  value        decoded tokens a second, device-timed over exactly K steps of the step function
               (ms_per_step their mean, ms_per_step_median the median of the steps timed one by one)
  e2e          the same through the Python entry point (Engine.step: host token ids in, host
               token ids out, index arrays copied from pinned memory every step)
  prefill      one step of 2,048 prompt tokens: tokens a second, ms, fraction of the bf16 peak
  prefill_own  the same with every product on this library's tcgen05 kernel
  roofline     bytes a decode step must read (weights once + the live cache) / its time
  points       decode tokens a second at batch 1, 16, 32 and 64 (with their fraction of the copy
               bandwidth) and at batch 8 with contexts 2,048 and 3,072
  index_bytes  host-to-device bytes of a decode step of 64 sequences, with the block tables
               resident on the device and with whole tables sent
  clocks       SM clock (median, maximum) and throttle reasons sampled through NVML every 2 ms
               during the timed steps

--impl reference runs the unmodified reference (built by baseline/build_reference.py into
baseline/_ref) through its own engine class on the same sizes, and prints the same line with
"impl": "reference", or an "unavailable" line when it is not built.

The cache of the decode measurements is filled with random keys and values instead of
being computed by a prompt pass (the decode step does the same work either way); the
prefill measurement and the e2e measurement run real prompts.  Inputs (15 GB of weights)
are larger than L2, so no L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
    intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
    sliding_window=None, max_window_layers=36, hidden_act="silu", attention_bias=False, initializer_range=0.02,
    eos_token_id=151645)
# The other dense shapes of the family, for measurements at further sizes (--shape); the default run is the 8B shape.
SHAPES = {
    "8b": dict(QWEN3_8B),
    "14b": dict(QWEN3_8B, hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40,
                max_window_layers=40),
    "32b": dict(QWEN3_8B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                max_window_layers=64),
}
PAGE = 16


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs: NVML every 2 ms from a thread of this
    process (dozens of samples for a region of a few hundred ms), nvidia-smi every 100 ms where NVML cannot be had.
    It only reads."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.rows, self.proc, self.thread, self.stop_flag = [], None, None, threading.Event()

    def _nvml_loop(self, nvml, handle):
        bits = [getattr(nvml, n, 0) for n in ("nvmlClocksThrottleReasonHwSlowdown", "nvmlClocksThrottleReasonHwThermalSlowdown",
                                              "nvmlClocksThrottleReasonSwThermalSlowdown", "nvmlClocksThrottleReasonSwPowerCap")]
        mx = nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM)
        while not self.stop_flag.is_set():
            try:
                sm = nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)
                reasons = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.rows.append([str(sm), str(mx)] + ["Active" if reasons & b else "Not Active" for b in bits])
            except Exception:
                break
            time.sleep(0.002)

    def start(self):
        self.rows, self.stop_flag = [], threading.Event()
        try:
            import pynvml as nvml
            nvml.nvmlInit()
            handle = nvml.nvmlDeviceGetHandleByIndex(0)
            self.thread = threading.Thread(target=self._nvml_loop, args=(nvml, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=1.0)
        if self.proc is not None:
            self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        reasons = [n for i, n in enumerate(self.NAMES) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def build_engine(shape: dict, n_layers: int, batch: int, context: int, max_chunk: int):
    import torch
    from pulsar_b200.config import config_from_dict
    from pulsar_b200.engine.engine import Engine
    from pulsar_b200.models import build_model
    from pulsar_b200.weights import load_random
    raw = dict(shape, num_hidden_layers=n_layers, max_window_layers=n_layers)
    cfg = config_from_dict(raw)
    model = build_model(cfg, torch.bfloat16)
    load_random(model, 0, 0.02, "cuda:0")
    pages = batch * (-(-(context + PAGE) // PAGE))
    engine = Engine.from_model(cfg, model, dict(dtype="bfloat16", device="cuda:0", page_size=PAGE, num_pages=pages,
                                                max_sessions=batch, max_running=batch, max_chunk_size=max_chunk,
                                                eos_id=-1, temperature=0.0))
    for g in engine.cache.groups:                 # random keys and values: attention is not degenerate
        for pool in g.pools.values():
            pool.normal_(0.0, 1.0)
    return engine


LAST = {}        # what the last time_decode saw beside its total: median step, index bytes per step


def decode_bytes_of_shape(raw: dict, batch: int, context: float) -> float:
    """Bytes a decode step must read, from the sizes alone: every weight once, ``batch`` embedding rows and the
    live cache (bfloat16)."""
    d, hq, hkv, hd, inter, v, layers = (raw["hidden_size"], raw["num_attention_heads"], raw["num_key_value_heads"],
                                        raw["head_dim"], raw["intermediate_size"], raw["vocab_size"], raw["num_hidden_layers"])
    per_layer = 2 * ((hq + 2 * hkv) * hd * d + hq * hd * d + 3 * inter * d) + 4 * (2 * d + 2 * hd)
    weights = layers * per_layer + 4 * d + 2 * v * d + 2 * batch * d
    return float(weights + batch * context * layers * 2 * hkv * hd * 2)


def decode_bytes(engine, batch: int, context: int) -> float:
    model = engine.model
    kv = sum(need.bytes_per_token(engine.cache.dtype) for need in engine.cache.needs if need.kind == "paged_kv")
    return float(model.weight_bytes(batch) + batch * context * kv)


def time_decode(engine, batch: int, context: int, steps: int, warmup: int, sampler=None):
    """Device time of exactly ``steps`` decode steps of ``batch`` requests that end at
    ``context`` tokens.  Returns (seconds, launches of this library's kernels)."""
    import torch
    from pulsar_b200 import ops
    from pulsar_b200.engine.runner import StepEntry
    runner, cache = engine.runner, engine.cache
    rids = [("bench", i) for i in range(batch)]
    settle = 4          # untimed steps before the warm-up: scratch buffers reach their size, the step is captured
    start_len = context - steps - warmup - settle
    for rid in rids:
        cache.open(rid)
        cache.append(rid, start_len)
    gen = torch.Generator().manual_seed(1)
    toks = torch.randint(0, engine.model.spec.vocab_size, (steps + warmup + settle, batch), generator=gen).tolist()
    ids = torch.empty(batch, dtype=torch.int32, device="cuda:0")

    def one(i):
        logits = runner.step([StepEntry(rid, [toks[i][b]], [0]) for b, rid in enumerate(rids)])
        ops.sample(logits, ids)
    for i in range(settle + warmup):
        one(i)
    torch.cuda.synchronize()
    warmup += settle
    if sampler is not None:
        sampler.start()
    launches0 = ops.LAUNCHES
    h2d0 = runner.h2d_bytes
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]      # one after every step: no waits added
    marks[0].record()
    for i in range(warmup, warmup + steps):
        one(i)
        marks[i - warmup + 1].record()
    torch.cuda.synchronize()
    seconds = marks[0].elapsed_time(marks[-1]) / 1e3
    clocks = sampler.stop() if sampler is not None else None
    launches = ops.LAUNCHES - launches0
    per_step = sorted(a.elapsed_time(b) for a, b in zip(marks, marks[1:]))
    LAST["median_ms"] = per_step[len(per_step) // 2]
    LAST["h2d_bytes_per_step"] = (runner.h2d_bytes - h2d0) / steps
    LAST["table_width"] = int(max(cache.n_logical_pages(rid) for rid in rids))
    for rid in rids:
        runner.finish(rid)
    return seconds, launches, clocks


def time_prefill(engine, tokens: int, reps: int = 7, backend: str = None):
    """One step of ``tokens`` prompt tokens.  ``backend`` "tcgen05": every product on this library's own kernel."""
    import torch
    from pulsar_b200 import ops
    from pulsar_b200.engine.runner import StepEntry
    saved = ops.GEMM_BACKEND
    if backend is not None:
        ops.GEMM_BACKEND = backend
    try:
        return _time_prefill(engine, tokens, reps)
    finally:
        ops.GEMM_BACKEND = saved


def _time_prefill(engine, tokens: int, reps: int):
    import torch
    from pulsar_b200.engine.runner import StepEntry
    gen = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, engine.model.spec.vocab_size, (tokens,), generator=gen).tolist()
    times = []
    for i in range(reps + 2):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record()
        engine.runner.step([StepEntry("prefill", prompt, [tokens - 1])])
        t1.record()
        torch.cuda.synchronize()
        engine.runner.finish("prefill")
        if i >= 2:
            times.append(t0.elapsed_time(t1) / 1e3)
    return sorted(times)[len(times) // 2]


def prefill_flops(raw: dict, tokens: int) -> float:
    d, hq, hkv, hd, inter, v = (raw["hidden_size"], raw["num_attention_heads"], raw["num_key_value_heads"],
                                raw["head_dim"], raw["intermediate_size"], raw["vocab_size"])
    per_token = 2.0 * ((hq + 2 * hkv) * hd * d + hq * hd * d + 3 * inter * d)
    attn = 4.0 * hq * hd * tokens * (tokens + 1) / 2.0          # QK^T and PV over the causal half
    return raw["num_hidden_layers"] * (per_token * tokens + attn) + 2.0 * d * v


def time_e2e(engine, batch: int, context: int, steps: int, warmup: int):
    """The same decode steps through Engine.step: host token ids in, host token ids out."""
    import torch
    # Requests finish their prompts on different steps (the prompts are fed in portions of the
    # token budget), so early ones decode a few tokens while the others still prefill.
    slack = 3 * batch + 8
    prompt_len = context - steps - warmup - 1 - slack
    gen = torch.Generator().manual_seed(3)
    prompts = torch.randint(0, engine.model.spec.vocab_size, (batch, prompt_len), generator=gen).tolist()
    sids = [engine.create_session(p) for p in prompts]
    for sid in sids:
        engine.feed(sid, [], context - prompt_len)
    started = set()
    while len(started) < batch:                   # prompts in portions until every request has its first token
        started.update(sid for sid, _, _ in engine.step(1))
    for i in range(warmup):
        engine.step(batch, lookahead=i + 1 < warmup)
    torch.cuda.synchronize()
    # Engine.step keeps one pass ahead of the tokens it returns: a call reads the ids of the pass that the call
    # before it launched and launches the next one, whose input tokens are those ids, taken on the device.  Nothing
    # is in flight when the clock starts, and the last call launches nothing more: exactly `steps` passes are launched
    # and read inside the timed region, each with its host->device copy of index arrays and its device->host read.
    h2d0 = engine.runner.h2d_bytes
    forwards0 = engine.forwards
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    t0.record()
    got = 0
    for i in range(steps):
        got += len(engine.step(batch, lookahead=i + 1 < steps))
    t1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    assert engine.forwards - forwards0 == steps, (engine.forwards - forwards0, steps)
    assert got == batch * steps, (got, batch, steps)
    h2d = (engine.runner.h2d_bytes - h2d0) / steps
    for sid in sids:
        engine.release(sid)
    return max(wall, t0.elapsed_time(t1) / 1e3), h2d, batch * 4


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: Qwen3-8B (default), 14B or 32B")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
        why = reference_arm.available()
        if why is not None:
            print(json.dumps({"impl": "reference", "unavailable": why}))
            return 0
        shape = SHAPES[args.shape]
        line = reference_arm.run(args, shape, f"Qwen3-{args.shape.upper()} shape", peaks(), prefill_flops,
                                 decode_bytes_of_shape, ClockSampler)
        print(json.dumps(line))
        return 0
    warmup = max(3, args.warmup)
    import torch
    from pulsar_b200 import ops
    pk = peaks()
    big = 64 if not args.no_points else args.batch
    shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    engine = build_engine(shape, args.layers, max(big, args.batch), args.context, 2048)
    raw = dict(shape, num_hidden_layers=args.layers)
    name = f"Qwen3-{args.shape.upper()} shape"

    sampler = ClockSampler()
    # The sampler is a thread of this process; on a busy host it can go without the processor for most of a region of
    # a few hundred ms.  A region that it saw fewer than ten times is measured again (twice at most).
    for attempt in range(3):
        seconds, launches, clocks = time_decode(engine, args.batch, args.context, args.steps, warmup, sampler)
        clocks["regions_measured"] = attempt + 1
        if clocks.get("samples", 0) >= 10:
            break
    value = args.batch * args.steps / seconds
    ms_step = seconds / args.steps * 1e3
    mid_context = args.context - args.steps / 2.0
    achieved = decode_bytes(engine, args.batch, mid_context) / (seconds / args.steps) / 1e9

    median_ms = LAST.get("median_ms")
    p_seconds = time_prefill(engine, 2048)
    p_flops = prefill_flops(raw, 2048)
    prefill = {"value": 2048 / p_seconds, "tokens": 2048, "ms": p_seconds * 1e3,
               "frac": p_flops / p_seconds / (pk["bf16_tflops"] * 1e12)}
    own_seconds = time_prefill(engine, 2048, backend="tcgen05")
    prefill_own = {"value": 2048 / own_seconds, "tokens": 2048, "ms": own_seconds * 1e3,
                   "frac": p_flops / own_seconds / (pk["bf16_tflops"] * 1e12), "what": "every product on gemm_tcgen05"}

    points, index_bytes = {}, {}
    if not args.no_points:
        for b in (1, 16, 32, 64):
            s, _, _ = time_decode(engine, b, args.context, args.steps, warmup)
            points[f"decode_b{b}"] = b * args.steps / s
            points[f"decode_b{b}_hbm_frac"] = decode_bytes(engine, b, mid_context) / (s / args.steps) / 1e9 / pk["hbm_gbs"]
            if b == 64:            # index arrays of a step: what travels with resident block tables, and what whole tables would be
                index_bytes = {"batch": 64, "h2d_bytes_per_step": LAST["h2d_bytes_per_step"],
                               "with_whole_tables": LAST["h2d_bytes_per_step"] + 4.0 * 64 * (-(-LAST["table_width"] // 64) * 64)}
        for ctx in (2048, 3072):
            if ctx < args.context:
                s, _, _ = time_decode(engine, args.batch, ctx, args.steps, warmup)
                points[f"decode_b{args.batch}_ctx{ctx}"] = args.batch * args.steps / s
    e2e = None
    if not args.no_e2e:
        # the entry point's first passes after an idle moment run slower than its steady state (4.0, 4.0, 3.8 ms before
        # 3.51): its warm-up is at least 8 passes, said in the line
        e2e_warmup = max(warmup, 8)
        e_seconds, h2d, d2h = time_e2e(engine, args.batch, args.context, args.steps, e2e_warmup)
        e2e = {"value": args.batch * args.steps / e_seconds, "unit": "tokens/s", "warmup": e2e_warmup, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h}

    line = {
        "metric": f"decode tok/s at batch {args.batch} ({name}, context {args.context}); prefill and batch 1/64 alongside",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids, random cache contents for decode",
        "impl": "ours",
        "config": {"model": name, "global_batch": args.batch, "seq_len": args.context, "parallelism": "single GPU",
                   "layers": args.layers, "layers_of_configuration": full_layers, "hidden": shape["hidden_size"],
                   "q_heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
                   "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
                   "page_size": PAGE, "prompt_tokens": 2048,
                   "l2": f"inputs larger than L2 (weights {engine.model.weight_bytes(1) / 1e9:.0f} GB)", "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "ms_per_step_median": median_ms,
        "prefill": prefill, "prefill_own": prefill_own, "index_bytes": index_bytes,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
