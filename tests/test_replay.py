"""Replay of the same requests in different cuts and batches against the plain
implementation, in float32 and in bfloat16 (GPU)."""
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
from helpers import TINY, TOL

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (raw, seed, page) in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny{name}")
        helpers.make_folder(d, raw, seed)
        out[name] = str(d)
    return out


def _reference(folder, dtype, requests):
    cfg, w = helpers.read_folder(folder)
    if dtype == "bfloat16":
        w = helpers.as_bf16_matrices(w)
    return {rid: helpers.plain_logits(cfg, w, toks) for rid, toks in requests.items()}


def _replay(folder, dtype, trace, max_tokens, page_size, max_running=8, inspect=None):
    from pulsar_b200.replay import Replay
    rp = Replay(folder, dtype, max_tokens, page_size=page_size, max_running=max_running)
    got = {}
    for rec, rows in zip(trace.records, trace.rows):
        logits = rp.run_step(rec)
        assert (logits is None) == (len(rows) == 0)
        for i, key in enumerate(rows):
            got[key] = logits[i]
    rp.cache.check_consistency()
    assert rp.cache.live_requests() == []
    assert all(f == g.allocator.n for f, g in zip(rp.cache.n_free_pages(), rp.cache.groups))
    if inspect is not None:
        inspect(rp)
    return got


def _compare(got, ref, dtype):
    assert got
    worst = 0.0
    for (rid, pos), row in got.items():
        err = helpers.rel_err(row, ref[rid][pos])
        worst = max(worst, err)
        assert err < TOL[dtype], f"request {rid} position {pos}: error {err:.3e} (first wrong place)"
    return helpers.report(os.environ.get("PYTEST_CURRENT_TEST", "replay").split("::")[-1].split(" ")[0], worst, dtype)


def _round64(n):
    return -(-n // 64) * 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole(folders, name, dtype):
    raw, seed, page = TINY[name]
    rng = random.Random(seed)
    toks = helpers.random_tokens(rng, 70, raw["vocab_size"])
    ref = _reference(folders[name], dtype, {"a": toks})
    got = _replay(folders[name], dtype, helpers.trace_whole(toks), _round64(len(toks)), page)
    _compare(got, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_tail_decoded_one_by_one(folders, name, dtype):
    raw, seed, page = TINY[name]
    rng = random.Random(seed + 10)
    toks = helpers.random_tokens(rng, 75, raw["vocab_size"])
    ref = _reference(folders[name], dtype, {"a": toks})
    got = _replay(folders[name], dtype, helpers.trace_tail(toks, 32), _round64(len(toks)), page)
    assert len(got) == 33
    _compare(got, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_portions_of_changing_size(folders, name, dtype):
    raw, seed, page = TINY[name]
    rng = random.Random(seed + 20)
    toks = helpers.random_tokens(rng, 83, raw["vocab_size"])
    ref = _reference(folders[name], dtype, {"a": toks})
    got = _replay(folders[name], dtype, helpers.trace_portions(toks, [7, 2, 13, 2, 5, 17, 3]), _round64(len(toks)), page)
    assert len(got) == len(toks)
    _compare(got, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_mixed_with_page_reuse(folders, name, dtype):
    raw, seed, page = TINY[name]
    rng = random.Random(seed + 30)
    lengths = [40, 23, 64, 9, 31, 50, 17, 28, 45]
    requests = {f"r{i}": helpers.random_tokens(rng, n, raw["vocab_size"]) for i, n in enumerate(lengths)}
    ref = _reference(folders[name], dtype, requests)
    trace = helpers.trace_mixed(requests, rng, max_live=4)
    # The four largest live together at worst: so few pages that every page is used again.
    budget = sum(sorted(_round64(n) for n in lengths)[-4:])
    assert budget < sum(_round64(n) for n in lengths)
    got = _replay(folders[name], dtype, trace, budget, page, max_running=4)
    assert len(got) == sum(lengths)
    _compare(got, ref, dtype)


# Ragged contexts of the reference's decode-attention test (pulsar/tests/test_paged_attention.py:21-45), shortened
# where the tiny models would make the plain implementation slow.
RAGGED = [1, 7, 16, 33, 40, 65, 100, 129]


def trace_many_decoding(requests, tail, per_step, order):
    """Prompts (all but the last ``tail`` tokens) whole, ``per_step`` requests to a step, the last row wanted; then
    ``tail`` steps in which every request brings one token.  All requests end with the last step."""
    t = helpers.Trace()
    for at in range(0, len(order), per_step):
        t.step([(rid, requests[rid][:-tail], [len(requests[rid]) - tail - 1]) for rid in order[at:at + per_step]])
    for i in range(tail, 0, -1):
        t.step([(rid, [requests[rid][-i]], [0]) for rid in order], end=order if i == 1 else [])
    return t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n", [("D", 20), ("E", 40), ("F", 40), ("F", 72), ("D", 72)])
def test_steps_of_many_single_tokens(folders, name, n, dtype):
    """The decode step of a large batch: 20, 40 and 72 requests with ragged contexts, then seven steps in which
    all of them bring one token (in bfloat16 more than 16 rows take the product for many tokens and a gating
    kernel of its own; with 8 kv heads 40 requests are more (sequence, kv head) pairs than the decode attention
    has block slots, so its blocks run in rounds; from the fourth such step on the captured graph is replayed).
    Two waves of requests on a pool that holds one: every page of the second wave was used by the first.
    Every row against the plain implementation."""
    raw, seed, page = TINY[name]
    rng = random.Random(seed + 70 + n)
    tail = 7
    waves = []
    for w in range(2):
        lens = [RAGGED[(i + 3 * w) % len(RAGGED)] % 70 + tail + 1 + (i % 5) for i in range(n)]
        waves.append({f"w{w}r{i}": helpers.random_tokens(rng, ln, raw["vocab_size"]) for i, ln in enumerate(lens)})
    ref = {}
    for reqs in waves:
        ref.update(_reference(folders[name], dtype, reqs))
    budget = max(sum(-(-len(t) // 64) * 64 for t in reqs.values()) for reqs in waves)
    trace = helpers.Trace()
    for reqs in waves:
        order = list(reqs)
        sub = trace_many_decoding(reqs, tail, 9, order)
        for rec in sub.records:
            trace.step([(e["id"], e["tokens"], e["want"]) for e in rec["entries"]], end=rec["end"])

    def inspect(rp):
        assert rp.runner.graph_replays >= 2 * (tail - 3), rp.runner.graph_replays      # the captured step ran

    got = _replay(folders[name], dtype, trace, budget, page, max_running=n, inspect=inspect)
    assert len(got) == 2 * n * (tail + 1)
    _compare(got, ref, dtype)


@pytest.mark.parametrize("name,n", [("D", 40), ("F", 72)])
def test_steps_of_many_single_tokens_on_the_weight_streaming_tcgen05_product(folders, name, n, monkeypatch):
    """The same large decode steps with every projection of 17 to 128 tokens on this library's weight-streaming
    tcgen05 kernel (slices of K over the blocks of a cluster, SwiGLU in its epilogue) instead of the library product."""
    from pulsar_b200 import ops
    monkeypatch.setattr(ops, "STREAM_GEMM", "1")
    raw, seed, page = TINY[name]
    rng = random.Random(seed + 170 + n)
    tail = 5
    lens = [RAGGED[i % len(RAGGED)] % 70 + tail + 1 + (i % 5) for i in range(n)]
    reqs = {f"r{i}": helpers.random_tokens(rng, ln, raw["vocab_size"]) for i, ln in enumerate(lens)}
    ref = _reference(folders[name], "bfloat16", reqs)
    trace = trace_many_decoding(reqs, tail, 9, list(reqs))
    got = _replay(folders[name], "bfloat16", trace, sum(-(-len(t) // 64) * 64 for t in reqs.values()), page, max_running=n)
    assert len(got) == n * (tail + 1)
    _compare(got, ref, "bfloat16")
    ops.check_wait_words()


@pytest.mark.parametrize("norms", ["all_inside", "none_inside"])
@pytest.mark.parametrize("name", ["D", "F"])
def test_decoding_with_the_norms_inside_the_products_or_in_kernels_of_their_own(folders, name, norms, monkeypatch):
    """Steps of a few tokens in bfloat16 take the residual addition, and the norm in front of q/k/v, into the weight-
    streaming products.  The same replay with the norm in front of gate/up inside its product too, and with
    everything in kernels of its own: all against the plain implementation."""
    from pulsar_b200 import ops
    monkeypatch.setattr(ops, "FUSED_NORM_MLP", norms == "all_inside")
    monkeypatch.setattr(ops, "FUSED_NORM", norms == "all_inside")
    raw, seed, page = TINY[name]
    rng = random.Random(seed + 90)
    requests = {f"r{i}": helpers.random_tokens(rng, n, raw["vocab_size"]) for i, n in enumerate([44, 71, 23, 50, 37])}
    ref = _reference(folders[name], "bfloat16", requests)
    trace = helpers.trace_mixed(requests, rng, max_live=3, portion=(2, 9), decode_tail=20)
    got = _replay(folders[name], "bfloat16", trace, 3 * 128, page, max_running=3)
    assert len(got) == sum(len(t) for t in requests.values())
    _compare(got, ref, "bfloat16")


@pytest.mark.parametrize("name", ["B", "D"])
def test_portions_with_the_tcgen05_products(folders, name, monkeypatch):
    """The same replay with every projection of more than 16 rows on the tcgen05 / TMA kernel
    (SwiGLU fused into the gate/up product) instead of the library product."""
    from pulsar_b200 import ops
    monkeypatch.setattr(ops, "GEMM_BACKEND", "tcgen05")
    raw, seed, page = TINY[name]
    rng = random.Random(seed + 40)
    toks = helpers.random_tokens(rng, 150, raw["vocab_size"])
    ref = _reference(folders[name], "bfloat16", {"a": toks})
    got = _replay(folders[name], "bfloat16", helpers.trace_portions(toks, [70, 3, 40, 17, 20]), _round64(len(toks)), page)
    assert len(got) == len(toks)
    _compare(got, ref, "bfloat16")
    assert ops.gemm_tcgen05_error() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_head_size_128(folders, dtype):
    """Head size 128 (bfloat16: the tcgen05 attention kernel): portions that cross its 128-row and
    128-key tiles and the window of the upper layer, a long tail decoded one by one."""
    from pulsar_b200 import ops
    raw, seed, page = TINY["E"]
    rng = random.Random(seed + 50)
    toks = helpers.random_tokens(rng, 420, raw["vocab_size"])
    ref = _reference(folders["E"], dtype, {"a": toks})
    got = _replay(folders["E"], dtype, helpers.trace_portions(toks, [130, 2, 127, 129, 5]), _round64(len(toks)), page)
    assert len(got) == len(toks)
    _compare(got, ref, dtype)
    got = _replay(folders["E"], dtype, helpers.trace_tail(toks[:300], 32), _round64(300), page)
    _compare(got, ref, dtype)
    assert ops.prefill_tcgen05_error() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_types_choose_the_sliding_layers(tmp_path, dtype):
    """config.json may list which layers slide: here the lower two of four, the opposite of what
    max_window_layers alone would give."""
    raw = dict(TINY["C"][0], layer_types=["sliding_attention", "sliding_attention", "full_attention", "full_attention"])
    folder = helpers.make_folder(tmp_path, raw, 12)
    rng = random.Random(61)
    toks = helpers.random_tokens(rng, 60, raw["vocab_size"])
    ref = _reference(folder, dtype, {"a": toks})
    got = _replay(folder, dtype, helpers.trace_portions(toks, [17, 2, 9, 21]), _round64(len(toks)), 4)
    assert len(got) == len(toks)
    _compare(got, ref, dtype)


def test_trace_run_program(folders, tmp_path):
    """The program itself: stdin records, done lines, .f32 files."""
    raw, seed, page = TINY["A"]
    rng = random.Random(5)
    toks = helpers.random_tokens(rng, 37, raw["vocab_size"])
    ref = _reference(folders["A"], "float32", {"a": toks})
    trace = helpers.trace_portions(toks, [11, 2, 6])
    out = tmp_path / "out"
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "64"], input=trace.lines(), text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    assert proc.stdout.split("\n")[:len(trace.records)] == [f"done {i}" for i in range(len(trace.records))]
    got = {}
    for rec, rows in zip(trace.records, trace.rows):
        data = np.fromfile(out / f"{rec['step']}.f32", dtype="<f4").reshape(len(rows), raw["vocab_size"])
        for i, key in enumerate(rows):
            got[key] = torch.from_numpy(data[i].copy())
    _compare(got, ref, "float32")
