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


def _replay(folder, dtype, trace, max_tokens, page_size, max_running=8):
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
    return got


def _compare(got, ref, dtype):
    assert got
    worst = 0.0
    for (rid, pos), row in got.items():
        err = helpers.rel_err(row, ref[rid][pos])
        worst = max(worst, err)
        assert err < TOL[dtype], f"request {rid} position {pos}: error {err:.3e} (first wrong place)"
    return worst


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
