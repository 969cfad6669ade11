"""The debug build (PULSAR_CHECK_BOUNDS=1): kernels check the page ids and slots they take from index arrays.

The checks run in a process of their own, because the flag chooses the library when it is built and loaded.  The
bad indices of the test lie outside the pool that the kernels are given and inside the tensor that was allocated,
so that even an unchecked access would touch this test's own memory only; that memory holds NaN, so a read that was
not skipped would show in the result."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import math, sys, torch
sys.path.insert(0, sys.argv[1])
from pulsar_b200 import ops
assert ops.bounds_checked()
torch.manual_seed(0)
hq, hkv, d, page, n_alloc, n_pool = 4, 2, 64, 16, 40, 32
scale = 1.0 / math.sqrt(d)
lens = [40, 70, 23]
for dtype in (torch.float32, torch.bfloat16):
    k_all = torch.randn(n_alloc, hkv, page, d, device="cuda").to(dtype)
    v_all = torch.randn(n_alloc, hkv, page, d, device="cuda").to(dtype)
    k_all[n_pool:] = float("nan")
    v_all[n_pool:] = float("nan")
    kp, vp = k_all[:n_pool], v_all[:n_pool]                       # the pool the kernels are given
    width = 5
    table = torch.arange(3 * width, dtype=torch.int32, device="cuda").view(3, width) + 1
    kv = torch.tensor(lens, dtype=torch.int32, device="cuda")
    q = torch.randn(3, hq, d, device="cuda").to(dtype)
    cu = torch.tensor([0, 1, 2, 3], dtype=torch.int32, device="cuda")
    seq = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
    bad = table.clone()
    bad[1, 2] = 35                                                 # outside the pool, inside the allocation
    zero = table.clone()
    zero[1, 2] = 0                                                 # what a skipped read takes instead

    def run(kind, tbl):
        out = torch.full_like(q, float("nan"))
        if kind == "generic":
            ops.paged_attention_generic(q, kp, vp, out, tbl, cu, kv, seq, scale, None)
        else:
            partial = torch.empty(3 * hq * 2 * (d + 2), device="cuda")
            ops.paged_attention_decode(q, kp, vp, out, partial, tbl, kv, scale, None, 2,
                                       tensor_cores=(kind == "decode_tc"), fused=False)
        torch.cuda.synchronize()
        return out

    kinds = ["generic", "decode"] + (["decode_tc"] if dtype == torch.bfloat16 else [])
    for kind in kinds:
        ops.clear_bounds_error()
        good = run(kind, table)
        assert ops.bounds_error() == 0 and torch.isfinite(good.float()).all(), kind
        got = run(kind, bad)
        assert ops.bounds_error() == 2, (kind, ops.bounds_error())
        assert torch.isfinite(got.float()).all(), kind             # the NaN page was not read
        ops.clear_bounds_error()
        assert torch.equal(got, run(kind, zero)), kind             # page 0 stood in for it
        assert ops.bounds_error() == 0
    # a slot outside the pool: the write is dropped, the word says so
    n = 3
    qkv = torch.randn(n, (hq + 2 * hkv) * d, device="cuda").to(dtype)
    q_out = torch.empty(n, hq, d, device="cuda", dtype=dtype)
    cos = torch.ones(n, d // 2, device="cuda")
    sin = torch.zeros(n, d // 2, device="cuda")
    before_k = kp.clone()
    slots = torch.tensor([5 * page + 1, 34 * page + 3, 7 * page], dtype=torch.int32, device="cuda")
    ops.clear_bounds_error()
    ops.qk_norm_rope_write(qkv, q_out, kp, vp, slots, cos, sin, None, None, 0.0, hq, hkv, d, d, page)
    torch.cuda.synchronize()
    assert ops.bounds_error() == 3
    assert torch.isnan(k_all[34].float()).all()                    # nothing was written beyond the pool
    changed = (kp.float() != before_k.float()).flatten(1).any(1).nonzero().flatten().tolist()
    assert changed == [5, 7], changed
    words = torch.zeros(8, dtype=torch.int32, device="cuda")
    ops.gather_wait_words(words)
    text = ops.describe_wait_words(words.tolist()[:ops.N_WAIT_WORDS])
    assert "slot outside its pool" in text, text
print("bounds checks ok")
'''


def test_debug_build_records_bad_page_ids_and_slots_and_skips_the_access():
    env = dict(os.environ, PULSAR_CHECK_BOUNDS="1")
    proc = subprocess.run([sys.executable, "-c", SCRIPT, ROOT], capture_output=True, text=True, timeout=1200, env=env)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "bounds checks ok" in proc.stdout


def test_the_ordinary_build_has_no_checks():
    from pulsar_b200 import ops
    assert not ops.bounds_checked() and ops.bounds_error() == 0
