"""The decode-attention entry point that allocates nothing, called through its exported C
symbol as a caller without an allocator would call it.

Some hosts cannot allocate device memory once they run (all of it was given to an arena
at start-up, or the loop may not take the allocator's lock), so
``pb_paged_attention_decode_noalloc`` keeps the scratch for the per-split partial
results in a fixed array inside the library.  This test calls it twice in a row, with
different sizes, so that whatever the first call left in the shared array would show in
the second, and compares both results with the entry point that takes the caller's
scratch: the two run the same kernels on the same inputs and merge the splits in a fixed
order, so the results must be equal bit for bit.  The device's free memory, as the driver
reports it, must not move across the second call (the first may look up the array's address).
It also checks that a problem beyond the array's size is refused.

The file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from pulsar_b200.csrc.build import build
    lib = ctypes.CDLL(build())
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.pb_paged_attention_decode_noalloc.argtypes = [I, P, P, P, P, P, I, P, I, I, I, I, I, F, I, I, P]
    lib.pb_paged_attention_decode_noalloc.restype = ctypes.c_int
    lib.pb_decode_noalloc_max_floats.restype = ctypes.c_longlong
    lib.pb_decode_scratch_floats.argtypes = [I, I, I, I]
    lib.pb_decode_scratch_floats.restype = ctypes.c_longlong
    return lib


def _case(seed, n_seqs, hq, hkv, d, page, dtype, max_ctx):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, max_ctx + 1, (n_seqs,), generator=g)
    lens[0] = max_ctx
    width = -(-max_ctx // page)
    n_pages = n_seqs * width + 2
    perm = torch.randperm(n_pages, generator=g)[: n_seqs * width].view(n_seqs, width).to(torch.int32)
    q = torch.randn(n_seqs, hq, d, generator=g).to(dtype).cuda()
    kp = torch.randn(n_pages, hkv, page, d, generator=g).to(dtype).cuda()
    vp = torch.randn(n_pages, hkv, page, d, generator=g).to(dtype).cuda()
    return q, kp, vp, perm.cuda(), lens.to(torch.int32).cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_matches_existing_entry_twice_in_a_row(dtype):
    from pulsar_b200 import ops
    lib = _library()
    code = ops.code(dtype)
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row; the second is smaller, so stale partials of the first lie beside its own
    for seed, (n_seqs, hq, hkv, d, page, max_ctx, n_splits, window) in enumerate(
            [(5, 8, 2, 64, 16, 300, 6, 0), (3, 6, 3, 32, 8, 90, 3, 40)]):
        q, kp, vp, table, lens = _case(seed, n_seqs, hq, hkv, d, page, dtype, max_ctx)
        scale = 1.0 / math.sqrt(d)
        want = torch.empty_like(q)
        partial = torch.empty(lib.pb_decode_scratch_floats(n_seqs, hq, d, n_splits), dtype=torch.float32, device="cuda")
        ops.paged_attention_decode(q, kp, vp, want, partial, table, lens, scale, window or None, n_splits,
                                   tensor_cores=False)     # the entry point this one is a variant of
        got = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]          # the driver's count: a cudaMalloc inside the library would show
        rc = lib.pb_paged_attention_decode_noalloc(code, q.data_ptr(), kp.data_ptr(), vp.data_ptr(), got.data_ptr(),
                                                   table.data_ptr(), table.shape[1], lens.data_ptr(), n_seqs, hq, hkv, d,
                                                   page, scale, window, n_splits, stream)
        assert rc == 0, f"status {rc}"
        torch.cuda.synchronize()
        if seed > 0:                                        # the first call on a device may look up the symbol's address
            assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want), (f"call {seed}: the entry point and its variant with the caller's scratch differ by "
                                        f"{float((got.double() - want.double()).abs().max()):.3e}")


def test_no_alloc_entry_refuses_what_does_not_fit():
    lib = _library()
    limit = lib.pb_decode_noalloc_max_floats()
    assert limit == 1 << 20
    n_seqs, hq, d, n_splits = 64, 64, 256, 64            # 64*64*64*258 floats: far beyond the array
    assert lib.pb_decode_scratch_floats(n_seqs, hq, d, n_splits) > limit
    q = torch.zeros(1, device="cuda")
    rc = lib.pb_paged_attention_decode_noalloc(0, q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), 1,
                                               q.data_ptr(), n_seqs, hq, 8, d, 16, 1.0, 0, n_splits,
                                               torch.cuda.current_stream().cuda_stream)
    assert rc == -5          # PB_ERR_SCRATCH_TOO_SMALL: refused before anything was launched
    torch.cuda.synchronize()
