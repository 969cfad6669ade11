"""Each CUDA kernel alone against a plain float64 reference of the same operation, at
sizes other than the engine's tiny models: widths and vocabularies that are no power of
two, head sizes in steps of 16, odd group sizes, ragged contexts, shuffled pages."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.6e-2}


def dev(t):
    return t.to("cuda")


def close(got, ref, tol, what=""):
    ref = ref.to(torch.float64)
    err = float((got.detach().cpu().to(torch.float64) - ref.cpu()).abs().max() / ref.abs().max().clamp_min(1e-30))
    assert err < tol, f"{what}: relative error {err:.3e} >= {tol}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,vocab", [(72, 301), (4096, 1000)])
def test_embed(dtype, width, vocab):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, width, generator=g).to(dtype)
    ids = torch.tensor([0, vocab - 1, 5, 5, 17], dtype=torch.int32)
    out = torch.empty(5, width, dtype=torch.float32, device="cuda")
    ops.embed(dev(table), dev(ids), out)
    assert torch.equal(out.cpu(), table.float()[ids.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 100, 4096, 5120])
def test_add_rmsnorm(dtype, width):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(1)
    n, eps = 7, 3e-6
    res = torch.randn(n, width, generator=g) * 3
    res[2] = 0.0                                  # the all-zero row that only eps keeps finite
    delta = (torch.randn(n, width, generator=g)).to(dtype)
    delta[2] = 0
    w = 1 + 0.1 * torch.randn(width, generator=g)
    x = res.double() + delta.double()
    ref = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()
    r = dev(res.clone())
    out = torch.empty(n, width, dtype=dtype, device="cuda")
    ops.add_rmsnorm(r, dev(delta), dev(w), eps, out)
    close(out, ref, TOL[dtype], "normalised")
    close(r, x, 1e-6, "residual written back")
    assert torch.isfinite(out).all() and float(out[2].abs().max()) == 0.0
    # gathered rows: residual untouched
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    r2 = dev(res.clone())
    out2 = torch.empty(3, width, dtype=dtype, device="cuda")
    ops.add_rmsnorm(r2, dev(delta), dev(w), eps, out2, rows=dev(rows))
    close(out2, ref[rows.long()], TOL[dtype], "gathered rows")
    assert torch.equal(r2.cpu(), res)
    # without delta
    out3 = torch.empty(n, width, dtype=dtype, device="cuda")
    r3 = dev(res.clone())
    ops.add_rmsnorm(r3, None, dev(w), eps, out3)
    x3 = res.double()
    close(out3, x3 * torch.rsqrt((x3 * x3).mean(-1, keepdim=True) + eps) * w.double(), TOL[dtype], "no delta")


@pytest.mark.parametrize("theta,rotary", [(1e4, 16), (1e6, 128), (5e5, 48)])
def test_rope_table_large_positions(theta, rotary):
    from pulsar_b200 import ops
    pos = torch.tensor([0, 1, 2, 17, 4095, 32767, 131071, 1000003], dtype=torch.int32)
    half = rotary // 2
    inv = torch.tensor([theta ** (-2.0 * j / rotary) for j in range(half)], dtype=torch.float64)
    ang = pos.double()[:, None] * inv[None, :]
    cos = torch.empty(len(pos), half, dtype=torch.float32, device="cuda")
    sin = torch.empty_like(cos)
    ops.rope_table(dev(pos), dev(inv * (2.0 / math.pi)), cos, sin)
    assert float((cos.cpu().double() - torch.cos(ang)).abs().max()) < 1e-6
    assert float((sin.cpu().double() - torch.sin(ang)).abs().max()) < 1e-6


def _rope_ref(x, pos, theta, rotary):
    d = x.shape[-1]
    half = rotary // 2
    inv = torch.tensor([theta ** (-2.0 * j / rotary) for j in range(half)], dtype=torch.float64)
    ang = pos.double()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:rotary]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., rotary:]], dim=-1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,rotary,page,norm", [(4, 2, 16, 16, 16, True), (6, 3, 48, 48, 4, True),
                                                       (5, 5, 80, 32, 8, False), (32, 8, 128, 128, 16, True),
                                                       (3, 0, 32, 32, 8, True)])
def test_qk_norm_rope_write(dtype, hq, hkv, d, rotary, page, norm):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(2)
    n, pages, theta, eps = 11, 9, 1e5, 1e-5
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=g).to(dtype)
    pos = torch.randint(0, 5000, (n,), generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * page, generator=g)[:n].to(torch.int32)
    slots[4] = -1                                                 # a token whose k/v is not stored
    qw = (1 + 0.1 * torch.randn(d, generator=g)) if norm else None
    kw = (1 + 0.1 * torch.randn(d, generator=g)) if norm else None
    half = rotary // 2
    inv = torch.tensor([theta ** (-2.0 * j / rotary) for j in range(half)], dtype=torch.float64)
    cos = torch.empty(n, half, dtype=torch.float32, device="cuda")
    sin = torch.empty_like(cos)
    ops.rope_table(dev(pos), dev(inv * (2.0 / math.pi)), cos, sin)
    q_out = torch.empty(n, hq, d, dtype=dtype, device="cuda")
    kp = torch.full((pages, max(hkv, 1), page, d), 7.0, dtype=dtype, device="cuda") if hkv else None
    vp = torch.full((pages, max(hkv, 1), page, d), 7.0, dtype=dtype, device="cuda") if hkv else None
    ops.qk_norm_rope_write(dev(qkv), q_out, kp, vp, dev(slots) if hkv else None, cos, sin,
                           dev(qw) if norm else None, dev(kw) if norm else None, eps, hq, hkv, d, rotary, page)
    x = qkv.double()
    q = x[:, :hq * d].view(n, hq, d)

    def normed(t, w):
        if w is None:
            return t
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w.double()
    close(q_out, _rope_ref(normed(q, qw), pos, theta, rotary), TOL[dtype], "q")
    if hkv:
        k = x[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
        v = x[:, (hq + hkv) * d:].view(n, hkv, d)
        k_ref = _rope_ref(normed(k, kw), pos, theta, rotary)
        kc, vc = kp.cpu().double(), vp.cpu().double()
        untouched = torch.ones(pages * page, dtype=torch.bool)
        for t in range(n):
            sl = int(slots[t])
            if sl < 0:
                continue
            untouched[sl] = False
            close(kc[sl // page, :, sl % page, :], k_ref[t], TOL[dtype], f"k of token {t}")
            assert torch.equal(vc[sl // page, :, sl % page, :], v[t]), "v is a plain copy"
        flat = kc.permute(0, 2, 1, 3).reshape(pages * page, -1)
        assert bool((flat[untouched] == 7.0).all()), "slots that were not addressed stay untouched"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [24, 176, 12288])
def test_silu_mul(dtype, inter):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(5, 2 * inter, generator=g) * 3).to(dtype)
    out = torch.empty(5, inter, dtype=dtype, device="cuda")
    ops.silu_mul(dev(gu), out)
    a, b = gu.double()[:, :inter], gu.double()[:, inter:]
    close(out, a * torch.sigmoid(a) * b, TOL[dtype])


@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (3, 130, 70), (65, 64, 33), (128, 301, 96), (200, 512, 1000)])
def test_gemm_simt_is_true_float32(m, n, k):
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(4)
    a, w = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g)
    out = torch.empty(m, n, dtype=torch.float32, device="cuda")
    ops.gemm_simt(dev(a), dev(w), out)
    close(out, a.double() @ w.double().T, 2e-6 * max(1, k / 64) ** 0.5)
    # rows do not depend on which other rows are in the batch: bit-equal
    if m > 2:
        out2 = torch.empty(2, n, dtype=torch.float32, device="cuda")
        ops.gemm_simt(dev(a[m - 2:].contiguous()), dev(w), out2)
        assert torch.equal(out2, out[m - 2:])


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(48, 96), (4096, 4096), (1024, 12288), (304, 160), (64, 2048), (32, 1536), (48, 832), (640, 5120)])
def test_gemm_skinny(m, n, k):
    """The weight-streaming product for a few tokens against float64, plain and with the
    SwiGLU epilogue, float32 and bfloat16 outputs; one weight made large so that a wrong
    k-permutation of the fragments would show.  The widths decide which paths a warp takes: 8, 24 or 10
    blocks of 64 per warp (register batches, the part prefetched through shared memory, the rest), 4 or 3
    (too few for the prefetch or for what follows it), 13 blocks over 8 warps (uneven), and widths that are
    no multiple of 64 (16-byte loads)."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(13)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).bfloat16()
    w[n // 3, (5 * k) // 7] = 3.0
    ref = a.double() @ w.double().T
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
        assert ops.gemm_skinny(dev(a), dev(w), out)
        close(out, ref, tol, f"plain {dt}")
    inter = n // 2
    gate, up = ref[:, :inter], ref[:, inter:]
    act = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.gemm_skinny(dev(a), dev(w), act, swiglu=True)
    close(act, gate * torch.sigmoid(gate) * up, 1e-2, "swiglu")


@pytest.mark.parametrize("m", [9, 12, 16])
@pytest.mark.parametrize("n,k", [(9536, 256), (19072, 192), (24576, 512)])
def test_gemm_skinny_with_32_rows_per_block(m, n, k):
    """9 to 16 tokens against weights with many tiles: blocks of two row groups (and, with PULSAR_SKINNY_TALL=0 in the
    environment, the blocks of 16 rows), plain and with the SwiGLU epilogue, against float64; one large weight in each
    row group's range, a width of three k-blocks over eight warps (warps without work)."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(19)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).bfloat16()
    w[n // 3, (5 * k) // 7] = 3.0
    w[n // 3 + 16, k // 9] = -3.0
    w[n - 1, k - 1] = 2.5
    ref = a.double() @ w.double().T
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
        assert ops.gemm_skinny(dev(a), dev(w), out)
        close(out, ref, tol, f"plain {dt}")
    inter = n // 2
    gate, up = ref[:, :inter], ref[:, inter:]
    act = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.gemm_skinny(dev(a), dev(w), act, swiglu=True)
    close(act, gate * torch.sigmoid(gate) * up, 1e-2, "swiglu")


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(96, 192), (4096, 4096), (1024, 12288), (64, 2048), (192, 832), (640, 5120)])
def test_gemm_skinny_adds_into_the_residual_and_prepares_the_norm_that_follows(m, n, k):
    """The product that adds its result to the float32 residual stream in place and prepares the RMSNorm behind it
    (residual * norm weight in bfloat16, the blocks' parts of the rows' sums of squares), and the product that
    takes tokens prepared so and scales each token's sums, plain and with the SwiGLU epilogue, against float64.
    One residual row is all zero (only eps keeps it finite), one is large, so that the per-token factor shows."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(17)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).bfloat16()
    w[n // 3, (5 * k) // 7] = 3.0
    res = torch.randn(m, n, generator=g) * 2.0
    res[m // 2] *= 40.0
    delta = a.double() @ w.double().T
    if m > 2:
        res[1] = 0.0
        a[1] = 0.0
        delta[1] = 0.0
    want_res = res.double() + delta
    res_dev = dev(res.clone())
    assert ops.fused_projection_supported(m, dev(w))
    assert ops.linear_accumulate(dev(a), dev(w), res_dev)
    close(res_dev, want_res, 2e-5, "accumulate")
    # once more, now preparing the norm that follows: it adds, it does not overwrite
    nw = 1.0 + 0.1 * torch.randn(n, generator=g)
    eps = 3e-6
    prepared = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    parts = torch.full((ops.norm_parts_numel(m, n),), float("nan"), dtype=torch.float32, device="cuda")
    assert ops.linear_accumulate(dev(a), dev(w), res_dev, dev(nw), prepared, parts)
    x = res.double() + 2 * delta
    close(res_dev, x, 2e-5, "accumulate twice")
    close(prepared, x * nw.double(), 1e-2, "prepared operand")
    close(parts[:(n // 16) * m].view(n // 16, m).sum(0), (x ** 2).sum(-1), 2e-5, "parts of the sums of squares")
    tagged = parts[(n // 16) * m:].view(torch.int32).view(m, 2)          # per row: the sum's bits, the tag
    assert int(tagged[:, 1].abs().sum()) == 0                # "the sums are not there yet"
    # the product behind the norm: rows of W2 [n2, n]
    n2 = 256
    w2 = (torch.randn(n2, n, generator=g) / n ** 0.5).bfloat16()
    exact = (x * torch.rsqrt((x ** 2).mean(-1, keepdim=True) + eps) * nw.double()) @ w2.double().T
    out = torch.full((m, n2), float("nan"), dtype=torch.bfloat16, device="cuda")
    if n % 64 == 0:
        assert ops.linear_prenormed(prepared, parts, eps, dev(w2), out)
        close(out, exact, 1.6e-2, "product behind the prepared norm")
        # its block 0 has left the sums behind the parts, each with its tag; the producing product takes the tags back
        assert bool((tagged[:, 1] == 1).all())
        close(tagged[:, 0].contiguous().view(torch.float32), (x ** 2).sum(-1), 2e-5, "sums of squares")
        if m > 2:
            assert float(out[1].float().abs().max()) == 0.0
        # the same bits on the path on which every block adds the parts itself (block 0 keeps its sums to itself)
        tagged.zero_()
        ops.fn("pb_gemm_skinny_publish_sums")(0)
        try:
            again = torch.full((m, n2), float("nan"), dtype=torch.bfloat16, device="cuda")
            assert ops.linear_prenormed(prepared, parts, eps, dev(w2), again)
            assert int(tagged[:, 1].abs().sum()) == 0 and torch.equal(again, out)
        finally:
            ops.fn("pb_gemm_skinny_publish_sums")(1)
        act = torch.full((m, n2 // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert ops.linear_prenormed(prepared, parts, eps, dev(w2), act, swiglu=True)
        gate, up = exact[:, :n2 // 2], exact[:, n2 // 2:]
        close(act, gate * torch.sigmoid(gate) * up, 2e-2, "the same with the SwiGLU epilogue")
    else:
        assert not ops.linear_prenormed(prepared, parts, eps, dev(w2), out)


def test_fused_projections_decline_other_sizes():
    from pulsar_b200 import ops
    w = torch.zeros(32, 96, dtype=torch.bfloat16, device="cuda")                  # K no multiple of 64
    assert not ops.fused_projection_supported(4, w)
    assert not ops.linear_accumulate(torch.zeros(4, 96, dtype=torch.bfloat16, device="cuda"), w, torch.zeros(4, 32, device="cuda"))
    w = torch.zeros(32, 128, dtype=torch.bfloat16, device="cuda")
    assert not ops.fused_projection_supported(17, w)                              # too many tokens
    assert not ops.linear_accumulate(torch.zeros(17, 128, dtype=torch.bfloat16, device="cuda"), w, torch.zeros(17, 32, device="cuda"))
    assert ops.fused_projection_supported(16, w)


def test_gemm_skinny_declines_other_sizes():
    from pulsar_b200 import ops
    a = torch.zeros(17, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device="cuda")
    assert not ops.gemm_skinny(a, w, torch.empty(17, 32, dtype=torch.bfloat16, device="cuda"))          # too many rows
    assert not ops.gemm_skinny(a[:4, :48].contiguous(), w[:, :48].contiguous(), torch.empty(4, 32, dtype=torch.bfloat16, device="cuda"))
    assert not ops.gemm_skinny(a[:4], w[:24], torch.empty(4, 24, dtype=torch.bfloat16, device="cuda"))  # rows no multiple of 16
    out = torch.empty(17, 32, dtype=torch.bfloat16, device="cuda")
    ops.linear(a, w, out)                                                                              # falls to the library product
    assert float(out.abs().max()) == 0.0


@pytest.mark.parametrize("m", [17, 33, 64, 100, 128])
@pytest.mark.parametrize("n,k", [(256, 64), (4096, 4096), (1024, 12288), (6144, 4096), (264, 200), (24576, 512), (1000, 1536),
                                 (48, 8192)])
def test_gemm_tcgen05_stream(m, n, k):
    """The weight-streaming tcgen05 product for 17 to 128 tokens against float64: tiles that hang over the rows of W
    and the tail of K, several slices of K whose partial sums meet in the workspace (few tiles) and whole tiles (many),
    float32 and bfloat16 outputs, the SwiGLU epilogue; weights made large in places so that a wrong swizzle,
    descriptor or owner of a column would show."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(15)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).bfloat16()
    w[n // 3, (5 * k) // 7] = 3.0
    w[n - 1, k - 1] = -2.0
    a[m - 1, k - 1] = 4.0
    ref = a.double() @ w.double().T
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
        assert ops.gemm_tcgen05_stream(dev(a), dev(w), out)
        close(out, ref, tol, f"plain {dt}")
    inter = n // 2
    gate, up = ref[:, :inter], ref[:, inter:]
    act = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.gemm_tcgen05_stream(dev(a), dev(w), act, swiglu=True)
    close(act, gate * torch.sigmoid(gate) * up, 1e-2, "swiglu")
    ops.check_wait_words()


@pytest.mark.parametrize("m,n,k", [(17, 256, 64), (128, 512, 128), (100, 320, 72), (300, 1000, 4096), (2048, 1024, 512),
                                   (129, 264, 200)])
def test_gemm_tcgen05(m, n, k):
    """The tcgen05 / TMA product against float64: tiles that hang over every edge (rows of x,
    rows of W, the tail of K), float32 and bfloat16 outputs, the SwiGLU epilogue; one weight made
    large so that a wrong swizzle or descriptor would show."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(14)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).bfloat16()
    w[n // 3, (5 * k) // 7] = 3.0
    w[n - 1, k - 1] = -2.0
    ref = a.double() @ w.double().T
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
        assert ops.gemm_tcgen05(dev(a), dev(w), out)
        close(out, ref, tol, f"plain {dt}")
    inter = n // 2
    gate, up = ref[:, :inter], ref[:, inter:]
    act = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.gemm_tcgen05(dev(a), dev(w), act, swiglu=True)
    close(act, gate * torch.sigmoid(gate) * up, 1e-2, "swiglu")
    assert ops.gemm_tcgen05_error() == 0
    assert not ops.gemm_tcgen05(dev(a[:, :k - 4].contiguous()), dev(w[:, :k - 4].contiguous()),
                                torch.empty(m, n, dtype=torch.bfloat16, device="cuda"))      # K no multiple of 8


def test_gemm_simt_mixed_dtypes():
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(5)
    a, w = torch.randn(9, 100, generator=g).bfloat16(), torch.randn(37, 100, generator=g).bfloat16()
    out = torch.empty(9, 37, dtype=torch.float32, device="cuda")
    ops.gemm_simt(dev(a), dev(w), out)
    close(out, a.double() @ w.double().T, 1e-5)


# ------------------------------------------------------------------ attention
def _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype, spike=None):
    """Random q and a shuffled paged cache for sequences with the given new / total lengths."""
    s = len(lens_q)
    n = sum(lens_q)
    pages_per = [-(-kv // page) for kv in lens_kv]
    total_pages = sum(pages_per) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    width = max(pages_per)
    table = torch.full((s, width), -1, dtype=torch.int32)
    k_seq = [torch.randn(kv, hkv, d, generator=g) for kv in lens_kv]
    v_seq = [torch.randn(kv, hkv, d, generator=g) for kv in lens_kv]
    q = torch.randn(n, hq, d, generator=g)
    if spike is not None:                 # one far key stands out: a kernel that loses it shows
        si, key, head = spike
        qrow = sum(lens_q[:si]) + lens_q[si] - 1
        k_seq[si][key, head // (hq // hkv)] = q[qrow, head] * 6.0
        v_seq[si][key, head // (hq // hkv)] = 50.0
    kp = torch.zeros(total_pages, hkv, page, d)
    vp = torch.zeros(total_pages, hkv, page, d)
    at = 0
    for i in range(s):
        for lp in range(pages_per[i]):
            pg = perm[at]
            at += 1
            table[i, lp] = pg
            lo, hi = lp * page, min(lens_kv[i], (lp + 1) * page)
            kp[pg, :, :hi - lo] = k_seq[i][lo:hi].permute(1, 0, 2)
            vp[pg, :, :hi - lo] = v_seq[i][lo:hi].permute(1, 0, 2)
    cu = [0]
    for ql in lens_q:
        cu.append(cu[-1] + ql)
    seq_of = [i for i, ql in enumerate(lens_q) for _ in range(ql)]
    q, kp, vp = q.to(dtype), kp.to(dtype), vp.to(dtype)
    k_seq = [k.to(dtype).double() for k in k_seq]
    v_seq = [v.to(dtype).double() for v in v_seq]
    return dict(q=q, kp=kp, vp=vp, table=table, cu=torch.tensor(cu, dtype=torch.int32),
                kv=torch.tensor(lens_kv, dtype=torch.int32), seq_of=torch.tensor(seq_of, dtype=torch.int32),
                k_seq=k_seq, v_seq=v_seq)


def _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, window):
    q = case["q"].double()
    out = torch.zeros_like(q)
    row = 0
    for i, (ql, kv) in enumerate(zip(lens_q, lens_kv)):
        for t in range(ql):
            p = kv - ql + t
            lo = max(0, p - window + 1) if window else 0
            for h in range(hq):
                g = h // (hq // hkv)
                sc = (case["k_seq"][i][lo:p + 1, g] @ q[row, h]) * scale
                out[row, h] = torch.softmax(sc, 0) @ case["v_seq"][i][lo:p + 1, g]
            row += 1
    return out


ATTN_SHAPES = [  # hq, hkv, d, page
    (4, 2, 16, 16), (8, 2, 32, 8), (6, 3, 48, 4), (5, 5, 64, 16), (32, 8, 128, 16), (14, 2, 96, 32), (3, 1, 256, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", ATTN_SHAPES)
@pytest.mark.parametrize("window", [None, 37])
def test_attention_generic_mixed_batch(dtype, hq, hkv, d, page, window):
    """First portions, later portions and single tokens in one ragged batch
    (the (new, total) pairs of pulsar/tests/test_paged_prefill.py:45-50 and more)."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(6)
    lens_q = [16, 7, 33, 1, 1, 2, 64]
    lens_kv = [16, 40, 33, 65, 1, 129, 100]
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype, spike=(5, 3, hq - 1))
    out = torch.empty(sum(lens_q), hq, d, dtype=dtype, device="cuda")
    scale = 1.0 / math.sqrt(d)
    ops.paged_attention_generic(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, dev(case["table"]), dev(case["cu"]),
                                dev(case["kv"]), dev(case["seq_of"]), scale, window)
    close(out, _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, window), TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", ATTN_SHAPES)
@pytest.mark.parametrize("window", [None, 50])
@pytest.mark.parametrize("n_splits", [1, 3, 8, 64])
def test_attention_decode_split(dtype, hq, hkv, d, page, window, n_splits):
    """Ragged contexts of pulsar/tests/test_paged_attention.py:21-45, forced split counts
    (empty splits included), one far key made to stand out."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(7)
    lens_kv = [1, 7, 16, 33, 40, 65, 100, 129, 700]
    lens_q = [1] * len(lens_kv)
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype, spike=(8, 5, 0))
    out = torch.empty(len(lens_kv), hq, d, dtype=dtype, device="cuda")
    partial = torch.empty(len(lens_kv) * hq * n_splits * (d + 2), dtype=torch.float32, device="cuda")
    scale = 1.0 / math.sqrt(d)
    ops.paged_attention_decode(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, partial, dev(case["table"]),
                               dev(case["kv"]), scale, window, n_splits)
    close(out, _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, window), TOL[dtype])


TC_SHAPES = [(32, 8, 128, 16), (5, 5, 64, 16), (16, 1, 128, 32), (8, 2, 64, 8), (12, 4, 128, 64), (7, 7, 128, 4),
             (10, 2, 128, 16)]


@pytest.mark.parametrize("hq,hkv,d,page", TC_SHAPES)
@pytest.mark.parametrize("window", [None, 50, 333])
@pytest.mark.parametrize("n_splits", [1, 2, 5, 37])
def test_attention_decode_tensor_cores(hq, hkv, d, page, window, n_splits):
    """The tensor-core decode kernel against the plain reference and against the CUDA-core
    kernel it stands in for: ragged contexts, tile and page edges (63, 64, 65, 128, 129),
    windows that start inside a tile, more splits than tiles."""
    from pulsar_b200 import ops
    dtype = torch.bfloat16
    assert ops.decode_tc_supported(dtype, hq, hkv, d, page)
    g = torch.Generator().manual_seed(11)
    lens_kv = [1, 15, 16, 17, 63, 64, 65, 128, 129, 700, 1025]
    lens_q = [1] * len(lens_kv)
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype, spike=(9, 5, hq - 1))
    scale = 1.0 / math.sqrt(d)
    outs = []
    for tc, fused in ((True, True), (True, False), (False, False), (True, True)):      # fused twice: its tickets reset themselves
        out = torch.full((len(lens_kv), hq, d), float("nan"), dtype=dtype, device="cuda")
        partial = torch.full((len(lens_kv) * hq * n_splits * (d + 2),), float("nan"), dtype=torch.float32, device="cuda")
        ops.paged_attention_decode(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, partial, dev(case["table"]),
                                   dev(case["kv"]), scale, window, n_splits, tensor_cores=tc, fused=fused)
        outs.append(out)
    ref = _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, window)
    close(outs[0], ref, TOL[dtype], "tensor cores, merged in the kernel, vs plain")
    close(outs[1], ref, TOL[dtype], "tensor cores + combine kernel vs plain")
    close(outs[0], outs[2].double(), TOL[dtype], "tensor cores vs CUDA cores")
    assert torch.equal(outs[0], outs[3]), "second fused launch on the same tickets"


@pytest.mark.parametrize("hq,hkv,d,page", TC_SHAPES)
@pytest.mark.parametrize("window", [None, 50])
@pytest.mark.parametrize("n_splits,with_norm", [(1, True), (3, True), (37, False)])
def test_attention_decode_from_the_projected_rows(hq, hkv, d, page, window, n_splits, with_norm):
    """The decode kernel that takes the step's raw q/k/v rows (per-head norm, rotation and the cache write of the
    newest key and value inside it) against the two kernels it stands in for: same pools afterwards (values bit
    for bit, keys up to the order of the sum of squares), same output; contexts of one key (only the newest), at
    tile and page edges; a wrong value left in the newest slot beforehand shows that the kernel reads what it wrote."""
    from pulsar_b200 import ops
    dtype = torch.bfloat16
    assert ops.decode_qkv_supported(dtype, hq, hkv, d, d, page)
    g = torch.Generator().manual_seed(12)
    lens_kv = [1, 15, 16, 17, 63, 64, 65, 128, 129, 700, 1025]
    s = len(lens_kv)
    lens_q = [1] * s
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype)
    scale = 1.0 / math.sqrt(d)
    qkv = (torch.randn(s, (hq + 2 * hkv) * d, generator=g) * 1.5).to(dtype)
    qw = (1.0 + 0.2 * torch.randn(d, generator=g)) if with_norm else None
    kw = (1.0 + 0.2 * torch.randn(d, generator=g)) if with_norm else None
    ang = torch.rand(s, d // 2, generator=g, dtype=torch.float64) * 6.28
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    # slot of the newest position of every sequence; what lies there now must not be read
    table = case["table"]
    slots = torch.tensor([int(table[i, (kv - 1) // page]) * page + (kv - 1) % page for i, kv in enumerate(lens_kv)], dtype=torch.int32)
    kp, vp = case["kp"].clone(), case["vp"].clone()
    for i, sl in enumerate(slots.tolist()):
        kp[sl // page, :, sl % page] = 77.0
        vp[sl // page, :, sl % page] = -55.0
    eps = 1e-5
    # the two kernels
    kp_a, vp_a = dev(kp), dev(vp)
    q_a = torch.empty(s, hq, d, dtype=dtype, device="cuda")
    ops.qk_norm_rope_write(dev(qkv), q_a, kp_a, vp_a, dev(slots), dev(cos), dev(sin), dev(qw) if with_norm else None,
                           dev(kw) if with_norm else None, eps, hq, hkv, d, d, page)
    out_a = torch.empty(s, hq, d, dtype=dtype, device="cuda")
    partial = torch.empty(s * hq * n_splits * (d + 2), dtype=torch.float32, device="cuda")
    ops.paged_attention_decode(q_a, kp_a, vp_a, out_a, partial, dev(table), dev(case["kv"]), scale, window, n_splits, tensor_cores=True)
    # the one kernel, merged by the combine kernel and merged in the kernel
    for fused in (False, True):
        kp_b, vp_b = dev(kp), dev(vp)
        out_b = torch.full((s, hq, d), float("nan"), dtype=dtype, device="cuda")
        partial.fill_(float("nan"))
        ops.paged_attention_decode_qkv(dev(qkv), dev(qw) if with_norm else None, dev(kw) if with_norm else None, dev(cos), dev(sin),
                                       eps, dev(slots), kp_b, vp_b, out_b, partial, dev(table), dev(case["kv"]), scale, window,
                                       n_splits, fused=fused)
        assert torch.equal(vp_b, vp_a), "values in the pool"
        close(kp_b, kp_a.double(), 1e-2, "keys in the pool")
        close(out_b, out_a.double(), TOL[dtype], f"output, merged in the kernel: {fused}")
    ops.check_wait_words()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_splits", [1, 3])
def test_attention_decode_of_a_sequence_without_keys_gives_zeros(dtype, n_splits):
    """The exported entry points take kv_len 0 (the engine never sends it): every split of such a sequence is empty,
    and the merge must give zeros, not 0 * inf; its neighbours in the batch are untouched by it."""
    from pulsar_b200 import ops
    hq, hkv, d, page = 8, 2, 64, 16
    g = torch.Generator().manual_seed(4)
    lens_kv = [40, 1, 90]
    case = _paged_case(g, [1, 1, 1], lens_kv, hq, hkv, d, page, dtype)
    scale = 1.0 / math.sqrt(d)
    ref = _attention_ref(case, [1, 1, 1], lens_kv, hq, hkv, scale, None)
    kv = case["kv"].clone()
    kv[1] = 0
    variants = [(False, False)] + ([(True, True), (True, False)] if dtype == torch.bfloat16 else [])
    for tc, fused in variants:
        out = torch.full((3, hq, d), float("nan"), dtype=dtype, device="cuda")
        partial = torch.full((3 * hq * n_splits * (d + 2),), float("nan"), dtype=torch.float32, device="cuda")
        ops.paged_attention_decode(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, partial, dev(case["table"]),
                                   dev(kv), scale, None, n_splits, tensor_cores=tc, fused=fused)
        assert float(out[1].float().abs().max()) == 0.0, (tc, fused)
        close(out[[0, 2]], ref[[0, 2]], TOL[dtype], f"neighbours of the empty sequence, tensor cores {tc}, fused {fused}")


@pytest.mark.parametrize("hq,hkv,d,page", TC_SHAPES)
@pytest.mark.parametrize("window", [None, 37, 200])
def test_attention_prefill_tensor_cores(hq, hkv, d, page, window):
    """Ragged batch: first portions, later portions that start inside a page and a tile,
    single tokens, lengths around the 64-row tile (63, 64, 65, 130), one far key that stands out."""
    from pulsar_b200 import ops
    dtype = torch.bfloat16
    assert ops.prefill_tc_supported(dtype, hq, hkv, d, page)
    g = torch.Generator().manual_seed(12)
    lens_q = [16, 7, 33, 1, 1, 2, 64, 63, 65, 130, 5]
    lens_kv = [16, 40, 33, 65, 1, 129, 100, 63, 300, 130, 517]
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype, spike=(10, 3, hq - 1))
    out = torch.full((sum(lens_q), hq, d), float("nan"), dtype=dtype, device="cuda")
    scale = 1.0 / math.sqrt(d)
    ops.paged_attention_prefill_tc(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, dev(case["table"]),
                                   dev(case["cu"]), dev(case["kv"]), ops.prefill_tc_tiles(lens_q), scale, window)
    close(out, _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, window), TOL[dtype])


TCGEN05_ATTN_SHAPES = [(32, 8, 128, 16), (16, 1, 128, 32), (12, 4, 128, 64), (7, 7, 128, 8), (6, 3, 128, 128), (4, 2, 128, 256),
                       (10, 2, 128, 16)]


@pytest.mark.parametrize("hq,hkv,d,page", TCGEN05_ATTN_SHAPES)
@pytest.mark.parametrize("window", [None, 37, 200])
def test_attention_prefill_tcgen05(hq, hkv, d, page, window):
    """The tcgen05 prefill kernel on a ragged batch: first portions, later portions that start inside
    a page and a tile, single tokens, lengths around the 128-row tile (127, 128, 129, 300), a context of
    several key tiles, one far key that stands out; pool rows that no sequence owns hold zeros."""
    from pulsar_b200 import ops
    dtype = torch.bfloat16
    assert ops.prefill_tcgen05_supported(dtype, hq, hkv, d, page)
    g = torch.Generator().manual_seed(13)
    lens_q = [16, 7, 33, 1, 1, 2, 128, 127, 129, 300, 5]
    lens_kv = [16, 40, 33, 65, 1, 129, 200, 127, 400, 300, 517]
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype, spike=(10, 3, hq - 1))
    out = torch.full((sum(lens_q), hq, d), float("nan"), dtype=dtype, device="cuda")
    scale = 1.0 / math.sqrt(d)
    ops.paged_attention_prefill_tcgen05(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, dev(case["table"]),
                                        dev(case["cu"]), dev(case["kv"]), ops.prefill_tcgen05_tiles(lens_q), scale, window)
    assert ops.prefill_tcgen05_error() == 0
    close(out, _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, window), TOL[dtype])


def test_attention_prefill_tcgen05_growing_scores():
    """Scores that grow along the keys force the running maximum to move again and again (the output
    in tensor memory is rescaled each time); scores that fall never move it after the first tile."""
    from pulsar_b200 import ops
    dtype, hq, hkv, d, page = torch.bfloat16, 4, 2, 128, 16
    g = torch.Generator().manual_seed(14)
    lens_q, lens_kv = [520, 260], [520, 700]
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype)
    # key j of sequence 0 gets a component along a fixed direction that grows with j; sequence 1: falls
    direction = torch.randn(d, generator=g)
    direction /= direction.norm()
    q = case["q"].float()
    q += 4.0 * direction
    case["q"] = q.to(dtype)
    kp = case["kp"].float()
    for si, sign in ((0, 1.0), (1, -1.0)):
        ramp = sign * torch.arange(lens_kv[si]).float() * 0.25
        case["k_seq"][si] = (case["k_seq"][si].float() + ramp[:, None, None] * direction).to(dtype).double()
        for lp in range(-(-lens_kv[si] // page)):
            pg = int(case["table"][si, lp])
            lo, hi = lp * page, min(lens_kv[si], (lp + 1) * page)
            kp[pg, :, :hi - lo] = case["k_seq"][si][lo:hi].permute(1, 0, 2).float()
    case["kp"] = kp.to(dtype)
    out = torch.full((sum(lens_q), hq, d), float("nan"), dtype=dtype, device="cuda")
    scale = 1.0 / math.sqrt(d)
    ops.paged_attention_prefill_tcgen05(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, dev(case["table"]),
                                        dev(case["cu"]), dev(case["kv"]), ops.prefill_tcgen05_tiles(lens_q), scale, None)
    assert ops.prefill_tcgen05_error() == 0
    close(out, _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, None), TOL[dtype])


@pytest.mark.parametrize("window", [None, 5000])
def test_attention_long_contexts(window):
    """Tens of thousands of cached tokens: a decoded token at 33,000 and portions that end at 20,000 and 9,000, with
    one key near the start that stands out (thousands of pages, block tables two thousand entries wide, every
    split of the decode kernels at work); all three bfloat16 kernels and the CUDA-core decode kernel."""
    from pulsar_b200 import ops
    dtype, hq, hkv, d, page = torch.bfloat16, 4, 2, 128, 16
    scale = 1.0 / math.sqrt(d)
    g = torch.Generator().manual_seed(21)
    lens_kv = [33000, 16385, 40]
    lens_q = [1, 1, 1]
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype, spike=(0, 29000 if window else 7, hq - 1))
    ref = _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, window)
    for tc in (True, False):
        for n_splits in (32, 7):
            out = torch.full((3, hq, d), float("nan"), dtype=dtype, device="cuda")
            partial = torch.full((3 * hq * n_splits * (d + 2),), float("nan"), dtype=torch.float32, device="cuda")
            ops.paged_attention_decode(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, partial, dev(case["table"]),
                                       dev(case["kv"]), scale, window, n_splits, tensor_cores=tc)
            close(out, ref, TOL[dtype], f"decode, tensor cores {tc}, {n_splits} splits")
    lens_q, lens_kv = [200, 130], [20000, 9000]
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype, spike=(0, 16000 if window else 11, 1))
    ref = _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, window)
    out = torch.full((sum(lens_q), hq, d), float("nan"), dtype=dtype, device="cuda")
    ops.paged_attention_prefill_tcgen05(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, dev(case["table"]),
                                        dev(case["cu"]), dev(case["kv"]), ops.prefill_tcgen05_tiles(lens_q), scale, window)
    assert ops.prefill_tcgen05_error() == 0
    close(out, ref, TOL[dtype], "tcgen05 portions")
    out = torch.full((sum(lens_q), hq, d), float("nan"), dtype=dtype, device="cuda")
    ops.paged_attention_prefill_tc(dev(case["q"]), dev(case["kp"]), dev(case["vp"]), out, dev(case["table"]),
                                   dev(case["cu"]), dev(case["kv"]), ops.prefill_tc_tiles(lens_q), scale, window)
    close(out, ref, TOL[dtype], "mma.sync portions")


@pytest.mark.parametrize("d,page", [(128, 16), (64, 8)])
def test_attention_dispatch_splits_a_mixed_step(d, page):
    """ops.attention on a step whose first sequences bring one token each (the scheduler's order): those take the
    decode kernel, the portions behind them the prefill kernel; single tokens further back stay with the portions."""
    from pulsar_b200 import ops

    class Host:
        pass

    class Ctx:
        def __init__(self, case, lens_q):
            self.host = Host()
            self.host.q_lens = list(lens_q)
            self.cu_q, self.kv_len, self.seq_of_token = dev(case["cu"]), dev(case["kv"]), dev(case["seq_of"])
            self.n_seqs, self.all_decode = len(lens_q), max(lens_q) == 1
            self._scratch = {}

        def scratch(self, tag, shape, dtype=None):
            key = (tag, tuple(shape), dtype)
            if key not in self._scratch:
                self._scratch[key] = torch.full(tuple(shape), float("nan"), dtype=dtype, device="cuda")
            return self._scratch[key]

    class View:
        pass

    dtype, hq, hkv = torch.bfloat16, 8, 2
    g = torch.Generator().manual_seed(17)
    lens_q = [1, 1, 1, 150, 1, 33, 2]
    lens_kv = [300, 17, 1, 150, 77, 260, 140]
    case = _paged_case(g, lens_q, lens_kv, hq, hkv, d, page, dtype, spike=(0, 3, hq - 1))
    view = View()
    view.k_pool, view.v_pool, view.block_table = dev(case["kp"]), dev(case["vp"]), dev(case["table"])
    scale = 1.0 / math.sqrt(d)
    for window in (None, 90):
        out = torch.full((sum(lens_q), hq, d), float("nan"), dtype=dtype, device="cuda")
        before = ops.LAUNCHES
        ops.attention(Ctx(case, lens_q), dev(case["q"]), view, out, scale, window)
        assert ops.LAUNCHES - before in (2, 3)                # decode (+ combine when the keys are split), one prefill kernel
        close(out, _attention_ref(case, lens_q, lens_kv, hq, hkv, scale, window), TOL[dtype])


def test_attention_prefill_tcgen05_applicability():
    from pulsar_b200 import ops
    assert not ops.prefill_tcgen05_supported(torch.float32, 32, 8, 128, 16)
    assert not ops.prefill_tcgen05_supported(torch.bfloat16, 32, 8, 64, 16)        # head size
    assert not ops.prefill_tcgen05_supported(torch.bfloat16, 32, 8, 128, 4)        # page below a swizzle group
    assert not ops.prefill_tcgen05_supported(torch.bfloat16, 32, 8, 128, 24)       # page no power of two
    assert not ops.prefill_tcgen05_supported(torch.bfloat16, 32, 5, 128, 16)       # groups do not divide the heads


def test_decode_tensor_cores_applicability():
    from pulsar_b200 import ops
    assert not ops.decode_tc_supported(torch.float32, 32, 8, 128, 16)
    assert not ops.decode_tc_supported(torch.bfloat16, 32, 8, 96, 16)       # head size
    assert not ops.decode_tc_supported(torch.bfloat16, 34, 2, 128, 16)      # group of 17
    assert not ops.decode_tc_supported(torch.bfloat16, 32, 8, 128, 24)      # page does not divide the tile
    q = torch.zeros(1, 4, 96, dtype=torch.bfloat16, device="cuda")
    kp = torch.zeros(2, 2, 16, 96, dtype=torch.bfloat16, device="cuda")
    z = torch.ones(1, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="unsupported size"):
        ops.paged_attention_decode(q, kp, kp, torch.empty_like(q), torch.empty(4 * 98, device="cuda"), z.view(1, 1), z, 1.0,
                                   None, 1, tensor_cores=True)


def test_attention_refuses_bad_sizes():
    from pulsar_b200 import ops
    q = torch.zeros(1, 2, 24, device="cuda")           # head size 24 is no multiple of 16
    kp = torch.zeros(1, 1, 16, 24, device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="unsupported size"):
        ops.paged_attention_generic(q, kp, kp, torch.empty_like(q), z.view(1, 1), torch.tensor([0, 1], dtype=torch.int32).cuda(),
                                    z + 1, z, 1.0, None)
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.silu_mul(torch.zeros(2, 4), torch.zeros(2, 2))


# ------------------------------------------------------------------ sampling
def test_argmax_lowest_index_on_ties():
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(6, 151936 // 8 + 3, generator=g)
    logits[1, 77] = logits[1, 9000] = 50.0
    logits[2, -1] = 60.0
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), out)
    ref = torch.argmax(logits, dim=-1)
    ref[1] = 77
    assert out.cpu().tolist() == ref.tolist()


def _survivors(row, temperature, top_k, top_p):
    import sys, os
    sys.path.insert(0, os.path.dirname(__file__))
    from plain import qwen3_plain as plain
    return plain.sample_filter(row, temperature, top_k, top_p)


@pytest.mark.parametrize("top_k,top_p", [(0, 1.0), (5, 1.0), (0, 0.7), (3, 0.9), (50, 0.3)])
def test_sample_survivors_and_inverse_cdf(top_k, top_p):
    """Logits built as log(probs) so the surviving set is known
    (pulsar-core/tests/runtime/test_sampler.cpp:56-135)."""
    from pulsar_b200 import ops
    vocab, temperature = 1000, 0.8
    g = torch.Generator().manual_seed(9)
    probs = torch.rand(vocab, generator=g).double() ** 4 + 1e-4
    probs /= probs.sum()
    logits = (torch.log(probs) * temperature).float()       # softmax(logits / T) == probs
    rows = 64
    uniform = (torch.arange(rows, dtype=torch.float32) + 0.5) / rows
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits.repeat(rows, 1)), out, dev(torch.full((rows,), temperature)),
               dev(torch.full((rows,), top_k, dtype=torch.int32)), dev(torch.full((rows,), top_p)), dev(uniform))
    sp, si = _survivors(logits, temperature, top_k, top_p)
    keep = torch.zeros(vocab, dtype=torch.bool)
    keep[si] = True
    got = out.cpu().long()
    assert bool(keep[got].all()), "a token outside the surviving set was drawn"
    # inverse CDF over the survivors in index order
    p = torch.softmax(logits.double() / temperature, 0) * keep
    cdf = torch.cumsum(p, 0)
    for r in range(rows):
        target = float(uniform[r]) * float(p.sum())
        want = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
        assert abs(float(cdf[got[r]]) - float(cdf[want])) <= 2e-6 or got[r] == want, (r, int(got[r]), want)


@pytest.mark.parametrize("vocab", [18995, 151936])
def test_sample_large_vocabulary_many_blocks_per_row(vocab):
    """Rows of a whole vocabulary are worked on by many blocks: every draw lies in the plain implementation's
    surviving set, ties at the threshold included; the same call twice gives the same tokens; rows do not
    depend on their neighbours."""
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(16)
    base = torch.randn(vocab, generator=g) * 2.5
    base[::97] = base[5]                                    # many equal logits
    cases = [(0.7, 40, 1.0), (1.0, 0, 0.92), (1.3, 200, 0.5), (0.9, 0, 1.0), (0.6, 1, 1.0), (1.0, 7, 0.999)]
    rows = len(cases) * 4
    logits = torch.stack([base + 0.01 * (r // len(cases)) * torch.randn(vocab, generator=g) for r in range(rows)])
    temp = torch.tensor([cases[r % len(cases)][0] for r in range(rows)])
    top_k = torch.tensor([cases[r % len(cases)][1] for r in range(rows)], dtype=torch.int32)
    top_p = torch.tensor([cases[r % len(cases)][2] for r in range(rows)])
    uniform = torch.rand(rows, generator=g)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    args = (dev(logits), out, dev(temp), dev(top_k), dev(top_p), dev(uniform))
    ops.sample(*args, any_greedy=False)
    got = out.cpu().tolist()
    ops.sample(*args, any_greedy=False)
    assert out.cpu().tolist() == got
    for r in range(rows):
        t, k, p = cases[r % len(cases)]
        sp, si = _survivors(logits[r], t, k, p)
        probs = torch.softmax(logits[r].double() / t, 0)
        edge = float(sp.min())
        near = set(torch.nonzero((probs - edge).abs() <= 1e-6 * edge).flatten().tolist())     # float32 ties at the edge
        assert got[r] in set(si.tolist()) | near, (r, got[r])
        if k == 1:
            assert got[r] == int(torch.argmax(logits[r]))
    # a row alone gives the same token as in the batch
    one = torch.empty(1, dtype=torch.int32, device="cuda")
    for r in (1, 8, rows - 1):
        ops.sample(dev(logits[r:r + 1]), one, dev(temp[r:r + 1]), dev(top_k[r:r + 1]), dev(top_p[r:r + 1]), dev(uniform[r:r + 1]),
                   any_greedy=False)
        assert int(one.cpu()) == got[r]


@pytest.mark.parametrize("vocab", [40, 5000])
def test_sample_keeps_exactly_k_when_probabilities_tie_at_the_cut(vocab):
    """Equal logits at the cut (bfloat16 heads and tied embeddings make them): a sort keeps exactly k tokens and the
    nucleus rule looks at the mass strictly before each token, so of the tied tokens only the first ones in index
    order survive (pulsar-core/src/runtime/sampler.cpp:30-40; the plain implementation's stable sort)."""
    from pulsar_b200 import ops
    logits = torch.full((vocab,), -4.0)
    tied = [3, 9, 17, 21, vocab - 2]                   # five tokens share the top probability, across slices of the row
    logits[tied] = 2.0
    logits[30] = 1.0
    rows = 48
    uniform = (torch.arange(rows, dtype=torch.float32) + 0.5) / rows
    for top_k, top_p, want in ((2, 1.0, tied[:2]), (4, 1.0, tied[:4]), (6, 1.0, tied + [30]), (0, 0.35, None), (3, 0.35, None)):
        out = torch.empty(rows, dtype=torch.int32, device="cuda")
        ops.sample(dev(logits.repeat(rows, 1)), out, dev(torch.ones(rows)), dev(torch.full((rows,), top_k, dtype=torch.int32)),
                   dev(torch.full((rows,), top_p)), dev(uniform))
        _, si = _survivors(logits, 1.0, top_k, top_p)
        keep = sorted(si.tolist())
        if want is not None:
            assert keep == sorted(want)
        got = sorted(set(out.cpu().tolist()))
        assert set(got) <= set(keep), (top_k, top_p, got, keep)        # nothing outside the surviving set is drawn
        if len(keep) <= 8:
            assert got == keep, (top_k, top_p, got, keep)              # and every survivor is reached by some uniform


def test_sample_mixed_rows_and_greedy_ignores_filters():
    from pulsar_b200 import ops
    g = torch.Generator().manual_seed(10)
    logits = torch.randn(4, 333, generator=g) * 3
    out = torch.empty(4, dtype=torch.int32, device="cuda")
    temp = torch.tensor([0.0, 1.0, 0.0, 0.5])
    ops.sample(dev(logits), out, dev(temp), dev(torch.tensor([1, 1, 7, 0], dtype=torch.int32)),
               dev(torch.tensor([0.1, 1.0, 0.5, 1.0])), dev(torch.tensor([0.9, 0.9, 0.9, 0.0])))
    got = out.cpu().tolist()
    am = torch.argmax(logits, -1).tolist()
    assert got[0] == am[0] and got[2] == am[2]
    assert got[1] == am[1]              # top_k 1 leaves only the most probable
    assert 0 <= got[3] < 333
