"""Typed Python wrappers over the C interface of the CUDA library.

Each wrapper checks what the kernel cannot check itself (device, dtype, shape,
contiguity), passes raw pointers and the current CUDA stream, and raises on any
non-zero status.  There is no CPU path: a tensor that is not on a CUDA device is an
error, and a missing library is an error at first use.

The reference exposes its kernels as ``torch.ops.pulsar.*`` through TorchBind
(pulsar/ext/ops.cpp:8-74; pulsar/src/pulsar/core/ops.py:198-494).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import profiling
from ..csrc.build import library

F32, BF16 = 0, 1
# Which product serves bfloat16 projections of more than 16 rows:
#   "auto"     with more than 128 rows the gate/up product with its SwiGLU gating fused runs on this
#              library's tcgen05 / TMA kernel (faster than the library product plus a gating kernel);
#              the plain projections, and gate/up of 17 to 128 rows, take the library product
#              (cuBLAS through torch.mm, as the reference does);
#   "tcgen05"  every projection on the tcgen05 kernel;
#   "library"  every projection on the library product, gating in a kernel of its own.
# Up to 16 rows always take the weight-streaming kernel.
GEMM_BACKEND = os.environ.get("PULSAR_GEMM", "auto")
# Attention of prompt portions in bfloat16: "auto" = the tcgen05 kernel where it applies, "mma" = never.
ATTENTION_BACKEND = os.environ.get("PULSAR_ATTENTION", "auto")
# The library product (torch.mm) must add its partial sums in float32: by default PyTorch lets cuBLAS reduce
# split-K partial sums of bfloat16 products in bfloat16.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {-2: "unsupported dtype", -3: "unsupported size or argument", -4: "size exceeds the kernel's limit"}

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_SIGNATURES = {
    "pb_embed": [_I, _P, _P, _P, _I, _I, _I, _F, _P],
    "pb_scale_cap": [_P, ctypes.c_longlong, _F, _F, _P],
    "pb_move_ids": [_P, _P, _P, _P, _I, _P],
    "pb_table_update": [_P, _I, _P, _P, _I, _I, _P, _P],
    "pb_add_rmsnorm": [_I, _P, _P, _P, _P, _P, _I, _I, _F, _I, _P],
    "pb_rope_table": [_P, _P, _P, _P, _I, _I, _P],
    "pb_qk_norm_rope_write": [_I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _I, _I, _P],
    "pb_silu_mul": [_I, _P, _P, _I, _I, _P],
    "pb_paged_attention_generic": [_I, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
    "pb_paged_attention_decode": [_I, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "pb_paged_attention_decode_tc": [_I, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "pb_decode_tc_supported": [_I, _I, _I, _I, _I],
    "pb_paged_attention_decode_tc_qkv": [_I, _P, _P, _P, _P, _P, _F, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "pb_paged_attention_decode_tc_fused": [_I, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "pb_paged_attention_prefill_tc": [_I, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    "pb_prefill_tc_supported": [_I, _I, _I, _I, _I],
    "pb_prefill_tc_tile": [],
    "pb_paged_attention_prefill_tcgen05": [_I, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    "pb_prefill_tcgen05_supported": [_I, _I, _I, _I, _I],
    "pb_prefill_tcgen05_tile": [],
    "pb_prefill_tcgen05_error": [],
    "pb_gemm_skinny": [_I, _I, _P, _P, _P, _I, _I, _I, _P],
    "pb_gemm_skinny_supported": [_I, _I, _I, _I],
    "pb_gemm_skinny_fused_supported": [_I, _I, _I, _I],
    "pb_gemm_skinny_publish_sums": [_I],
    "pb_gemm_skinny_accumulate": [_P, _P, _P, _I, _I, _I, _P, _P, _P, _P],
    "pb_gemm_skinny_scaled": [_I, _P, _P, _P, _I, _I, _I, _P, _F, _P],
    "pb_gemm_tcgen05": [_I, _I, _P, _P, _P, _I, _I, _I, _P],
    "pb_gemm_tcgen05_supported": [_I, _I, _I, _I],
    "pb_gemm_tcgen05_error": [],
    "pb_gemm_tcgen05_stream": [_I, _I, _P, _P, _P, _I, _I, _I, _P, ctypes.c_longlong, _P, _I, _P],
    "pb_gemm_tcgen05_stream_workspace": [_I, _I, _I, _I, _P, _P],
    "pb_gemm_tcgen05_stream_supported": [_I, _I, _I, _I],
    "pb_gemm_tcgen05_stream_wait_control": [ctypes.c_longlong, _I, _P],
    "pb_gemm_tcgen05_wait_control": [ctypes.c_longlong, _I, _P],
    "pb_gemm_tcgen05_wait_selftest": [_P],
    "pb_prefill_tcgen05_wait_control": [ctypes.c_longlong, _I, _P],
    "pb_gather_words": [_P, _I, _P, _P],
    "pb_bounds_checked": [],
    "pb_set_pool_bounds": [_I, _P],
    "pb_gemm_simt": [_I, _I, _I, _P, _P, _P, _I, _I, _I, _P],
    "pb_sample": [_P, _I, _I, _P, _P, _P, _P, _I, _P, _P, _P, _P],
    "pb_sample_workspace": [_I],
    "pb_argmax": [_P, _I, _I, _P, _P, _P],
}
_fns = {}
# the entry points that launch kernels (the others answer questions on the host): what PULSAR_PROF=1 times
_LAUNCHERS = {"embed", "scale_cap", "move_ids", "add_rmsnorm", "rope_table", "qk_norm_rope_write", "silu_mul", "gather_words",
              "paged_attention_generic", "paged_attention_decode", "paged_attention_decode_tc", "paged_attention_decode_tc_fused",
              "paged_attention_decode_tc_qkv",
              "paged_attention_prefill_tc", "paged_attention_prefill_tcgen05", "gemm_skinny", "gemm_skinny_accumulate",
              "gemm_skinny_scaled", "gemm_tcgen05", "gemm_tcgen05_stream", "gemm_simt", "sample", "argmax", "table_update"}


class KernelError(RuntimeError):
    pass


def fn(name: str):
    f = _fns.get(name)
    if f is None:
        f = getattr(library(), name)
        f.argtypes = _SIGNATURES[name]
        f.restype = ctypes.c_int
        if profiling.ENABLED and name[3:] in _LAUNCHERS:
            f = profiling.timed_launcher(name, f)
        _fns[name] = f
    return f


def register_signature(name: str, argtypes) -> None:
    _SIGNATURES[name] = list(argtypes)


LAUNCHES = 0      # kernels of this library launched so far (each wrapper call launches one or more)


def check(status: int, name: str, kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += kernels
    if status != 0:
        what = _ERRORS.get(status, f"CUDA error {status}")
        raise KernelError(f"{name}: {what}")


def code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not float32 or bfloat16") from None


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernel arguments must be contiguous CUDA tensors "
                              f"(found device {t.device}, contiguous={t.is_contiguous()}); there is no CPU path")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] (float32) = table[ids[t]] * scale."""
    _cuda(table, ids, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and out.shape == (ids.numel(), table.shape[1])
    check(fn("pb_embed")(code(table.dtype), _p(table), _p(ids), _p(out), ids.numel(), table.shape[1], table.shape[0],
                         float(scale), stream()), "embed")


def scale_cap(x: torch.Tensor, scale: float = 1.0, cap: Optional[float] = None) -> None:
    """In place on float32 values: x *= scale, then cap * tanh(x / cap) where a cap is given."""
    _cuda(x)
    assert x.dtype == torch.float32
    check(fn("pb_scale_cap")(_p(x), x.numel(), float(scale), float(cap or 0.0), stream()), "scale_cap")


def move_ids(ids: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, src_ids: torch.Tensor) -> None:
    """ids[dst[i]] = src_ids[src[i]] (all int32 on the device): sampled tokens of the step before become
    this step's input without a trip through the host."""
    _cuda(ids, dst, src, src_ids)
    assert ids.dtype == dst.dtype == src.dtype == src_ids.dtype == torch.int32 and dst.numel() == src.numel()
    check(fn("pb_move_ids")(_p(ids), _p(dst), _p(src), _p(src_ids), dst.numel(), stream()), "move_ids")


def table_update(resident: torch.Tensor, updates: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """Apply a step's (row, logical page, page id) triples to the resident block tables [rows, stride] and copy the
    step's rows (``rows`` [S]) into ``out`` [S, width]; ``updates`` = the count, then the triples (all int32)."""
    _cuda(resident, updates, rows, out)
    assert resident.dtype == updates.dtype == rows.dtype == out.dtype == torch.int32
    s, width = out.shape
    assert rows.numel() == s and resident.dim() == 2 and width <= resident.shape[1]
    check(fn("pb_table_update")(_p(resident), resident.shape[1], _p(updates), _p(rows), s, width, _p(out), stream()), "table_update")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
    """x = residual (+ delta); residual = x when write_back; out = rmsnorm(x) * weight.
    With ``rows`` only those rows are normalised, gathered into ``out``; the residual is left alone."""
    _cuda(residual, delta, weight, out, rows)
    width = residual.shape[-1]
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == width
    assert delta is None or (delta.dtype == out.dtype and delta.shape == residual.shape)
    if rows is not None:
        assert rows.dtype == torch.int32
        write_back = False
    n_out = rows.numel() if rows is not None else residual.shape[0]
    assert out.shape == (n_out, width)
    check(fn("pb_add_rmsnorm")(code(out.dtype), _p(residual), _p(delta), _p(weight), _p(out), _p(rows), n_out, width,
                               float(eps), int(write_back), stream()), "add_rmsnorm")


def rope_table(positions: torch.Tensor, quadrants_per_position: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    _cuda(positions, quadrants_per_position, cos, sin)
    half = quadrants_per_position.numel()
    assert positions.dtype == torch.int32 and quadrants_per_position.dtype == torch.float64
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32
    assert cos.shape == (positions.numel(), half) and sin.shape == cos.shape
    check(fn("pb_rope_table")(_p(positions), _p(quadrants_per_position), _p(cos), _p(sin), positions.numel(), half,
                              stream()), "rope_table")


def qk_norm_rope_write(qkv: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                       v_pool: Optional[torch.Tensor], slots: Optional[torch.Tensor], cos: torch.Tensor,
                       sin: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                       eps: float, n_heads: int, n_kv_heads: int, head_dim: int, rotary: int, page_size: int) -> None:
    """Per-head RMSNorm (when weights are given) and rotation of q and k, q to ``q_out``,
    k and v into their pages.  ``n_kv_heads`` 0: the row holds q only."""
    _cuda(qkv, q_out, k_pool, v_pool, slots, cos, sin, q_weight, k_weight)
    _check_against(k_pool)
    n = qkv.shape[0]
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim and q_out.dtype == qkv.dtype
    assert cos.shape == (n, rotary // 2) and sin.shape == cos.shape and cos.dtype == torch.float32
    if n_kv_heads:
        assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype and slots.dtype == torch.int32
        assert k_pool.shape[1:] == (n_kv_heads, page_size, head_dim) and v_pool.shape == k_pool.shape
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == head_dim)
    check(fn("pb_qk_norm_rope_write")(code(qkv.dtype), _p(qkv), _p(q_out), _p(k_pool), _p(v_pool), _p(slots), _p(cos),
                                      _p(sin), _p(q_weight), _p(k_weight), float(eps), n, n_heads, n_kv_heads, head_dim,
                                      rotary, page_size, stream()), "qk_norm_rope_write")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(gate_up, out)
    n, two_i = gate_up.shape
    assert out.shape == (n, two_i // 2) and out.dtype == gate_up.dtype and two_i % 2 == 0
    check(fn("pb_silu_mul")(code(out.dtype), _p(gate_up), _p(out), n, two_i // 2, stream()), "silu_mul")


def paged_attention_generic(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                            block_table: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                            seq_of_token: torch.Tensor, scale: float, window: Optional[int]) -> None:
    _cuda(q, k_pool, v_pool, out, block_table, cu_q, kv_len, seq_of_token)
    _check_against(k_pool)
    n, hq, d = q.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and out.shape == q.shape
    assert k_pool.dtype == q.dtype and v_pool.dtype == q.dtype and out.dtype == q.dtype
    for t in (block_table, cu_q, kv_len, seq_of_token):
        assert t.dtype == torch.int32
    assert block_table.dim() == 2 and seq_of_token.numel() == n
    check(fn("pb_paged_attention_generic")(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(block_table),
                                           block_table.shape[1], _p(cu_q), _p(kv_len), _p(seq_of_token), n, hq, hkv, d,
                                           page_size, float(scale), int(window or 0), stream()), "paged_attention_generic")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = a @ w.T in float32 multiply-adds (no tensor cores)."""
    _cuda(a, w, out)
    m, k = a.shape
    n, k2 = w.shape
    assert k2 == k and out.shape == (m, n)
    check(fn("pb_gemm_simt")(code(a.dtype), code(w.dtype), code(out.dtype), _p(a), _p(w), _p(out), m, n, k, stream()),
          "gemm_simt")


_argmax_keys = {}
_sample_work = {}


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None, any_greedy: bool = True) -> None:
    """out[r] = argmax (temperature <= 0 or None) or a draw from the filtered softmax.
    ``any_greedy=False`` promises that every row has a temperature > 0."""
    _cuda(logits, out, temperature, top_k, top_p, uniform)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() == rows
    assert temperature is None or (temperature.dtype == torch.float32 and temperature.numel() == rows)
    assert top_k is None or (top_k.dtype == torch.int32 and top_k.numel() == rows)
    assert top_p is None or (top_p.dtype == torch.float32 and top_p.numel() == rows)
    assert uniform is None or (uniform.dtype == torch.float32 and uniform.numel() == rows)
    keys = _argmax_keys.get(logits.device)
    if keys is None or keys.numel() < rows:
        keys = _argmax_keys[logits.device] = torch.empty(max(rows, 256), dtype=torch.int64, device=logits.device)
    if temperature is None:                       # all rows greedy: many blocks per row
        check(fn("pb_argmax")(_p(logits), rows, vocab, _p(keys), _p(out), stream()), "argmax", kernels=2)
        return
    if uniform is None:
        raise KernelError("sample: rows with a temperature need uniform numbers")
    need = int(fn("pb_sample_workspace")(rows)) * 1024
    work = _sample_work.get(logits.device)
    if work is None or work.numel() < need:
        work = _sample_work[logits.device] = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=logits.device)
    filtered = top_k is not None or top_p is not None
    check(fn("pb_sample")(_p(logits), rows, vocab, _p(temperature), _p(top_k), _p(top_p), _p(uniform), 1 if any_greedy else 0,
                          _p(work), _p(keys), _p(out), stream()), "sample", kernels=(2 if any_greedy else 0) + (5 if filtered else 2))


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> bool:
    """The weight-streaming product for up to 16 tokens (bfloat16).  ``swiglu``: ``w`` holds
    gate rows then up rows and ``out`` [M, inter] receives silu(gate) * up.  Returns False,
    having done nothing, when the sizes are not the kernel's."""
    m, k = a.shape
    n = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k:
        return False
    mode = 1 if swiglu else 0
    if not fn("pb_gemm_skinny_supported")(mode, m, n, k):
        return False
    _cuda(a, w, out)
    assert out.shape == (m, n // 2 if swiglu else n)
    check(fn("pb_gemm_skinny")(mode, code(out.dtype), _p(a), _p(w), _p(out), m, n, k, stream()), "gemm_skinny")
    return True


# Steps of up to 16 tokens (bfloat16): the output and down projections add their result to the float32 residual
# stream inside the product (no bfloat16 rounding of it, no addition in the norm kernel), and the down projection
# prepares the next layer's first norm, which the q/k/v product then applies itself (one norm kernel per layer
# less).  PULSAR_FUSED_NORM=0 turns both off.  The same for the norm in front of gate/up is built and tested but
# off: that product has thousands of short-lived blocks, and what each of them adds at its end costs more than the
# norm kernel it saves (measured: 3.77 against 3.61 ms per step at batch 8); PULSAR_FUSED_NORM_MLP=1 turns it on.
FUSED_NORM = os.environ.get("PULSAR_FUSED_NORM", "1") != "0"
FUSED_NORM_MLP = os.environ.get("PULSAR_FUSED_NORM_MLP", "0") != "0"


def _aligned32(*tensors) -> bool:
    return all(t.data_ptr() % 32 == 0 for t in tensors)


def fused_projection_supported(m: int, w: torch.Tensor, swiglu: bool = False) -> bool:
    """Whether ``linear_prenormed`` / ``linear_accumulate`` take ``m`` tokens against the weight ``w`` [N, K]."""
    return bool(FUSED_NORM and w.dtype == torch.bfloat16 and w.is_cuda and w.data_ptr() % 32 == 0
                and fn("pb_gemm_skinny_fused_supported")(1 if swiglu else 0, m, w.shape[0], w.shape[1]))


def norm_parts_numel(m: int, width: int) -> int:
    """Floats of the buffer in which ``linear_accumulate`` leaves the parts of the sums of squares of ``m`` rows
    ``width`` wide: a part per 16 columns and row, then a 64-bit word per row (its sum and a tag)."""
    return (width // 16 + 2) * m


def linear_accumulate(a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, next_norm_weight: Optional[torch.Tensor] = None,
                      prepared: Optional[torch.Tensor] = None, parts: Optional[torch.Tensor] = None) -> bool:
    """residual (float32) += a @ w.T for up to 16 tokens: the projection's result goes into the residual stream
    without a bfloat16 rounding and without a kernel for the addition.  With ``next_norm_weight`` (the weight of
    the RMSNorm that follows) the kernel also prepares that norm: ``prepared`` [M, N] bfloat16 = residual *
    weight and ``parts`` (float32, ``norm_parts_numel(M, N)`` elements) = each block's part of the rows' sums of
    squares [N / 16, M], which ``linear_prenormed`` takes (and behind which it keeps the sums).  Returns False, having done nothing, when the sizes or dtypes are not the kernel's."""
    m, k = a.shape
    n = w.shape[0]
    if (not FUSED_NORM or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or residual.dtype != torch.float32
            or w.shape[1] != k or residual.shape != (m, n)):
        return False
    if not fn("pb_gemm_skinny_fused_supported")(0, m, n, k) or not _aligned32(a, w):
        return False
    _cuda(a, w, residual, next_norm_weight, prepared, parts)
    if next_norm_weight is not None:
        assert next_norm_weight.dtype == torch.float32 and next_norm_weight.numel() == n
        assert prepared.dtype == torch.bfloat16 and prepared.shape == (m, n)
        assert parts.dtype == torch.float32 and parts.numel() >= norm_parts_numel(m, n)
    check(fn("pb_gemm_skinny_accumulate")(_p(a), _p(w), _p(residual), m, n, k, _p(next_norm_weight), _p(prepared), _p(parts),
                                          stream()), "gemm_skinny_accumulate")
    return True


def linear_prenormed(prepared: torch.Tensor, parts: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor,
                     swiglu: bool = False) -> bool:
    """out = rmsnorm(residual) @ w.T (or its SwiGLU form) from what ``linear_accumulate`` prepared: the product of
    ``prepared`` (residual * norm weight, bfloat16) with each token's sums scaled by rsqrt(mean(residual^2) + eps),
    the mean from ``parts``.  Returns False, having done nothing, when the sizes or dtypes are not the kernel's."""
    m, k = prepared.shape
    n = w.shape[0]
    if (not FUSED_NORM or prepared.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16
            or w.shape[1] != k or parts.dtype != torch.float32 or k % 64):
        return False
    mode = 1 if swiglu else 0
    if not fn("pb_gemm_skinny_fused_supported")(mode, m, n, k) or not _aligned32(prepared, w):
        return False
    _cuda(prepared, parts, w, out)
    assert out.shape == (m, n // 2 if swiglu else n) and parts.numel() >= norm_parts_numel(m, k)
    check(fn("pb_gemm_skinny_scaled")(mode, _p(prepared), _p(w), _p(out), m, n, k, _p(parts), float(eps), stream()),
          "gemm_skinny_scaled")
    return True


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> bool:
    """The tcgen05 / TMA product for many tokens (bfloat16 operands, float32 accumulation in
    tensor memory).  ``swiglu`` as in ``gemm_skinny``.  Returns False, having done nothing,
    when the sizes are not the kernel's (K must be a multiple of 8)."""
    m, k = a.shape
    n = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k:
        return False
    mode = 1 if swiglu else 0
    if not fn("pb_gemm_tcgen05_supported")(mode, m, n, k):
        return False
    _cuda(a, w, out)
    assert out.shape == (m, n // 2 if swiglu else n)
    check(fn("pb_gemm_tcgen05")(mode, code(out.dtype), _p(a), _p(w), _p(out), m, n, k, stream()), "gemm_tcgen05")
    return True


# Which products of 17 to 128 tokens take this library's weight-streaming tcgen05 kernel instead of the library
# product: "auto" those whose weights have tiles for four rounds of all SMs or more (the head: there the kernel's
# persistent form is ahead of the library, 6.1 against 6.0 TB/s at 64 tokens); "1" all of them (measured behind the
# library for the projections of a layer at the 8B sizes: see profiles/); "0" none.
STREAM_GEMM = os.environ.get("PULSAR_GEMM_STREAM", "auto")
_STREAM_MIN_ROWS = 4 * 148 * 128


def _stream_wanted(m: int, n: int) -> bool:
    if m > 128 or STREAM_GEMM == "0" or GEMM_BACKEND == "library":
        return False
    return STREAM_GEMM == "1" or n >= _STREAM_MIN_ROWS


# Float32 partial sums and tile tickets of the product below, one pair per device, grown on demand.  A buffer
# that was outgrown stays alive: a captured graph may still name it.  Kernels of one stream share the pair (each
# finishes with it before the next one starts, and leaves the tickets zero).
_stream_scratch = {}
_stream_scratch_old = []


def _stream_workspace(device: torch.device, mode: int, m: int, n: int, k: int):
    floats, tickets = ctypes.c_longlong(0), ctypes.c_int(0)
    fn("pb_gemm_tcgen05_stream_workspace")(mode, m, n, k, ctypes.byref(floats), ctypes.byref(tickets))
    if floats.value == 0:
        return None, None
    have = _stream_scratch.get(device)
    if have is None or have[0].numel() < floats.value or have[1].numel() < tickets.value:
        if torch.cuda.is_current_stream_capturing():
            return None, None                 # no allocation inside a capture: whole tiles this once
        if have is not None:
            _stream_scratch_old.append(have)
        have = (torch.empty(max(floats.value, have[0].numel() if have else 0), dtype=torch.float32, device=device),
                torch.zeros(max(tickets.value, have[1].numel() if have else 0, 2048), dtype=torch.int32, device=device))
        _stream_scratch[device] = have
    return have


def gemm_tcgen05_stream(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> bool:
    """The weight-streaming tcgen05 / TMA product for up to 128 tokens (bfloat16 operands, float32 accumulation
    in tensor memory, K cut into slices whose partial sums meet in a float32 workspace).  ``swiglu`` as in
    ``gemm_skinny``.  Returns False, having done nothing, when the sizes are not the kernel's."""
    m, k = a.shape
    n = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k:
        return False
    mode = 1 if swiglu else 0
    if not fn("pb_gemm_tcgen05_stream_supported")(mode, m, n, k):
        return False
    _cuda(a, w, out)
    assert out.shape == (m, n // 2 if swiglu else n)
    work, tickets = _stream_workspace(a.device, mode, m, n, k)
    status = fn("pb_gemm_tcgen05_stream")(mode, code(out.dtype), _p(a), _p(w), _p(out), m, n, k,
                                          _p(work) if work is not None else None, work.numel() if work is not None else 0,
                                          _p(tickets) if tickets is not None else None,
                                          tickets.numel() if tickets is not None else 0, stream())
    if status == -3:
        return False                 # sizes that leave no room for its ring of stages
    check(status, "gemm_tcgen05_stream")
    return True


def gemm_tcgen05_error() -> int:
    """0 unless a block of the tcgen05 product ever gave up a bounded wait (synchronises)."""
    return int(fn("pb_gemm_tcgen05_error")())


# ---------------------------------------------------------------- bounded waits: limit and error words
# The kernels that wait on barriers (the tcgen05 product, the two tcgen05 attention kernels) bound every wait by
# a clock limit; a block whose wait runs out sets its kernel's error word, lets its copies land, frees its tensor
# memory and returns, and what the kernel wrote is then not to be trusted.  The reference's engine turns a step
# that cannot go on into an exception (pulsar-core/src/runtime/engine.cpp:809-814) and its Python layer
# poisons the engine (pulsar/src/pulsar/rt/sync.py:21-34); the words below are how this engine learns of it.
WAIT_WORD_NAMES = ("tcgen05 product", "tcgen05 attention, one head per block", "tcgen05 attention, two heads per block",
                   "tcgen05 product for up to 128 tokens", "bounds check of the debug build")
N_WAIT_WORDS = len(WAIT_WORD_NAMES)          # the last one is 0 in a build without the checks
BOUNDS_CODES = {2: "a block table named a page outside its pool (the access was skipped)",
                3: "a slot outside its pool (the write was dropped)"}
_bounds_words = {}


def bounds_checked() -> bool:
    """Whether the loaded library is the debug build whose kernels check page ids and slots
    (built with PULSAR_CHECK_BOUNDS=1)."""
    return bool(fn("pb_bounds_checked")())


def _bounds_word() -> torch.Tensor:
    dev = torch.cuda.current_device()
    word = _bounds_words.get(dev)
    if word is None:
        word = _bounds_words[dev] = torch.zeros(1, dtype=torch.int32, device="cuda")
    return word


def _check_against(pool: Optional[torch.Tensor]) -> None:
    """Debug build: the kernels launched next check page ids and slots against this pool's size."""
    if pool is not None and bounds_checked():
        fn("pb_set_pool_bounds")(int(pool.shape[0]), _p(_bounds_word()))


def bounds_error() -> int:
    """0, or the largest code a bounds check recorded (synchronises); always 0 without the debug build."""
    return int(_bounds_word().item()) if bounds_checked() else 0


def clear_bounds_error() -> None:
    if bounds_checked():
        _bounds_word().zero_()
WAIT_ROLES = {2: "the TMA producer", 3: "the MMA issuer", 4: "the epilogue or softmax warps", 9: "the wait self-test"}
_wait_words = {}
_check_buf = {}


class DeviceWaitError(KernelError):
    """A kernel gave up a bounded wait: its output, and everything computed from it, is not valid."""


def wait_word_addresses() -> "ctypes.Array":
    """Device addresses of the error words of the current device (looked up once per device)."""
    dev = torch.cuda.current_device()
    got = _wait_words.get(dev)
    if got is None:
        got = (ctypes.c_void_p * N_WAIT_WORDS)()
        one = (ctypes.c_void_p * 1)()
        two = (ctypes.c_void_p * 2)()
        three = (ctypes.c_void_p * 1)()
        if (fn("pb_gemm_tcgen05_wait_control")(0, -1, one) != 0 or fn("pb_prefill_tcgen05_wait_control")(0, -1, two) != 0
                or fn("pb_gemm_tcgen05_stream_wait_control")(0, -1, three) != 0):
            raise KernelError("the addresses of the wait error words could not be had")
        got[0], got[1], got[2], got[3] = one[0], two[0], two[1], three[0]
        got[4] = _bounds_word().data_ptr()
        _wait_words[dev] = got
    return got


def gather_wait_words(out: torch.Tensor) -> None:
    """out[:N_WAIT_WORDS] (int32, device) = the error words, read in the stream behind whatever was launched before."""
    _cuda(out)
    assert out.dtype == torch.int32 and out.numel() >= N_WAIT_WORDS
    check(fn("pb_gather_words")(wait_word_addresses(), N_WAIT_WORDS, _p(out), stream()), "gather_words")


def set_wait_limit(cycles: int) -> None:
    """The limit of every bounded wait, in clock cycles (4e9 at first, about two seconds)."""
    if cycles <= 0:
        raise ValueError("the wait limit must be positive")
    if fn("pb_gemm_tcgen05_wait_control")(int(cycles), -1, None) != 0 or \
            fn("pb_prefill_tcgen05_wait_control")(int(cycles), -1, None) != 0 or \
            fn("pb_gemm_tcgen05_stream_wait_control")(int(cycles), -1, None) != 0:
        raise KernelError("the wait limit could not be set")


def set_wait_words(value: int) -> None:
    """Write all three error words (0 clears them once a failure has been dealt with)."""
    if fn("pb_gemm_tcgen05_wait_control")(0, int(value), None) != 0 or \
            fn("pb_prefill_tcgen05_wait_control")(0, int(value), None) != 0 or \
            fn("pb_gemm_tcgen05_stream_wait_control")(0, int(value), None) != 0:
        raise KernelError("the wait error words could not be written")


def wait_selftest() -> None:
    """One thread waits on a barrier nobody arrives on until the limit runs out and sets the product's error word to 9."""
    check(fn("pb_gemm_tcgen05_wait_selftest")(stream()), "wait_selftest")


def describe_wait_words(words) -> Optional[str]:
    """None when all words are 0, else which kernel gave up and in which role."""
    bad = [(i, WAIT_WORD_NAMES[i], int(w)) for i, w in enumerate(words) if int(w) != 0]
    if not bad:
        return None
    return "; ".join(f"{name}: {BOUNDS_CODES.get(w, 'code ' + str(w))}" if i == N_WAIT_WORDS - 1 else
                     f"{name}: {WAIT_ROLES.get(w, 'role ' + str(w))} gave up a bounded wait" for i, name, w in bad)


def check_wait_words() -> None:
    """Read the words now (synchronises) and raise DeviceWaitError if one is set."""
    buf = _check_buf.get(torch.cuda.current_device())
    if buf is None:
        buf = _check_buf[torch.cuda.current_device()] = torch.zeros(8, dtype=torch.int32, device="cuda")
    gather_wait_words(buf)
    what = describe_wait_words(buf[:N_WAIT_WORDS].tolist())
    if what is not None:
        raise DeviceWaitError(what)


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = a @ w.T.  float32 operands take the float32 CUDA-core product (true 32-bit,
    no reduced-precision mode).  bfloat16 operands: up to 16 rows take this library's
    weight-streaming kernel; more rows take the library product with float32 accumulation,
    as the reference does for every projection (pulsar-core/src/model/qwen3.cpp:82-84:
    at::linear)."""
    if a.dtype == torch.float32 and w.dtype == torch.float32:
        gemm_simt(a, w, out)
        return
    _cuda(a, w, out)
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: operand dtypes {a.dtype} / {w.dtype} must both be float32 or both bfloat16")
    if gemm_skinny(a, w, out):
        return
    if _stream_wanted(a.shape[0], w.shape[0]) and gemm_tcgen05_stream(a, w, out):
        return
    if GEMM_BACKEND == "tcgen05" and gemm_tcgen05(a, w, out):
        return
    with profiling.kernel("library product (torch.mm)"):
        if out.dtype == torch.bfloat16:
            torch.mm(a, w.t(), out=out)
        else:
            out.copy_(torch.mm(a, w.t(), out_dtype=torch.float32))


def gated_linear(ctx, a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out [M, I] = silu(a Wg^T) * (a Wu^T) with ``w_gate_up`` = gate rows then up rows.  In
    bfloat16, up to 16 rows (the weight-streaming kernel) and more than 128 rows (the tcgen05 kernel)
    take one kernel that never writes the [M, 2I] intermediate; otherwise the product followed by the
    gating kernel."""
    if gemm_skinny(a, w_gate_up, out, swiglu=True):
        return
    if _stream_wanted(a.shape[0], w_gate_up.shape[0]) and gemm_tcgen05_stream(a, w_gate_up, out, swiglu=True):
        return
    # Between 17 and 128 rows the product is still bound by streaming the weights, which the library's small
    # tiles do faster (4.5 against 3.2 TB/s at the 8B sizes) than the tcgen05 kernel's 128 x 256 tiles.
    fused = GEMM_BACKEND == "tcgen05" or (GEMM_BACKEND == "auto" and a.shape[0] > 128)
    if fused and gemm_tcgen05(a, w_gate_up, out, swiglu=True):
        return
    gate_up = ctx.scratch("mlp.gate_up", (a.shape[0], w_gate_up.shape[0]), a.dtype)
    linear(a, w_gate_up, gate_up)
    silu_mul(gate_up, out)


_FORCED_SPLITS = int(os.environ.get("PULSAR_DECODE_SPLITS", "0") or 0)      # > 0: this many splits, for measurements
_DECODE_SLOTS = 296          # two blocks of the decode attention kernel on each of the 148 SMs


def decode_splits(n_seqs: int, n_kv_heads: int, table_tokens: int = 4096) -> int:
    """Splits of the keys per (sequence, kv head), at most 32 and at most one per 256 tokens that the
    block table can name.  While all blocks fit the SMs at once: as many splits as still fit.  With
    more (sequence, kv head) pairs than that, the blocks run in rounds, and what costs is a last round
    too thin to keep HBM busy (a block alone pulls about 37 GB/s against its 22 GB/s share of a full
    round, so a last round under 0.6 of the slots takes 0.6 of a round all the same); splits shorten
    the rounds and cost about 4 % for the merge.  Measured at context 4096, 8 kv heads: batch 48 runs
    12 % faster with 3 splits than with 1, batch 64 is fastest with 1.  A function of the batch and of
    the block table's width alone (the width of a step of single tokens grows in buckets), so that a
    captured step stays valid while its sequences grow."""
    pairs = max(1, n_seqs * n_kv_heads)
    most = max(1, min(32, table_tokens // 256))
    if _FORCED_SPLITS > 0:
        return min(most, _FORCED_SPLITS)
    if pairs <= _DECODE_SLOTS:
        return max(1, min(most, _DECODE_SLOTS // pairs))
    best, best_cost = 1, None
    for k in range(1, min(most, 8) + 1):
        rounds = pairs * k / _DECODE_SLOTS
        whole, rest = int(rounds), rounds - int(rounds)
        cost = (whole + (max(0.6, rest) if rest > 1e-9 else 0.0)) / k * (1.0 if k == 1 else 1.04 + 0.005 * k)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = k, cost
    return best


_TICKETS = 1 << 16
_decode_tickets = {}


def decode_tc_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tensor-core decode kernel takes these sizes (bfloat16, head size 64 or 128,
    groups up to 16, pages that divide 64)."""
    if dtype != torch.bfloat16:
        return False
    return bool(fn("pb_decode_tc_supported")(BF16, n_heads, n_kv_heads, head_dim, page_size))


def paged_attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                           partial: torch.Tensor, block_table: torch.Tensor, kv_len: torch.Tensor, scale: float,
                           window: Optional[int], n_splits: int, tensor_cores: Optional[bool] = None,
                           fused: Optional[bool] = None) -> None:
    """One query token per sequence: q, out [S, Hq, D].  ``partial`` is float32 scratch of at
    least S * Hq * n_splits * (D + 2) elements.  ``tensor_cores``: None picks the tensor-core
    kernel where it applies, False forces the CUDA-core kernel, True insists.  ``fused``: the
    tensor-core kernel finishes the job itself (a single split writes the result; of several the
    last one to finish merges) instead of a second kernel.  None: only for a single split, where
    it saves a launch; with several splits the ticket and fences cost what the combine kernel costs
    (measured: 5.04 vs 4.99 ms per step at batch 8)."""
    _cuda(q, k_pool, v_pool, out, partial, block_table, kv_len)
    _check_against(k_pool)
    s, hq, d = q.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and out.shape == q.shape and kv_len.numel() == s
    assert k_pool.dtype == q.dtype and v_pool.dtype == q.dtype and out.dtype == q.dtype
    assert block_table.dtype == torch.int32 and kv_len.dtype == torch.int32 and block_table.shape[0] == s
    assert partial.dtype == torch.float32 and partial.numel() >= s * hq * n_splits * (d + 2)
    if tensor_cores is None:
        tensor_cores = decode_tc_supported(q.dtype, hq, hkv, d, page_size)
    if fused is None:
        fused = n_splits == 1
    if tensor_cores and fused and n_splits <= 64 and s * hkv <= _TICKETS:
        tickets = _decode_tickets.get(q.device)
        if tickets is None:
            tickets = _decode_tickets[q.device] = torch.zeros(_TICKETS, dtype=torch.int32, device=q.device)
        check(fn("pb_paged_attention_decode_tc_fused")(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(partial),
                                                       _p(tickets), _p(block_table), block_table.shape[1], _p(kv_len), s, hq,
                                                       hkv, d, page_size, float(scale), int(window or 0), n_splits, stream()),
              "paged_attention_decode_tc_fused")
        return
    name = "pb_paged_attention_decode_tc" if tensor_cores else "pb_paged_attention_decode"
    check(fn(name)(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(partial),
                   _p(block_table), block_table.shape[1], _p(kv_len), s, hq, hkv, d, page_size,
                   float(scale), int(window or 0), n_splits, stream()), name[3:], kernels=2)


# A step of single tokens can leave the per-head norm, the rotation and the cache write of its projected rows to
# the attention kernel (one launch less per layer in a chain of dependent launches).  PULSAR_FUSED_QK=0: a kernel
# of its own does them, as in every other step.
FUSED_QK = os.environ.get("PULSAR_FUSED_QK", "1") != "0"


def decode_qkv_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, rotary: int, page_size: int) -> bool:
    """Whether ``paged_attention_decode_qkv`` takes these sizes: those of the tensor-core decode kernel, heads of
    their own keys and values, the whole head rotating."""
    return bool(FUSED_QK and n_kv_heads > 0 and rotary == head_dim
                and decode_tc_supported(dtype, n_heads, n_kv_heads, head_dim, page_size))


def paged_attention_decode_qkv(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                               cos: torch.Tensor, sin: torch.Tensor, eps: float, slots: torch.Tensor, k_pool: torch.Tensor,
                               v_pool: torch.Tensor, out: torch.Tensor, partial: torch.Tensor, block_table: torch.Tensor,
                               kv_len: torch.Tensor, scale: float, window: Optional[int], n_splits: int,
                               fused: Optional[bool] = None) -> None:
    """Decode attention straight from the projected rows ``qkv`` [S, (Hq + 2 Hkv) * D] (bfloat16): the kernel
    normalises and rotates the query heads and the newest key itself and writes that key and the value to
    ``slots`` of their pools before it reads them.  ``out`` [S, Hq, D]; the rest as ``paged_attention_decode``."""
    _cuda(qkv, q_weight, k_weight, cos, sin, slots, k_pool, v_pool, out, partial, block_table, kv_len)
    _check_against(k_pool)
    s, hq, d = out.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and qkv.shape == (s, (hq + 2 * hkv) * d) and kv_len.numel() == s
    assert qkv.dtype == torch.bfloat16 and k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype and out.dtype == qkv.dtype
    assert cos.shape == (s, d // 2) and sin.shape == cos.shape and cos.dtype == torch.float32 and sin.dtype == torch.float32
    assert slots.dtype == torch.int32 and slots.numel() == s
    assert block_table.dtype == torch.int32 and kv_len.dtype == torch.int32 and block_table.shape[0] == s
    assert partial.dtype == torch.float32 and partial.numel() >= s * hq * n_splits * (d + 2)
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == d)
    if fused is None:
        fused = n_splits == 1
    tickets = None
    if fused and n_splits <= 64 and s * hkv <= _TICKETS:
        tickets = _decode_tickets.get(qkv.device)
        if tickets is None:
            tickets = _decode_tickets[qkv.device] = torch.zeros(_TICKETS, dtype=torch.int32, device=qkv.device)
    check(fn("pb_paged_attention_decode_tc_qkv")(code(qkv.dtype), _p(qkv), _p(q_weight), _p(k_weight), _p(cos), _p(sin), float(eps),
                                                 _p(slots), _p(k_pool), _p(v_pool), _p(out), _p(partial), _p(tickets),
                                                 _p(block_table), block_table.shape[1], _p(kv_len), s, hq, hkv, d, page_size,
                                                 float(scale), int(window or 0), n_splits, stream()),
          "paged_attention_decode_tc_qkv", kernels=1 if tickets is not None else 2)


def prefill_tc_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(fn("pb_prefill_tc_supported")(BF16, n_heads, n_kv_heads, head_dim, page_size))


def prefill_tc_tiles(q_lens) -> int:
    """Blocks along the query axis: each sequence's new tokens in tiles of 64."""
    tile = fn("pb_prefill_tc_tile")()
    return sum(-(-int(n) // tile) for n in q_lens)


def paged_attention_prefill_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                               block_table: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor, n_q_tiles: int,
                               scale: float, window: Optional[int]) -> None:
    """Tensor-core attention for a ragged batch of portions (bfloat16, head size 64 or 128)."""
    _cuda(q, k_pool, v_pool, out, block_table, cu_q, kv_len)
    _check_against(k_pool)
    n, hq, d = q.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and out.shape == q.shape
    assert k_pool.dtype == q.dtype and v_pool.dtype == q.dtype and out.dtype == q.dtype
    assert block_table.dtype == torch.int32 and cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    s = kv_len.numel()
    assert cu_q.numel() == s + 1 and block_table.shape[0] == s
    check(fn("pb_paged_attention_prefill_tc")(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(block_table),
                                              block_table.shape[1], _p(cu_q), _p(kv_len), s, n_q_tiles, hq, hkv, d,
                                              page_size, float(scale), int(window or 0), stream()),
          "paged_attention_prefill_tc")


def prefill_tcgen05_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(fn("pb_prefill_tcgen05_supported")(BF16, n_heads, n_kv_heads, head_dim, page_size))


def prefill_tcgen05_tiles(q_lens) -> int:
    """Blocks along the query axis: each sequence's new tokens in tiles of 128."""
    tile = fn("pb_prefill_tcgen05_tile")()
    return sum(-(-int(n) // tile) for n in q_lens)


def prefill_tcgen05_error() -> int:
    """0 unless a block of the tcgen05 attention ever gave up a bounded wait (synchronises)."""
    return int(fn("pb_prefill_tcgen05_error")())


def paged_attention_prefill_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                                    block_table: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor, n_q_tiles: int,
                                    scale: float, window: Optional[int]) -> None:
    """tcgen05 attention for a ragged batch of portions (bfloat16, head size 128, pages of 8 or more
    tokens).  Pool rows that were never written must hold finite values."""
    _cuda(q, k_pool, v_pool, out, block_table, cu_q, kv_len)
    _check_against(k_pool)
    n, hq, d = q.shape
    pages, hkv, page_size, d2 = k_pool.shape
    assert d2 == d and v_pool.shape == k_pool.shape and out.shape == q.shape
    assert q.is_contiguous() and k_pool.is_contiguous() and v_pool.is_contiguous() and out.is_contiguous()
    assert k_pool.dtype == q.dtype and v_pool.dtype == q.dtype and out.dtype == q.dtype
    assert block_table.dtype == torch.int32 and cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    s = kv_len.numel()
    assert cu_q.numel() == s + 1 and block_table.shape[0] == s
    check(fn("pb_paged_attention_prefill_tcgen05")(code(q.dtype), _p(q), _p(k_pool), _p(v_pool), _p(out), _p(block_table),
                                                   block_table.shape[1], _p(cu_q), _p(kv_len), n, s, n_q_tiles, pages, hq,
                                                   hkv, d, page_size, float(scale), int(window or 0), stream()),
          "paged_attention_prefill_tcgen05")


def attention(ctx, q: torch.Tensor, cache, out: torch.Tensor, scale: float, window: Optional[int]) -> None:
    """Attention of the step's query tokens over their pages.  ``cache`` is a CacheView
    (pools, block table), ``ctx`` the StepContext (cu_q, kv_len, seq_of_token).  A step of
    single tokens only takes a split-key decode kernel; anything else the tcgen05 kernel where it
    applies (bfloat16, head size 128, pages of 8 or more), else the mma.sync kernel (bfloat16, head
    size 64 or 128), else the generic kernel.  ``PULSAR_ATTENTION=mma`` leaves the tcgen05 kernel out."""
    if ctx.all_decode:
        n_splits = decode_splits(ctx.n_seqs, cache.k_pool.shape[1], cache.block_table.shape[1] * cache.k_pool.shape[2])
        partial = ctx.scratch("attn.partial", (ctx.n_seqs * q.shape[1] * n_splits * (q.shape[2] + 2),), torch.float32)
        paged_attention_decode(q, cache.k_pool, cache.v_pool, out, partial, cache.block_table, ctx.kv_len, scale,
                               window, n_splits)
        return
    hkv, page_size = cache.k_pool.shape[1], cache.k_pool.shape[2]
    use_tcgen05 = ATTENTION_BACKEND != "mma" and prefill_tcgen05_supported(q.dtype, q.shape[1], hkv, q.shape[2], page_size)
    if use_tcgen05 or prefill_tc_supported(q.dtype, q.shape[1], hkv, q.shape[2], page_size):
        # The scheduler puts the decoded tokens of a mixed step first: those sequences take the decode kernel
        # (a tile of 64 or 128 query rows for one token would waste the tensor cores on every key tile), the
        # portions behind them the prefill kernel, over the same arrays.
        q_lens = ctx.host.q_lens
        n_dec = 0
        while n_dec < len(q_lens) and q_lens[n_dec] == 1:
            n_dec += 1
        table, cu_q, kv_len = cache.block_table, ctx.cu_q, ctx.kv_len
        if n_dec > 0:
            n_splits = decode_splits(n_dec, hkv, table.shape[1] * page_size)
            partial = ctx.scratch("attn.partial", (n_dec * q.shape[1] * n_splits * (q.shape[2] + 2),), torch.float32)
            paged_attention_decode(q[:n_dec], cache.k_pool, cache.v_pool, out[:n_dec], partial, table[:n_dec], kv_len[:n_dec],
                                   scale, window, n_splits)
            table, cu_q, kv_len, q_lens = table[n_dec:], cu_q[n_dec:], kv_len[n_dec:], q_lens[n_dec:]
        if use_tcgen05:
            paged_attention_prefill_tcgen05(q, cache.k_pool, cache.v_pool, out, table, cu_q, kv_len,
                                            prefill_tcgen05_tiles(q_lens), scale, window)
        else:
            paged_attention_prefill_tc(q, cache.k_pool, cache.v_pool, out, table, cu_q, kv_len, prefill_tc_tiles(q_lens),
                                       scale, window)
        return
    paged_attention_generic(q, cache.k_pool, cache.v_pool, out, cache.block_table, ctx.cu_q, ctx.kv_len,
                            ctx.seq_of_token, scale, window)
