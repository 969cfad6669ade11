#!/usr/bin/env python3
"""Makes ``tests/golden/reference_kernels.safetensors`` with the reference's own CUDA kernels.

    python baseline/build_reference.py --src /path/to/cosmonomic-pulsar      # once, builds baseline/_ref
    python tests/golden/make_reference_kernel_golden.py --out tests/golden/reference_kernels.safetensors   # on a GPU

The reference's kernels are compiled unchanged (baseline/build_reference.py) and called through the ops
that the reference registers itself (pulsar/ext/ops.cpp:8-74): ``rmsnorm``
(pulsar-core/src/kernels/rmsnorm.cu:17-51), ``rope`` (pulsar-core/src/kernels/rope.cu:27-52),
``write_kv`` (pulsar-core/src/kernels/paged_attention.cu:47-70) and the scalar attention
``attn_prefill_scalar`` / ``attn_decode_scalar`` (pulsar-core/src/kernels/paged_common.cu:21-142),
plus the tensor-core ``attn_prefill`` / ``attn_decode`` on one bfloat16 case.  Inputs are small,
drawn on the CPU from a seed and stored in the file beside the outputs (tensors ``<kind>.<case>.<name>``, the
cases' parameters as JSON in the file's metadata), so that the comparison (tests/test_plain.py) needs
neither a GPU nor the same random generator.

The attention ops hold UNROTATED keys and rotate key j to position j as they read it
(pulsar-core/inc/pulsar/ops.hpp:34-43); queries arrive rotated.  The file therefore stores the
unrotated keys; the plain implementation rotates them once, at their positions, and must then
agree with the op.
"""
import argparse
import json
import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def load_reference():
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    import pulsar.core  # noqa: F401  (registers torch.ops.pulsar.*)
    return torch.ops.pulsar


TENSORS = {}


def keep(name: str, t: torch.Tensor) -> str:
    TENSORS[name] = t.detach().to("cpu").contiguous().clone()
    return name


def attention_case(tag, ops, gen, dtype, hq, hkv, d, page, theta, seqs, scalar, decode=False):
    """seqs: list of (new tokens, context after them).  Keys and values of every context are
    scattered over shuffled pages with the reference's own write_kv."""
    dev = "cuda:0"
    n_pages_of = [-(-k // page) for _, k in seqs]
    total_pages = sum(n_pages_of) + 3
    order = torch.randperm(total_pages, generator=gen).tolist()
    tables, at = [], 0
    width = max(n_pages_of)
    for n in n_pages_of:
        tables.append(order[at:at + n] + [0] * (width - n))
        at += n
    k_pool = torch.zeros(total_pages, page, hkv, d, dtype=dtype, device=dev)
    v_pool = torch.zeros_like(k_pool)
    ks, vs, qs, q_pos = [], [], [], []
    for (nq, ctx), table in zip(seqs, tables):
        k = torch.randn(ctx, hkv, d, generator=gen).to(dtype)
        v = torch.randn(ctx, hkv, d, generator=gen).to(dtype)
        slots = torch.tensor([table[j // page] * page + j % page for j in range(ctx)], dtype=torch.int32)
        ops.write_kv(k_pool, v_pool, k.to(dev), v.to(dev), slots.to(dev))
        ks.append(k)
        vs.append(v)
        qs.append(torch.randn(nq, hq, d, generator=gen).to(dtype))      # taken as already rotated
        q_pos.append(list(range(ctx - nq, ctx)))
    q = torch.cat(qs, 0).to(dev)
    page_tables = torch.tensor(tables, dtype=torch.int32, device=dev)
    seqlens_k = torch.tensor([k for _, k in seqs], dtype=torch.int32, device=dev)
    layout = torch.tensor([[0, 0, -1]] * len(seqs), dtype=torch.int32, device=dev)       # the identity layout
    scale = 1.0 / math.sqrt(d)
    if decode:
        fn = ops.attn_decode_scalar if scalar else ops.attn_decode
        out = fn(q, k_pool, v_pool, page_tables, seqlens_k, layout, theta, scale)
    else:
        cu = [0]
        for nq, _ in seqs:
            cu.append(cu[-1] + nq)
        fn = ops.attn_prefill_scalar if scalar else ops.attn_prefill
        out = fn(q, k_pool, v_pool, page_tables, torch.tensor(cu, dtype=torch.int32, device=dev), seqlens_k, layout, theta, scale)
    torch.cuda.synchronize()
    return dict(op=("attn_decode" if decode else "attn_prefill") + ("_scalar" if scalar else ""),
                dtype=str(dtype).replace("torch.", ""), n_q_heads=hq, n_kv_heads=hkv, head_dim=d, page_size=page, theta=theta,
                scale=scale, seqs=[list(s) for s in seqs], q=keep(tag + ".q", torch.cat(qs, 0)),
                k_unrotated=keep(tag + ".k_unrotated", torch.cat(ks, 0)), v=keep(tag + ".v", torch.cat(vs, 0)),
                out=keep(tag + ".out", out))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "reference_kernels.safetensors"))
    args = ap.parse_args()
    ops = load_reference()
    gen = torch.Generator().manual_seed(20)
    dev = "cuda:0"
    cases = {"rmsnorm": [], "rope": [], "attention": []}

    for rows, width, eps in ((5, 48, 1e-5), (3, 80, 1e-6), (2, 16, 3e-6)):
        x = torch.randn(rows, width, generator=gen) * 3.0
        x[rows - 1].zero_()                                    # the row that only eps keeps finite
        w = 1.0 + 0.1 * torch.randn(width, generator=gen)
        y = ops.rmsnorm(x.to(dev), w.to(dev), eps)
        tag = f"rmsnorm.{len(cases['rmsnorm'])}"
        cases["rmsnorm"].append(dict(rows=rows, width=width, eps=eps, x=keep(tag + ".x", x), weight=keep(tag + ".weight", w),
                                     out=keep(tag + ".out", y)))

    for heads, seq, d, theta, positions in ((3, 7, 16, 1e4, [0, 1, 2, 5, 17, 1000, 40000]),
                                            (2, 5, 32, 1e6, [3, 4, 100000, 7, 1000003]),
                                            (1, 4, 48, 5e5, [0, 11, 12, 13])):
        x = torch.randn(heads, seq, d, generator=gen)
        pos = torch.tensor(positions, dtype=torch.int64)
        y = ops.rope(x.to(dev), pos.to(dev), theta)              # layout [heads, seq, head_dim] (rope.cu:56-89)
        tag = f"rope.{len(cases['rope'])}"
        cases["rope"].append(dict(heads=heads, seq=seq, head_dim=d, theta=theta, positions=positions, x=keep(tag + ".x", x),
                                  out=keep(tag + ".out", y)))

    f32, bf16 = torch.float32, torch.bfloat16
    specs = [
        # ragged batches of first portions and later portions, as pulsar/tests/test_paged_prefill.py:45-50 has them
        (f32, 4, 2, 16, 16, 1e4, [(16, 16), (7, 40), (33, 33), (1, 65)], True, False),
        (f32, 6, 3, 48, 16, 5e5, [(5, 21), (2, 2)], True, False),
        (f32, 4, 2, 32, 32, 1e6, [(9, 40), (20, 20)], True, False),
        # one query per sequence over ragged contexts (pulsar/tests/test_paged_attention.py:21-45)
        (f32, 4, 2, 16, 16, 1e4, [(1, c) for c in (1, 7, 16, 33, 65)], True, True),
        # the tensor-core kernels, bfloat16
        (bf16, 4, 2, 64, 16, 1e6, [(16, 16), (7, 40)], False, False),
        (bf16, 4, 2, 64, 16, 1e6, [(1, c) for c in (1, 7, 33)], False, True),
    ]
    for i, (dtype, hq, hkv, d, page, theta, seqs, scalar, decode) in enumerate(specs):
        cases["attention"].append(attention_case(f"attention.{i}", ops, gen, dtype, hq, hkv, d, page, theta, seqs, scalar, decode))
    from safetensors.torch import save_file
    meta = dict(made_by="tests/golden/make_reference_kernel_golden.py", device=torch.cuda.get_device_name(0),
                torch=torch.__version__, cases=json.dumps(cases))
    save_file(TENSORS, args.out, metadata=meta)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
