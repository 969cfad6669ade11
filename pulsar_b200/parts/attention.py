"""Grouped-query attention over a paged key/value cache."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..cache.manager import CacheNeed
from ..config.registry import MIXERS, POSITIONS
from ..config.specs import MixerSpec
from .base import CacheView, Mixer, StepContext, WeightSpec
from .norm import RMSNorm, accumulate_and_prepare


@MIXERS.register("attention")
class Attention(Mixer):
    """q/k/v projection without bias (one fused product), optional per-head RMSNorm of
    q and k before rotation, rotation at the tokens' explicit positions, write of k and v
    into the pages, attention over the pages (causal, optional window, grouped heads),
    output projection (pulsar-core/src/model/qwen3.cpp:81-114;
    pulsar-core/src/model/paged_forward.cpp:30-80).

    Keys are stored rotated, once, at their absolute position.  With ``own_kv`` False the
    mixer has no k/v projection and attends over pages another layer wrote this step.
    """

    def __init__(self, spec: MixerSpec, prefix: str, dtype: torch.dtype):
        if spec.n_heads <= 0 or spec.n_kv_heads <= 0 or spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"attention: {spec.n_heads} query heads cannot be grouped over {spec.n_kv_heads} kv heads")
        if spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"attention: head_dim {spec.head_dim} must be a multiple of 16, at most 256")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("attention: window must be positive")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.position = POSITIONS.get(spec.position.kind)(spec.position) if spec.position is not None else None
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    # ---------------------------------------------------------------- weights
    def weight_specs(self) -> List[WeightSpec]:
        s, p = self.spec, self.prefix
        specs = [WeightSpec(p + "q_proj.weight", (s.n_heads * s.head_dim, s.hidden))]
        if s.own_kv:
            specs += [WeightSpec(p + "k_proj.weight", (s.n_kv_heads * s.head_dim, s.hidden)),
                      WeightSpec(p + "v_proj.weight", (s.n_kv_heads * s.head_dim, s.hidden))]
        specs.append(WeightSpec(p + "o_proj.weight", (s.hidden, s.n_heads * s.head_dim)))
        if s.qk_norm_eps is not None:
            specs.append(WeightSpec(p + "q_norm.weight", (s.head_dim,), role="vector", init="ones_normal"))
            if s.own_kv:
                specs.append(WeightSpec(p + "k_norm.weight", (s.head_dim,), role="vector", init="ones_normal"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s, p = self.spec, self.prefix
        parts = [tensors[p + "q_proj.weight"]]
        if s.own_kv:
            parts += [tensors[p + "k_proj.weight"], tensors[p + "v_proj.weight"]]
        self.w_qkv = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0]   # rows: q | k | v
        self.w_o = tensors[p + "o_proj.weight"]
        if s.qk_norm_eps is not None:
            self.q_norm = tensors[p + "q_norm.weight"]
            self.k_norm = tensors.get(p + "k_norm.weight")

    def weight_bytes(self) -> int:
        ts = [self.w_qkv, self.w_o, self.q_norm, self.k_norm]
        return sum(t.numel() * t.element_size() for t in ts if t is not None)

    def cache_need(self) -> CacheNeed:
        return CacheNeed.paged_kv(self.spec.n_kv_heads, self.spec.head_dim, self.spec.window)

    # ---------------------------------------------------------------- one step
    def forward(self, ctx: StepContext, h: torch.Tensor, cache: CacheView) -> torch.Tensor:
        s = self.spec
        n = ctx.n_tokens
        n_kv = s.n_kv_heads if s.own_kv else 0
        qkv = ctx.scratch("attn.qkv", (n, (s.n_heads + 2 * n_kv) * s.head_dim))
        ops.linear(h, self.w_qkv, qkv)
        o = self._attend(ctx, qkv, cache)
        out = ctx.scratch("attn.out", (n, s.hidden))
        ops.linear(o.view(n, s.n_heads * s.head_dim), self.w_o, out)
        return out

    def forward_normed(self, ctx: StepContext, residual: torch.Tensor, norm, cache: CacheView, next_norm=None) -> bool:
        s = self.spec
        n = ctx.n_tokens
        if n > 16 or not isinstance(norm, RMSNorm) or self.dtype != torch.bfloat16:
            return False
        if not (ops.fused_projection_supported(n, self.w_qkv) and ops.fused_projection_supported(n, self.w_o)):
            return False
        n_kv = s.n_kv_heads if s.own_kv else 0
        qkv = ctx.scratch("attn.qkv", (n, (s.n_heads + 2 * n_kv) * s.head_dim))
        prepared = ctx.prepared_norms.pop(id(norm), None)
        if prepared is None or not ops.linear_prenormed(prepared[0], prepared[1], norm.spec.eps, self.w_qkv, qkv):
            ops.linear(norm.forward(ctx, residual, None), self.w_qkv, qkv)
        o = self._attend(ctx, qkv, cache)
        ctx.prepared_norms.clear()              # the residual changes now
        if not accumulate_and_prepare(ctx, o.view(n, s.n_heads * s.head_dim), self.w_o, residual,
                                      next_norm if ops.FUSED_NORM_MLP else None):
            raise ops.KernelError("attention: the output projection refused sizes it had declared supported")
        return True

    def _attend(self, ctx: StepContext, qkv: torch.Tensor, cache: CacheView) -> torch.Tensor:
        """Per-head norm, rotation and cache write of the projected row, then attention: o [N, heads, head_dim]."""
        s = self.spec
        n = ctx.n_tokens
        n_kv = s.n_kv_heads if s.own_kv else 0
        q = ctx.scratch("attn.q", (n, s.n_heads, s.head_dim))
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
            rotary = s.position.rotary_dim
        else:
            cos = sin = ctx.scratch("attn.norope", (n, 0), torch.float32)
            rotary = 0
        # (A lone sequence keeps the kernel of its own: its keys are cut into so many splits that every block's share
        # is short, and the norm and rotation in each block's start then cost more than the launch they save:
        # 2.990 against 2.973 ms per step; with two sequences and more the one kernel is ahead by 1.1 to 1.4 %.)
        if (ctx.all_decode and ctx.n_seqs >= 2 and self.position is not None and qkv.dtype == torch.bfloat16
                and ops.decode_qkv_supported(qkv.dtype, s.n_heads, n_kv, s.head_dim, rotary, cache.page_size)):
            # a step of single tokens: the attention kernel normalises, rotates and writes the cache itself
            o = ctx.scratch("attn.o", (n, s.n_heads, s.head_dim))
            n_splits = ops.decode_splits(ctx.n_seqs, n_kv, cache.block_table.shape[1] * cache.page_size)
            partial = ctx.scratch("attn.partial", (ctx.n_seqs * s.n_heads * n_splits * (s.head_dim + 2),), torch.float32)
            ops.paged_attention_decode_qkv(qkv, self.q_norm, self.k_norm, cos, sin, s.qk_norm_eps or 0.0, cache.slots, cache.k_pool,
                                           cache.v_pool, o, partial, cache.block_table, ctx.kv_len, s.scale, s.window, n_splits)
            return o
        ops.qk_norm_rope_write(qkv, q, cache.k_pool if n_kv else None, cache.v_pool if n_kv else None,
                               cache.slots if n_kv else None, cos, sin, self.q_norm, self.k_norm,
                               s.qk_norm_eps or 0.0, s.n_heads, n_kv, s.head_dim, rotary, cache.page_size)
        o = ctx.scratch("attn.o", (n, s.n_heads, s.head_dim))
        ops.attention(ctx, q, cache, o, s.scale, s.window)
        return o
