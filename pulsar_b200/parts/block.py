"""Arrangements of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from ..config.specs import BlockSpec
from .base import Block, CacheView, StepContext, WeightSpec


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x))
    (pulsar-core/src/model/qwen3.cpp:77-121).  The additions happen inside the norm
    kernels, in float32, on the float32 residual stream."""

    def __init__(self, spec: BlockSpec, dtype: torch.dtype):
        self.spec = spec
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, spec.sub_prefix("mixer_norm"), dtype, "norm.mixer")
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, spec.sub_prefix("mixer"), dtype)
        self.feed_forward_norm = NORMS.get(spec.feed_forward_norm.kind)(
            spec.feed_forward_norm, spec.sub_prefix("feed_forward_norm"), dtype, "norm.ffn")
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, spec.sub_prefix("feed_forward"), dtype)
        self.parts = (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def weight_specs(self) -> List[WeightSpec]:
        return [w for p in self.parts for w in p.weight_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts:
            p.load(tensors)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts)

    def forward(self, ctx: StepContext, residual: torch.Tensor, delta: Optional[torch.Tensor],
                cache: CacheView) -> Optional[torch.Tensor]:
        # With nothing pending, a part may take the norm before it and the addition behind it into its own products
        # (steps of a few tokens); otherwise the norm kernel adds what is pending and normalises.
        if delta is not None or not self.mixer.forward_normed(ctx, residual, self.mixer_norm, cache, self.feed_forward_norm):
            ctx.prepared_norms.clear()
            h = self.mixer_norm.forward(ctx, residual, delta)
            delta = self.mixer.forward(ctx, h, cache)
        if delta is None and self.feed_forward.forward_normed(ctx, residual, self.feed_forward_norm, ctx.next_norm):
            return None
        ctx.prepared_norms.clear()
        h = self.feed_forward_norm.forward(ctx, residual, delta)
        return self.feed_forward.forward(ctx, h)
