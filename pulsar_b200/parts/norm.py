"""RMSNorm fused with the residual add that precedes it."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.registry import NORMS
from ..config.specs import NormSpec
from .base import Norm, StepContext, WeightSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * w in float32, one rounding on store
    (pulsar-core/src/kernels/rmsnorm.cu:29-49).  The weight is held in float32."""

    def __init__(self, spec: NormSpec, prefix: str, dtype: torch.dtype, tag: str = "norm"):
        self.spec, self.prefix, self.dtype, self.tag = spec, prefix, dtype, tag
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.prefix + "weight", (self.spec.size,), role="vector", init="ones_normal")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.prefix + "weight"]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx: StepContext, residual: torch.Tensor, delta: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = residual.shape[0] if rows is None else rows.numel()
        out = ctx.scratch(self.tag + (".rows" if rows is not None else ""), (n, self.spec.size))
        ops.add_rmsnorm(residual, delta, self.weight, self.spec.eps, out, rows=rows)
        return out


def accumulate_and_prepare(ctx: StepContext, a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, next_norm) -> bool:
    """residual += a @ w.T inside the product (a few tokens, bfloat16), and, where the norm that follows is an
    RMSNorm, that norm prepared by the same kernel and left in ``ctx.prepared_norms`` for whoever applies it
    (``ops.linear_accumulate`` / ``ops.linear_prenormed``).  False, having done nothing, when the product declines."""
    n, width = residual.shape
    if isinstance(next_norm, RMSNorm) and next_norm.spec.size == width and width % 16 == 0:
        tag = next_norm.tag
        prepared = ctx.scratch(tag + ".prepared", (n, width), torch.bfloat16)
        parts = ctx.scratch(tag + ".parts", (ops.norm_parts_numel(n, width),), torch.float32)
        if ops.linear_accumulate(a, w, residual, next_norm.weight, prepared, parts):
            ctx.prepared_norms[id(next_norm)] = (prepared, parts)
            return True
        return False
    return ops.linear_accumulate(a, w, residual)
