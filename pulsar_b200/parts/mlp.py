"""Dense gated feed-forward."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..config.registry import FEED_FORWARDS
from ..config.specs import FeedForwardSpec
from .base import FeedForward, StepContext, WeightSpec
from .norm import RMSNorm, accumulate_and_prepare


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """(silu(h Wg^T) * (h Wu^T)) Wd^T without bias (pulsar-core/src/model/qwen3.cpp:117-119).
    Gate and up are one fused product (rows: gate | up); the gating runs in float32 and
    rounds once."""

    def __init__(self, spec: FeedForwardSpec, prefix: str, dtype: torch.dtype):
        if spec.activation != "silu":
            raise ValueError(f"swiglu: activation '{spec.activation}' is not implemented (only 'silu')")
        self.spec, self.prefix, self.dtype = spec, prefix, dtype
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        s, p = self.spec, self.prefix
        return [WeightSpec(p + "gate_proj.weight", (s.intermediate, s.hidden)),
                WeightSpec(p + "up_proj.weight", (s.intermediate, s.hidden)),
                WeightSpec(p + "down_proj.weight", (s.hidden, s.intermediate))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"]

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def forward_normed(self, ctx: StepContext, residual: torch.Tensor, norm, next_norm=None) -> bool:
        s, n = self.spec, ctx.n_tokens
        if n > 16 or not isinstance(norm, RMSNorm) or self.dtype != torch.bfloat16:
            return False
        if not (ops.fused_projection_supported(n, self.w_gate_up, swiglu=True) and ops.fused_projection_supported(n, self.w_down)):
            return False
        act = ctx.scratch("mlp.act", (n, s.intermediate))
        prepared = ctx.prepared_norms.pop(id(norm), None) if ops.FUSED_NORM_MLP else None
        if prepared is None or not ops.linear_prenormed(prepared[0], prepared[1], norm.spec.eps, self.w_gate_up, act, swiglu=True):
            ops.gated_linear(ctx, norm.forward(ctx, residual, None), self.w_gate_up, act)
        ctx.prepared_norms.clear()              # the residual changes now
        if not accumulate_and_prepare(ctx, act, self.w_down, residual, next_norm):
            raise ops.KernelError("swiglu: the down projection refused sizes it had declared supported")
        return True

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        s, n = self.spec, ctx.n_tokens
        act = ctx.scratch("mlp.act", (n, s.intermediate))
        ops.gated_linear(ctx, h, self.w_gate_up, act)
        out = ctx.scratch("mlp.out", (n, s.hidden))
        ops.linear(act, self.w_down, out)
        return out
