"""Dense gated feed-forward."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..config.registry import FEED_FORWARDS
from ..config.specs import FeedForwardSpec
from .base import FeedForward, StepContext, WeightSpec


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

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        s, n = self.spec, ctx.n_tokens
        act = ctx.scratch("mlp.act", (n, s.intermediate))
        ops.gated_linear(ctx, h, self.w_gate_up, act)
        out = ctx.scratch("mlp.out", (n, s.hidden))
        ops.linear(act, self.w_down, out)
        return out
