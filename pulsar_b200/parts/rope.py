"""Rotary position encoding from an explicit array of positions."""
from __future__ import annotations

import math
from typing import Tuple

import torch

from .. import ops
from ..config.registry import POSITIONS
from ..config.specs import PositionSpec
from .base import PositionEncoding, StepContext


@POSITIONS.register("rope")
class RotaryEmbedding(PositionEncoding):
    """cos/sin of p_t * theta^(-2j/rotary_dim) for the tokens of a step, computed once per
    step and shared by every layer with an equal specification.  The frequency table is
    float64 and carries quadrants per position, as the reference's does
    (pulsar-core/inc/pulsar/rope.hpp:52-69): its relative error is scaled by the position."""

    def __init__(self, spec: PositionSpec):
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and within head_dim {spec.head_dim}")
        self.spec = spec
        self._table = {}

    def quadrants_per_position(self, device) -> torch.Tensor:
        t = self._table.get(device)
        if t is None:
            half = self.spec.rotary_dim // 2
            values = [self.spec.theta ** (-2.0 * j / self.spec.rotary_dim) * (2.0 / math.pi) for j in range(half)]
            t = torch.tensor(values, dtype=torch.float64).to(device)
            self._table[device] = t
        return t

    def tables(self, ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor]:
        key = ("rope", self.spec)
        got = ctx.shared.get(key)
        if got is None:
            half = self.spec.rotary_dim // 2
            tag = f"rope.{self.spec.rotary_dim}.{self.spec.theta}"
            cos = ctx.scratch(tag + ".cos", (ctx.n_tokens, half), torch.float32)
            sin = ctx.scratch(tag + ".sin", (ctx.n_tokens, half), torch.float32)
            ops.rope_table(ctx.positions, self.quadrants_per_position(ctx.device), cos, sin)
            got = ctx.shared[key] = (cos, sin)
        return got
