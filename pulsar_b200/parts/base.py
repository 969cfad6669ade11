"""Interfaces of the parts a model is assembled from, and the context of one step.

A part is built from its specification alone, declares the tensors it wants by name
(``weight_specs``), receives them (``load``), declares what cache it needs
(``cache_need``, mixers only) and runs on the tokens of one step (``forward``).  It
never learns which model it is part of.

The residual stream of a step is float32 ``[N, hidden]``; a mixer or feed-forward
returns its contribution ``delta`` in the activation dtype and the next norm adds it
(in float32) while normalising.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import CacheNeed


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part wants.  role "matrix": kept in the compute dtype (bfloat16 or
    float32); "vector": kept in float32 (exact for bfloat16-stored values; a tensor
    stored in 32-bit stays so); "int": kept as int32."""
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"          # "normal": N(0, std); "ones_normal": 1 + N(0, 0.1); "zeros"
    optional: bool = False


@dataclass
class CacheView:
    """What a mixer sees of its cache entry in one step."""
    kind: str                                    # "paged_kv", "state", "none"
    pools: Optional[Dict[str, torch.Tensor]] = None   # cached tensor name -> [pages, heads, page, width]
    block_table: Optional[torch.Tensor] = None   # int32 [S, width], logical page -> page id
    slots: Optional[torch.Tensor] = None         # int32 [N], page * page_size + offset of each new token
    page_size: int = 0
    state: Optional[torch.Tensor] = None         # [max_requests, *state_shape]
    group: int = -1

    @property
    def k_pool(self) -> Optional[torch.Tensor]:
        return self.pools.get("k") if self.pools else None

    @property
    def v_pool(self) -> Optional[torch.Tensor]:
        return self.pools.get("v") if self.pools else None


@dataclass
class HostBatch:
    """The step's shape as the host knows it (no device read needed)."""
    q_lens: List[int]
    kv_lens: List[int]        # lengths after this step
    state_slots: List[int]

    @property
    def starts(self) -> List[int]:
        return [k - q for q, k in zip(self.q_lens, self.kv_lens)]


class StepContext:
    """Device arrays of one step plus scratch memory.  Built by the step function."""

    def __init__(self, runner, n_tokens: int, n_seqs: int, host: HostBatch):
        self.runner = runner
        self.dtype: torch.dtype = runner.dtype
        self.device = runner.device
        self.n_tokens, self.n_seqs = n_tokens, n_seqs
        self.host = host
        self.max_q_len = max(host.q_lens) if host.q_lens else 0
        self.max_kv_len = max(host.kv_lens) if host.kv_lens else 0
        self.all_decode = self.max_q_len == 1
        # int32 device arrays
        self.token_ids = self.positions = self.seq_of_token = None      # [N]
        self.position_axes = None               # [axes, N] where the model's positions have more than one axis, else None
        self.cu_q = self.kv_len = self.state_slots = None               # [S+1], [S], [S]
        self.logit_rows = None                                          # [R]
        self.group_tables: List[torch.Tensor] = []                      # per group [S, width]
        self.group_slots: List[torch.Tensor] = []                       # per group [N]
        self.shared: Dict[object, object] = {}                          # per-step tables shared by layers
        # What a product has prepared for the norm that follows it, by that norm's id: (residual * norm weight in
        # the activation dtype, parts of the rows' sums of squares).  Valid while nothing else touches the residual.
        self.prepared_norms: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.next_norm = None                   # the first norm of the block that runs after the current one, if known

    def scratch(self, tag: str, shape: Sequence[int], dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return self.runner.scratch(tag, tuple(shape), dtype or self.dtype)

    def cache(self, entry: int) -> CacheView:
        return self.runner.cache_view(self, entry)


class Part:
    """Common base: weights by name."""

    # A step of single tokens is captured into a CUDA graph and replayed while its shape stays the same.  A part
    # whose ``forward`` decides anything on the host from the step's contents (``ctx.host``: lengths, slots) would
    # replay stale decisions: it sets this to False, and a model that holds such a part is never captured.
    graph_safe: bool = True

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take the tensors named in ``weight_specs`` (already on the device, in the dtype
        their role asks for).  Parts may fuse or re-lay them here, once."""

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads (for roofline accounting)."""
        return 0


class Norm(Part):
    """forward(ctx, residual f32 [N, d], delta | None, rows | None) -> normalised [N or R, d]
    in the activation dtype; adds ``delta`` into ``residual`` first (unless rows are gathered)."""

    def forward(self, ctx: StepContext, residual: torch.Tensor, delta: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding:
    """tables(ctx) -> whatever its mixers consume, computed once per step from
    ``ctx.positions`` (or, for positions of several axes, ``ctx.position_axes``) and shared
    by all layers with an equal specification."""

    def tables(self, ctx: StepContext):
        raise NotImplementedError


class Mixer(Part):
    """forward(ctx, h [N, hidden], cache: CacheView) -> delta [N, hidden]."""

    def cache_need(self) -> CacheNeed:
        return CacheNeed.none()

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: CacheView) -> torch.Tensor:
        raise NotImplementedError

    def forward_normed(self, ctx: StepContext, residual: torch.Tensor, norm: Norm, cache: CacheView,
                       next_norm: Optional[Norm] = None) -> bool:
        """Optional short cut for steps of a few tokens: this part applies ``norm`` to the float32 ``residual``
        itself and adds its contribution to ``residual`` inside its last product, so that neither the norm nor the
        addition is a kernel of its own.  ``next_norm`` is the norm that will be applied to the residual next (by
        whoever follows); the part may prepare it (``ctx.prepared_norms``).  Returns False, having done nothing,
        when it cannot (the block then runs the norm and ``forward``)."""
        return False


class FeedForward(Part):
    """forward(ctx, h [N, hidden]) -> delta [N, hidden]."""

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_normed(self, ctx: StepContext, residual: torch.Tensor, norm: Norm, next_norm: Optional[Norm] = None) -> bool:
        """As ``Mixer.forward_normed``."""
        return False


class Block(Part):
    """An arrangement of norm, mixer and feed-forward.  forward(ctx, residual, delta,
    cache) -> the new pending delta (``residual`` is updated in place)."""

    mixer: Mixer
    parts: Tuple[Part, ...] = ()

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", True) for p in self.parts)

    def forward(self, ctx: StepContext, residual: torch.Tensor, delta: Optional[torch.Tensor],
                cache: CacheView) -> torch.Tensor:
        raise NotImplementedError
