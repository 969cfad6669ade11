"""A decoder-only language model assembled from parts by a ``ModelSpec``."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .. import parts  # noqa: F401  (registers the built-in kinds)
from ..cache.manager import CacheNeed
from ..config.registry import BLOCKS, NORMS
from ..config.specs import ModelSpec
from ..parts.base import Part, StepContext, WeightSpec


class DecoderModel(Part):
    """embedding -> the blocks in ``run_order`` -> final norm at the wanted rows -> head
    (pulsar-core/src/model/paged_forward.cpp:82-94; pulsar-core/src/model/qwen3.cpp:123-129).

    The run order is data: an entry names a block and a cache entry.  A block may be named
    twice (its weights are shared, each call has a cache entry of its own) and two calls may
    name one cache entry (the second reads what the first wrote and must not own k/v).
    """

    def __init__(self, spec: ModelSpec, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype {dtype} must be float32 or bfloat16")
        if spec.position_axes < 1:
            raise ValueError("a model's positions have at least one axis (the index in the sequence)")
        if spec.logit_softcap is not None and not (spec.logit_softcap > 0.0):
            raise ValueError("logit_softcap must be positive")
        self.spec, self.dtype = spec, dtype
        self.blocks = [BLOCKS.get(b.kind)(b, dtype) for b in spec.blocks]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, spec.final_norm_name[: -len("weight")], dtype,
                                                          "norm.final")
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.tied = False
        needs: List[Optional[CacheNeed]] = [None] * spec.n_cache_entries
        for call in spec.run_order:
            if not (0 <= call.block < len(self.blocks)):
                raise ValueError(f"run order names block {call.block}, the model has {len(self.blocks)}")
            mixer = self.blocks[call.block].mixer
            need = mixer.cache_need()
            owns = getattr(mixer.spec, "own_kv", True)
            if needs[call.cache] is None:
                if not owns:
                    raise ValueError(f"cache entry {call.cache}: its first user must write it (own_kv)")
                needs[call.cache] = need
            else:
                if owns:
                    raise ValueError(f"cache entry {call.cache} is written by two layer calls")
                if need != needs[call.cache]:
                    raise ValueError(f"cache entry {call.cache}: reader needs {need}, writer made {needs[call.cache]}")
        if any(n is None for n in needs):
            raise ValueError("run order leaves a cache entry unused")
        self._needs = needs

    def cache_needs(self) -> List[CacheNeed]:
        return list(self._needs)

    @property
    def graph_safe(self) -> bool:
        """Whether a step of this model may be captured into a CUDA graph (every part says so)."""
        return all(getattr(b, "graph_safe", True) for b in self.blocks) and getattr(self.final_norm, "graph_safe", True)

    # ---------------------------------------------------------------- weights
    def weight_specs(self) -> List[WeightSpec]:
        s = self.spec
        specs = [WeightSpec(s.embed_name, (s.vocab_size, s.hidden))]
        for b in self.blocks:
            specs += b.weight_specs()
        specs += self.final_norm.weight_specs()
        if s.head_name is not None and s.tie_word_embeddings is not True:
            # Tied iff the head tensor is absent (pulsar-core/src/model/qwen3.cpp:51-53); a
            # config that says "not tied" makes the tensor mandatory.
            specs.append(WeightSpec(s.head_name, (s.vocab_size, s.hidden), optional=s.tie_word_embeddings is None))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embed = tensors[s.embed_name]
        for b in self.blocks:
            b.load(tensors)
        self.final_norm.load(tensors)
        head = tensors.get(s.head_name) if s.head_name is not None else None
        self.tied = head is None
        self.head = self.embed if head is None else head

    def weight_bytes(self, n_tokens: int = 0) -> int:
        """Bytes of weights one step reads: every block as often as the run order names
        it, the final norm, the head, and ``n_tokens`` rows of the embedding."""
        total = sum(self.blocks[c.block].weight_bytes() for c in self.spec.run_order)
        total += self.final_norm.weight_bytes() + self.head.numel() * self.head.element_size()
        return total + n_tokens * self.spec.hidden * self.embed.element_size()

    # ---------------------------------------------------------------- one step
    def forward(self, ctx: StepContext) -> torch.Tensor:
        """Logits float32 [len(ctx.logit_rows), vocab] for the tokens of ``ctx``."""
        s = self.spec
        residual = ctx.scratch("residual", (ctx.n_tokens, s.hidden), torch.float32)
        ops.embed(self.embed, ctx.token_ids, residual, s.embedding_multiplier)
        delta = None
        for i, call in enumerate(s.run_order):
            following = self.blocks[s.run_order[i + 1].block] if i + 1 < len(s.run_order) else None
            ctx.next_norm = getattr(following, "mixer_norm", None)
            delta = self.blocks[call.block].forward(ctx, residual, delta, ctx.cache(call.cache))
        rows = ctx.logit_rows
        logits = ctx.scratch("logits", (rows.numel(), s.vocab_size), torch.float32)
        if rows.numel():
            h = self.final_norm.forward(ctx, residual, delta, rows=rows)
            ops.linear(h, self.head, logits)
            if s.logit_scale != 1.0 or s.logit_softcap is not None:
                ops.scale_cap(logits, s.logit_scale, s.logit_softcap)
        return logits
