"""Specifications of the parts a decoder is assembled from.

A specification is plain data: it carries every size and constant its part needs and
the ``kind`` under which the part's class is registered.  Architectures translate
their ``config.json`` into these; parts never see a ``config.json`` and never know
which model they are in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    kind: str            # "rmsnorm"
    size: int
    eps: float


@dataclass(frozen=True)
class PositionSpec:
    kind: str            # "rope"
    head_dim: int
    rotary_dim: int      # leading dims of each head that rotate (== head_dim for Qwen3)
    theta: float


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of a block.  ``kind`` "attention" is grouped-query attention over
    a paged key/value cache."""
    kind: str
    hidden: int
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0               # softmax scale
    window: Optional[int] = None     # None: all keys; w: keys p-w < j <= p
    qk_norm_eps: Optional[float] = None   # None: no per-head q/k norm
    position: Optional[PositionSpec] = None
    own_kv: bool = True              # False: attends over another layer's cache, has no k/v projection
    extra: Tuple[Tuple[str, object], ...] = ()   # free-form parameters of other kinds

    def option(self, name, default=None):
        return dict(self.extra).get(name, default)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str            # "swiglu"
    hidden: int
    intermediate: int
    activation: str = "silu"
    extra: Tuple[Tuple[str, object], ...] = ()

    def option(self, name, default=None):
        return dict(self.extra).get(name, default)


@dataclass(frozen=True)
class BlockSpec:
    """Arrangement of one layer.  ``kind`` "prenorm": x += mixer(norm1(x)); x += ffn(norm2(x))."""
    kind: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    weight_prefix: str                      # e.g. "model.layers.3."
    names: Tuple[Tuple[str, str], ...] = ()  # sub-prefixes: mixer, feed_forward, mixer_norm, feed_forward_norm

    def sub_prefix(self, part: str) -> str:
        return self.weight_prefix + dict(self.names)[part]


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run block ``block`` against cache entry ``cache``.
    A block may be named by several entries, and two entries may name one cache entry
    (the later one then reads what the earlier one wrote: its mixer has own_kv False)."""
    block: int
    cache: int


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    blocks: Tuple[BlockSpec, ...]
    run_order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: Optional[str] = "lm_head.weight"   # None: always tied
    tie_word_embeddings: Optional[bool] = None    # None: decided by the head tensor's presence
    init_std: float = 0.02
    eos_token_id: int = -1
    # What sits around the blocks.  Qwen3 dense uses none of it.
    embedding_multiplier: float = 1.0             # the embedding row is scaled by this before the first block
    logit_scale: float = 1.0                      # logits are scaled by this ...
    logit_softcap: Optional[float] = None         # ... and then capped: cap * tanh(logits / cap)
    position_axes: int = 1                        # axes of a token's position; axis 0 is its index in the sequence
    ignore: Tuple[str, ...] = ()                  # tensor-name patterns (fnmatch) that a folder may hold and nobody reads

    @property
    def n_cache_entries(self) -> int:
        return 1 + max(call.cache for call in self.run_order) if self.run_order else 0
