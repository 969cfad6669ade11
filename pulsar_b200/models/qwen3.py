"""Qwen3 dense: the architecture's typed configuration and its name in the registry.

Field names are the ``config.json`` keys.  The reference reads eleven of them
(pulsar/src/pulsar/checkpoint.py:36-51) and maps the prefix "qwen3" of a caller's string to its
Qwen3Model (pulsar-core/src/runtime/engine.cpp:43-84); here ``config.json`` names the class, every key
that changes the arithmetic is read, and ``model_spec()`` states the reference's block
(pulsar-core/src/model/qwen3.cpp:77-129) as data for the generic decoder.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, fields
from typing import Any, Dict, Optional

from ..config.model_config import ConfigError, require as _require
from ..config.registry import register_architecture
from ..config.specs import (BlockSpec, FeedForwardSpec, LayerCall, MixerSpec, ModelSpec, NormSpec,
                            PositionSpec)


@dataclass(frozen=True)
class Qwen3Config:
    """Qwen3 dense decoder.  Field names are the ``config.json`` keys."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: Optional[bool]
    eos_token_id: int
    max_position_embeddings: int
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    hidden_act: str
    attention_bias: bool
    initializer_range: float
    architecture: str = "Qwen3ForCausalLM"
    layer_types: Optional[tuple] = None        # per layer "full_attention" | "sliding_attention", where config.json lists them

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen3Config":
        heads = _require(raw, "num_attention_heads", int)
        hidden = _require(raw, "hidden_size", int)
        # head_dim defaults to hidden/heads (pulsar/src/pulsar/checkpoint.py:46).
        head_dim = raw.get("head_dim") or hidden // heads
        eos = raw.get("eos_token_id", -1)
        if isinstance(eos, (list, tuple)):      # scripts/migrate.py:28-34 resolves a list to its first id
            eos = eos[0] if eos else -1
        # Newer config.json files carry the rotary settings as one dictionary, ``rope_parameters``
        # ({"rope_theta": ..., "rope_type": "default"}), in place of ``rope_theta`` / ``rope_scaling``.
        params = raw.get("rope_parameters")
        if isinstance(params, dict):
            kind = params.get("rope_type", params.get("type", "default"))
            if kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_parameters of type '{kind}' (rope_scaling) is not implemented by this engine")
            if "rope_theta" not in raw and "rope_theta" in params:
                raw = dict(raw, rope_theta=params["rope_theta"])
        cfg = cls(
            vocab_size=_require(raw, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_require(raw, "intermediate_size", int),
            num_hidden_layers=_require(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=int(raw.get("num_key_value_heads") or heads),
            head_dim=int(head_dim),
            rope_theta=_require(raw, "rope_theta", float),
            rms_norm_eps=_require(raw, "rms_norm_eps", float),
            tie_word_embeddings=raw.get("tie_word_embeddings"),
            eos_token_id=-1 if eos is None else int(eos),
            max_position_embeddings=int(raw.get("max_position_embeddings") or 0),
            use_sliding_window=bool(raw.get("use_sliding_window", False)),
            sliding_window=None if raw.get("sliding_window") is None else int(raw["sliding_window"]),
            max_window_layers=int(raw.get("max_window_layers") or 0),
            hidden_act=str(raw.get("hidden_act", "silu")),
            attention_bias=bool(raw.get("attention_bias", False)),
            initializer_range=float(raw.get("initializer_range", 0.02)),
            layer_types=None if raw.get("layer_types") is None else tuple(str(t) for t in raw["layer_types"]),
        )
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: rope_scaling is not implemented by this engine; found "
                              f"{raw['rope_scaling']!r}")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        positive = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim")
        for name in positive:
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: '{name}' must be positive, found {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("config.json: num_attention_heads "
                              f"({self.num_attention_heads}) is not a multiple of num_key_value_heads "
                              f"({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even for rotary embedding")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not implemented (only 'silu')")
        if self.attention_bias:
            raise ConfigError("config.json: attention_bias=true is not implemented")
        if not (self.rms_norm_eps > 0.0) or not (self.rope_theta > 0.0):
            raise ConfigError("config.json: rms_norm_eps and rope_theta must be positive")
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            raise ConfigError("config.json: use_sliding_window=true needs a positive sliding_window")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(f"config.json: layer_types names {len(self.layer_types)} layers, num_hidden_layers is "
                                  f"{self.num_hidden_layers}")
            for i, kind in enumerate(self.layer_types):
                if kind not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"config.json: layer_types[{i}] = '{kind}' is not implemented "
                                      "(known: full_attention, sliding_attention)")
                if kind == "sliding_attention" and (self.sliding_window is None or self.sliding_window <= 0):
                    raise ConfigError(f"config.json: layer_types[{i}] slides but sliding_window is not a positive number")

    def to_dict(self) -> Dict[str, Any]:
        out = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "architecture"}
        out["architectures"] = [self.architecture]
        out["model_type"] = "qwen3"
        out["rope_scaling"] = None
        if self.layer_types is None:
            del out["layer_types"]
        else:
            out["layer_types"] = list(self.layer_types)
        return out

    def layer_window(self, layer: int) -> Optional[int]:
        """Where config.json lists ``layer_types`` they decide; else layers with index >=
        max_window_layers slide when use_sliding_window is set."""
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        return self.sliding_window if layer >= self.max_window_layers else None

    def model_spec(self) -> ModelSpec:
        """The Qwen3 block of the reference (pulsar-core/src/model/qwen3.cpp:77-129) as data."""
        position = PositionSpec("rope", self.head_dim, self.head_dim, self.rope_theta)
        blocks = []
        for i in range(self.num_hidden_layers):
            mixer = MixerSpec(
                kind="attention", hidden=self.hidden_size, n_heads=self.num_attention_heads,
                n_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                scale=1.0 / math.sqrt(self.head_dim),        # qwen3.cpp:47
                window=self.layer_window(i),
                qk_norm_eps=self.rms_norm_eps,                # qwen3.cpp:88-91: same eps as the layer norms
                position=position)
            ffn = FeedForwardSpec("swiglu", self.hidden_size, self.intermediate_size, self.hidden_act)
            norm = NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps)
            blocks.append(BlockSpec(
                kind="prenorm", mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm,
                weight_prefix=f"model.layers.{i}.",
                names=(("mixer", "self_attn."), ("feed_forward", "mlp."),
                       ("mixer_norm", "input_layernorm."), ("feed_forward_norm", "post_attention_layernorm."))))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden=self.hidden_size,
            blocks=tuple(blocks),
            run_order=tuple(LayerCall(i, i) for i in range(self.num_hidden_layers)),
            final_norm=NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps),
            tie_word_embeddings=self.tie_word_embeddings, init_std=self.initializer_range,
            eos_token_id=self.eos_token_id)


@register_architecture("Qwen3ForCausalLM", "qwen3")
def qwen3_config(raw: dict) -> Qwen3Config:
    return Qwen3Config.from_dict(raw)
