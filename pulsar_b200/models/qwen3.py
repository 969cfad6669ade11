"""Qwen3 dense: the architecture's name in the registry."""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture


@register_architecture("Qwen3ForCausalLM", "qwen3")
def qwen3_config(raw: dict) -> Qwen3Config:
    """The reference maps the prefix "qwen3" of a caller's string to its Qwen3Model
    (pulsar-core/src/runtime/engine.cpp:43-84); here ``config.json`` names the class."""
    return Qwen3Config.from_dict(raw)
