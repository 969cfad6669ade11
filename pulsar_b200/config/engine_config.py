"""Flat engine configuration with the reference's names and defaults.

The reference builds an ``EngineConfig`` from a flat ``dict`` and rejects unknown
keys with the sorted list (pulsar/ext/engine.cpp:168-224, 255-287;
pulsar-core/inc/pulsar/runtime/engine.hpp:221-320).  The keys kept here are the ones
whose concept survives without eviction/recall; ``num_pages`` sizes the pool directly
and, when absent, the reference's rule ``max_sessions * active_buffer_size /
page_size`` (pulsar-core/src/runtime/engine.cpp:141) applies.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Dict, Optional

from .model_config import ConfigError

_DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass
class EngineConfig:
    page_size: int = 16
    num_pages: Optional[int] = None
    max_sessions: int = 8
    active_buffer_size: int = 32768
    max_running: int = 8
    max_chunk_size: int = 512        # token budget of one step (decoded tokens count too)
    dtype: str = "bfloat16"
    device: str = "cuda:0"
    eos_id: int = -1
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int = -1
    cuda_graphs: bool = True

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "EngineConfig":
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(raw) - known)
        if unknown:
            raise ConfigError(f"EngineConfig: unknown keys {unknown}; known keys: {sorted(known)}")
        cfg = cls(**raw)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.dtype not in _DTYPES:
            raise ConfigError(f"EngineConfig: dtype '{self.dtype}' is not one of {sorted(set(_DTYPES))}")
        self.dtype = _DTYPES[self.dtype]
        if self.page_size <= 0:
            raise ConfigError("EngineConfig: page_size must be > 0")
        if self.num_pages is None:
            if self.active_buffer_size % self.page_size:
                raise ConfigError("EngineConfig: active_buffer_size must be a multiple of page_size")
            self.num_pages = self.max_sessions * self.active_buffer_size // self.page_size
        if self.num_pages <= 0:
            raise ConfigError("EngineConfig: num_pages must be > 0")
        if self.max_running <= 0 or self.max_chunk_size <= 0:
            raise ConfigError("EngineConfig: max_running and max_chunk_size must be > 0")
        if not (0.0 < self.top_p <= 1.0):
            raise ConfigError("EngineConfig: top_p must lie in (0, 1]")
        if self.top_k < 0:
            raise ConfigError("EngineConfig: top_k must be >= 0")
