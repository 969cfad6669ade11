"""Registries: architecture name -> configuration, part kind -> part class.

The reference picks its model class by a prefix of a caller-supplied string
(pulsar-core/src/runtime/engine.cpp:43-84).  Here the name comes from
``config.json`` (``architectures[0]``, else ``model_type``), and every registry is
open: a test or a user registers a new architecture, mixer, feed-forward, norm,
position encoding or block arrangement without touching the package.
"""
from __future__ import annotations

from typing import Any, Callable, Dict

from .model_config import ConfigError


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Any] = {}

    def register(self, name: str, item: Any = None, *, replace: bool = False):
        def put(obj):
            if name in self._items and not replace and self._items[name] is not obj:
                raise ValueError(f"{self.what} '{name}' is already registered")
            self._items[name] = obj
            return obj
        return put if item is None else put(item)

    def unregister(self, name: str) -> None:
        self._items.pop(name, None)

    def get(self, name: str):
        if name not in self._items:
            raise ConfigError(f"unknown {self.what} '{name}'; known: {sorted(self._items)}")
        return self._items[name]

    def names(self):
        return sorted(self._items)

    def __contains__(self, name: str) -> bool:
        return name in self._items


ARCHITECTURES = Registry("architecture")      # name -> callable(raw config dict) -> object with .model_spec()
MIXERS = Registry("mixer")                    # kind -> class(spec: MixerSpec, prefix, dtype)
FEED_FORWARDS = Registry("feed-forward")      # kind -> class(spec: FeedForwardSpec, prefix, dtype)
NORMS = Registry("norm")                      # kind -> class(spec: NormSpec, prefix, dtype)
POSITIONS = Registry("position encoding")     # kind -> class(spec: PositionSpec)
BLOCKS = Registry("block arrangement")        # kind -> class(spec: BlockSpec, dtype)


def architecture_name(raw: Dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        return str(archs[0])
    if raw.get("model_type"):
        return str(raw["model_type"])
    raise ConfigError("config.json: neither 'architectures' nor 'model_type' names the model")


def config_from_dict(raw: Dict[str, Any]):
    """Typed configuration of whatever architecture ``raw`` names."""
    return ARCHITECTURES.get(architecture_name(raw))(raw)


def register_architecture(*names: str) -> Callable:
    def put(factory):
        for n in names:
            ARCHITECTURES.register(n, factory)
        return factory
    return put
