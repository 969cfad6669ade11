"""What every architecture's typed configuration shares: the error type, checked reads of
``config.json`` keys, and the reader of the file itself.

The reference reads eleven keys into ``PulsarModelConfig``
(pulsar/src/pulsar/checkpoint.py:22-51) and silently ignores the rest.  Here an architecture's
configuration (``pulsar_b200/models/<name>.py``) reads every key that changes its arithmetic and
rejects a value that the engine does not implement, instead of running a silently different model.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict


class ConfigError(ValueError):
    pass


def require(raw: Dict[str, Any], key: str, kind):
    """``raw[key]`` as ``kind`` (int or float); missing or of another type is a ConfigError."""
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    value = raw[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ConfigError(f"config.json: '{key}' must be an integer, found {value!r}")
    if kind is float and (isinstance(value, bool) or not isinstance(value, (int, float))):
        raise ConfigError(f"config.json: '{key}' must be a number, found {value!r}")
    return kind(value)


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)
