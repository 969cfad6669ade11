"""From a model folder to a model with weights on the device."""
from __future__ import annotations

import torch

from ..config.model_config import read_config_json
from ..config.registry import config_from_dict
from ..models import build_model
from ..weights.loader import load_weights

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def torch_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype '{name}' is not one of {sorted(DTYPES)}") from None


def load_model(model_dir: str, dtype, device):
    """(typed config, model) for the folder; the model class is chosen by ``config.json``."""
    config = config_from_dict(read_config_json(model_dir))
    model = build_model(config, torch_dtype(dtype))
    load_weights(model, model_dir, device)
    return config, model
