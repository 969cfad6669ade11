"""Random weights from a configuration and a seed.

The reference has random weights only inside tests (``randn * 0.05`` / ``randn * 0.02``,
norm weights 1: pulsar-core/tests/runtime/test_engine.cpp:46-75,
pulsar/tests/test_session.py:47-72).  Here it is a mode of its own: one seeded CPU
generator is consumed in the order of ``model.weight_specs()`` (embedding, layers in
order, final norm, head), matrices N(0, std), norm weights 1 + N(0, 0.1), and the
result is written as a model folder that every other entry point loads like a real one.
"""
from __future__ import annotations

import json
import os
from typing import Iterator, Optional, Tuple

import torch

from ..parts.base import WeightSpec
from .safetensors_io import write_safetensors


def _draw(spec: WeightSpec, std: float, gen: torch.Generator, device) -> torch.Tensor:
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    noise = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
    if spec.init == "ones_normal":
        return 1.0 + 0.1 * noise
    if spec.init == "normal":
        return std * noise
    raise ValueError(f"weight '{spec.name}': unknown init '{spec.init}'")


def random_tensors(model, seed: int, std: float, device="cpu", untied_head: Optional[bool] = None
                   ) -> Iterator[Tuple[str, torch.Tensor]]:
    """(name, float32 tensor) in the order of ``model.weight_specs()``.  An optional head
    is drawn unless ``untied_head`` is False."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    for spec in model.weight_specs():
        if spec.optional and untied_head is False:
            continue
        if spec.role == "int":
            raise ValueError(f"weight '{spec.name}': integer tables have no random init")
        yield spec.name, _draw(spec, std, gen, device)


def write_model_folder(config, out_dir: str, seed: int, std: Optional[float] = None,
                       store_dtype: torch.dtype = torch.float32, untied_head: Optional[bool] = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (anything with
    ``model_spec()`` and ``to_dict()``).  Returns ``out_dir``."""
    from ..models import build_model
    model = build_model(config, torch.float32)
    if std is None:
        std = model.spec.init_std
    if untied_head is None and model.spec.tie_word_embeddings is None:
        untied_head = True
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1, sort_keys=True)
    tensors = ((n, t.to(store_dtype)) for n, t in random_tensors(model, seed, std, "cpu", untied_head))
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed), "std": repr(std)})
    return out_dir


def load_random(model, seed: int, std: Optional[float], device, untied_head: Optional[bool] = None) -> None:
    """Fill ``model`` with random weights drawn on ``device`` (for measurements of large
    shapes: nothing touches the disk; values differ from the CPU generator's)."""
    from .loader import held_dtype
    if std is None:
        std = model.spec.init_std
    if untied_head is None and model.spec.tie_word_embeddings is None:
        untied_head = True
    specs = {s.name: s for s in model.weight_specs()}
    tensors = {}
    for name, t in random_tensors(model, seed, std, device, untied_head):
        tensors[name] = t.to(held_dtype(specs[name], model.dtype))
    model.load(tensors)
