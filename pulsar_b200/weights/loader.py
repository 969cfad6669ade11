"""Weights from a model folder, by tensor name.

The reference copies every tensor of every shard under its name and resolves the names
it needs when the model is constructed; a missing name is reported one at a time, extra
tensors are ignored and shapes are not checked (pulsar/src/pulsar/checkpoint.py:122-142;
pulsar-core/src/model/qwen3.cpp:19-22, 48-72).  Here the headers are compared with what
the model's parts declare before any data moves, and one error lists every missing
tensor, every unexpected tensor and every wrong shape or dtype.  An architecture may list
name patterns of tensors that its checkpoints carry and nobody reads (``ModelSpec.ignore``).
"""
from __future__ import annotations

from fnmatch import fnmatchcase
from typing import Dict, List, Sequence

import torch

from ..parts.base import WeightSpec
from .safetensors_io import SafetensorsError, TensorEntry, open_model_files

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


class WeightError(ValueError):
    """The folder's tensors do not fit the model.  ``missing``, ``unexpected`` and ``wrong``
    hold the details that the message lists."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"{where}: the tensors do not fit the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def held_dtype(spec: WeightSpec, compute_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "matrix":
        return compute_dtype
    if spec.role == "vector":
        return torch.float32
    if spec.role == "int":
        return torch.int32
    raise ValueError(f"weight '{spec.name}': unknown role '{spec.role}'")


def check_entries(where: str, specs: List[WeightSpec], entries: Dict[str, TensorEntry], ignore: Sequence[str] = ()) -> None:
    """``ignore``: name patterns (fnmatch) of tensors that the folder may hold although no part reads them
    (buffers that checkpoints of an architecture carry along); a tensor that a part wants is never ignored."""
    by_name = {s.name: s for s in specs}
    missing = [s.name for s in specs if not s.optional and s.name not in entries]
    unexpected = sorted(n for n in entries if n not in by_name and not any(fnmatchcase(n, pat) for pat in ignore))
    wrong = []
    for s in specs:
        e = entries.get(s.name)
        if e is None:
            continue
        if tuple(e.shape) != tuple(s.shape):
            wrong.append(f"{s.name}: expected shape {list(s.shape)}, found {list(e.shape)}")
        elif s.role == "int" and e.dtype not in _INTS:
            wrong.append(f"{s.name}: expected an integer tensor, found {e.dtype}")
        elif s.role != "int" and e.dtype not in _FLOATS:
            wrong.append(f"{s.name}: expected a floating-point tensor, found {e.dtype}")
    if missing or unexpected or wrong:
        raise WeightError(where, missing, unexpected, wrong)


def load_weights(model, model_dir: str, device) -> None:
    """Read the tensors ``model.weight_specs()`` names from ``model_dir`` and hand them to
    ``model.load``.  Matrices are held in the model's compute dtype, vectors in float32,
    integer tables in int32."""
    files = open_model_files(model_dir)
    entries: Dict[str, TensorEntry] = {}
    owner = {}
    for f in files:
        for name, e in f.entries.items():
            if name in entries:
                raise SafetensorsError(f"{model_dir}: tensor '{name}' appears in {entries[name].file} and {e.file}")
            entries[name] = e
            owner[name] = f
    specs = model.weight_specs()
    check_entries(model_dir, specs, entries, getattr(getattr(model, "spec", None), "ignore", ()))
    tensors: Dict[str, torch.Tensor] = {}
    for s in specs:
        if s.name not in entries:
            continue
        host = owner[s.name].tensor(s.name)
        tensors[s.name] = host.to(device=device, dtype=held_dtype(s, model.dtype)).contiguous()
    for f in files:
        f.close()
    model.load(tensors)
