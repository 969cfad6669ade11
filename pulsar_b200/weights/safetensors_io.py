"""A small reader and writer for the safetensors container.

Layout: 8 bytes little-endian header length n, n bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the raw little-endian tensor bytes.  The reference goes through the
``safetensors`` package (pulsar/src/pulsar/checkpoint.py:136-140); the engine reads
the file itself so that shapes can be checked from the header before a byte of data
moves, and so that tensors are copied one by one from a memory map.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int
    file: str


class SafetensorsFile:
    """One open file: header parsed, data memory-mapped on demand."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise SafetensorsError(f"{path}: too short for a safetensors header")
            (n,) = struct.unpack("<Q", head)
            if n > size - 8:
                raise SafetensorsError(f"{path}: header length {n} exceeds the file size {size}")
            try:
                header = json.loads(f.read(n).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.data_start = 8 + n
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {info['dtype']}")
            dtype = _DTYPES[info["dtype"]]
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(v) for v in info["data_offsets"])
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * dtype.itemsize or self.data_start + end > size:
                raise SafetensorsError(f"{path}: tensor '{name}' has data_offsets {begin}:{end} that do not match "
                                       f"shape {list(shape)} of {info['dtype']}")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, path)
        self._file = None
        self._map = None

    def _mapped(self):
        if self._map is None:
            self._file = open(self.path, "rb")
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        return self._map

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that aliases the mapped file (read-only: copy before writing)."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._mapped())[self.data_start + e.begin: self.data_start + e.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # the buffer is read-only; callers only read
            flat = torch.frombuffer(buf, dtype=e.dtype)
        return flat.view(e.shape)

    def close(self) -> None:
        self._map = None      # tensors handed out keep the map alive through their buffer
        if self._file is not None:
            self._file.close()
            self._file = None


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """``model.safetensors``, or the shards ``model.safetensors.index.json`` names
    (the two layouts scripts/migrate.py:37-47 reads)."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str] | None = None):
    """Write ``(name, tensor)`` pairs in the given order.  The header is built first
    from shapes, then the tensors stream out one at a time."""
    items = [(n, t) for n, t in tensors]
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = f"{path}.tmp{os.getpid()}"       # tensors being written may alias a map of the old file
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            c = t.detach().contiguous().cpu()
            f.write(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"")
    os.replace(tmp, path)
