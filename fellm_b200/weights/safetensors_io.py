"""The safetensors container, read and written directly: an 8-byte little-endian header length,
a JSON header {name: {dtype, shape, data_offsets}}, then the raw little-endian data.

The checks are those FeLLM's one safetensors reader makes
(plugins/dspark/src/checkpoint.rs:59-118): header length inside the file, `__metadata__`
skipped, known dtype, data_offsets length = element size x element count, extent inside the file.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict

import numpy as np
import torch

from ..config.errors import WeightError

_DTYPES = {"F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
           "I32": (torch.int32, 4), "I64": (torch.int64, 8), "U8": (torch.uint8, 1)}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """Header parsed at open; tensors are read from a memory map on demand."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._f = open(self.path, "rb")
        except FileNotFoundError:
            raise WeightError(f"no weight file {self.path}") from None
        size = self.path.stat().st_size
        if size < 8:
            raise WeightError(f"{self.path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise WeightError(f"{self.path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._f.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise WeightError(f"{self.path}: header is not valid JSON: {e}") from None
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: Dict[str, tuple] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dt = meta.get("dtype")
            if dt not in _DTYPES:
                raise WeightError(f"{self.path}: tensor {name} has unsupported dtype {dt}")
            shape = tuple(int(s) for s in meta["shape"])
            lo, hi = (int(v) for v in meta["data_offsets"])
            n = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if hi - lo != n * _DTYPES[dt][1]:
                raise WeightError(f"{self.path}: tensor {name} has {hi - lo} bytes for shape {list(shape)} {dt}")
            if lo < 0 or hi > data_len:
                raise WeightError(f"{self.path}: tensor {name} lies outside the file")
            self.entries[name] = (_DTYPES[dt][0], shape, lo, hi)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return self.entries[name][1]

    def dtype(self, name):
        return self.entries[name][0]

    def tensor(self, name) -> torch.Tensor:
        """A CPU tensor that owns its memory."""
        dt, shape, lo, hi = self.entries[name]
        buf = bytearray(self._mm[self._data_start + lo:self._data_start + hi])
        if not buf:
            return torch.empty(shape, dtype=dt)
        return torch.frombuffer(buf, dtype=dt).reshape(shape)

    def close(self):
        if self._mm is not None:
            self._mm.close()
        self._f.close()


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata=None):
    header, offset, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightError(f"cannot write tensor {name} of dtype {t.dtype}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
