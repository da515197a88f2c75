"""Reading and writing the safetensors format: an 8-byte little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the raw little-endian tensor bytes.

xsmccc/llaisys reads these files through the `safetensors` package
(python/llaisys/models/qwen2.py:99-112); this reader maps the file and hands out torch tensors
that view the mapping, so a tensor is copied once, straight to where it is kept.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Tuple

import torch

DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped file.  `entries[name] = (dtype string, shape)`; `get(name)` is a CPU tensor
    that views the mapping (valid while this object lives)."""

    def __init__(self, path):
        self.path = Path(path)
        self._fh = open(self.path, "rb")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{self.path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not JSON ({e})") from None
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, Tuple[str, Tuple[int, ...]]] = {}
        self._offsets = {}
        for name, info in header.items():
            dt, shape, (lo, hi) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
            if dt not in DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {dt}")
            n = 1
            for s in shape:
                n *= s
            if hi - lo != n * DTYPES[dt].itemsize or self._base + hi > size:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has inconsistent offsets")
            self.entries[name] = (dt, shape)
            self._offsets[name] = (lo, hi)

    def get(self, name: str) -> torch.Tensor:
        dt, shape = self.entries[name]
        lo, hi = self._offsets[name]
        if hi == lo:
            return torch.empty(shape, dtype=DTYPES[dt])
        flat = torch.frombuffer(self._mm, dtype=DTYPES[dt], count=(hi - lo) // DTYPES[dt].itemsize,
                                offset=self._base + lo)
        return flat.view(shape)

    def close(self):
        # tensors handed out may still view the mapping; it is released with the last of them
        self._fh.close()


class Deferred:
    """A tensor that is made only when its bytes are written: dtype and shape are known
    beforehand (the header needs them), `make()` returns the tensor."""

    def __init__(self, dtype: torch.dtype, shape, make):
        self.dtype, self.shape, self.make = dtype, tuple(shape), make

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


def write_safetensors(path, tensors, metadata: dict | None = None):
    """Writes (name, tensor) pairs (a dict, or a sequence of pairs) in the given order.  A value may
    be a `Deferred`: it is made when its turn comes and dropped once written, so a file larger than
    the host's memory can be written one tensor at a time (the header, which comes first in the
    file, is laid out from the declared dtypes and shapes)."""
    path = Path(path)
    items = list(tensors.items()) if isinstance(tensors, dict) else list(tensors)
    header, off = {}, 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in items:
        if t.dtype not in NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for i in range(len(items)):
            name, t = items[i]
            items[i] = None                       # nothing keeps the tensor once it is written
            if isinstance(t, Deferred):
                made = t.make()
                if made.dtype != t.dtype or tuple(made.shape) != t.shape:
                    raise SafetensorsError(f"tensor {name!r} was declared {t.dtype} {list(t.shape)} but made "
                                           f"{made.dtype} {list(made.shape)}")
                t = made
                del made
            c = t.detach().to("cpu").contiguous()
            if c.numel():
                f.write(c.view(torch.uint8).numpy().data)
            del c, t
