"""Binding weights to a model by tensor name.

xsmccc/llaisys maps every tensor of every *.safetensors file of the folder to a slot of its
weights struct by exact name, converts 16-bit tensors to float32 and silently skips what it
does not know (python/llaisys/models/qwen2.py:99-210).  Here the model's parts declare the
tensors they want; the file must hold exactly those, with those shapes, or loading stops with
one error that lists everything that is missing, unexpected or mis-shaped.

Kept dtypes.  xsmccc/llaisys converts every tensor to the one dtype of its model
(python/llaisys/models/qwen2.py:118-119, 141).  Here: under a float32 model every floating
tensor becomes float32.  Under a bfloat16 model the operands of matrix products and the
embedding table (declared use="matrix") become bfloat16 whatever the file stores, so that a
checkpoint stored in 32 bits runs on the tensor cores like any other; tensors that only enter
32-bit arithmetic (use="vector": norm weights, biases) are kept as bfloat16 when stored in 16
bits and stay float32 when stored in 32 (or 64) bits.  Integer tensors are kept as int32.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Tuple

import torch

from .safetensors_io import DTYPES, SafetensorsFile


class WeightsError(ValueError):
    """The tensors on offer do not fit the model.  `missing`, `unexpected`, `wrong_shape`
    (name -> (got, want)) and `wrong_kind` hold the details that the message lists."""

    def __init__(self, where, missing, unexpected, wrong_shape, wrong_kind):
        self.missing, self.unexpected = sorted(missing), sorted(unexpected)
        self.wrong_shape, self.wrong_kind = dict(wrong_shape), dict(wrong_kind)
        lines = [f"weights of {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for n, (got, want) in sorted(self.wrong_shape.items()):
            lines.append(f"  wrong shape: {n} is {list(got)}, the model wants {list(want)}")
        for n, (got, want) in sorted(self.wrong_kind.items()):
            lines.append(f"  wrong type: {n} is stored as {got}, the model wants a {want} tensor")
        super().__init__("\n".join(lines))


_FLOAT = {"F64", "F32", "F16", "BF16"}
_INT = {"I64", "I32", "I16", "I8", "U8"}


class FolderSource:
    """All *.safetensors files of a model folder, in sorted order."""

    def __init__(self, folder):
        self.folder = Path(folder)
        self.files = [SafetensorsFile(p) for p in sorted(self.folder.glob("*.safetensors"))]
        if not self.files:
            raise FileNotFoundError(f"no *.safetensors file in {self.folder}")
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.entries:
                if name in self._where:
                    raise ValueError(f"tensor {name!r} appears in both {self._where[name].path.name} and {f.path.name}")
                self._where[name] = f

    def describe(self) -> str:
        return str(self.folder)

    def entries(self) -> Dict[str, Tuple[str, Tuple[int, ...]]]:
        return {n: f.entries[n] for n, f in self._where.items()}

    def get(self, name: str) -> torch.Tensor:
        return self._where[name].get(name)


class RandomSource:
    """Seeded random tensors for a model's declarations: matrices, embeddings and biases
    N(0, 0.02), norm weights 1 + N(0, 0.02), drawn in float32 and rounded to `dtype`.  The
    generator is counter-based (weights/rng.py): element i of a tensor is a function of (seed,
    tensor name, i) alone, so a tensor does not depend on which other tensors exist, and a
    source on the CPU and a source on a CUDA device (filled there by a kernel, which is what a
    65 GB model needs) hold the same values."""

    def __init__(self, decls, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu", std: float = 0.02):
        self.decls, self.seed, self.dtype, self.device, self.std = dict(decls), int(seed), dtype, torch.device(device), std

    def describe(self) -> str:
        return f"random weights (seed {self.seed})"

    def entries(self):
        from .safetensors_io import NAMES
        return {n: (NAMES[self.dtype] if d.kind == "float" else "I32", tuple(d.shape)) for n, d in self.decls.items()}

    def get(self, name: str) -> torch.Tensor:
        from .rng import normal, tensor_key
        d = self.decls[name]
        if d.kind == "int":
            return torch.zeros(d.shape, dtype=torch.int32, device=self.device)
        key = tensor_key(self.seed, name)
        mean = 1.0 if d.init == "one_plus_normal" else 0.0
        n = 1
        for s in d.shape:
            n *= s
        if self.device.type == "cuda":
            from .. import kernels
            out = torch.empty(d.shape, dtype=self.dtype, device=self.device)
            kernels.fill_normal(out, key, mean, self.std)
            return out
        x = torch.from_numpy(normal(key, n, 0, mean, self.std)).view(d.shape)
        return x.to(self.dtype)


def kept_dtype(stored: str, compute: torch.dtype, use: str = "matrix") -> torch.dtype:
    if stored in _INT:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if use == "matrix":
        return compute
    return torch.bfloat16 if stored in ("F16", "BF16") else torch.float32


def check_tensors(model, source) -> None:
    expected = model.expected_tensors()
    have = source.entries()
    ignorable = set(model.ignorable_tensors())
    missing = [n for n in expected if n not in have]
    unexpected = [n for n in have if n not in expected and n not in ignorable]
    wrong_shape, wrong_kind = {}, {}
    for n, decl in expected.items():
        if n not in have:
            continue
        stored, shape = have[n]
        if tuple(shape) != tuple(decl.shape):
            wrong_shape[n] = (tuple(shape), tuple(decl.shape))
        if (decl.kind == "float" and stored not in _FLOAT) or (decl.kind == "int" and stored not in _INT):
            wrong_kind[n] = (stored, "floating-point" if decl.kind == "float" else "integer")
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightsError(source.describe(), missing, unexpected, wrong_shape, wrong_kind)


def load_weights(model, source) -> None:
    """Checks `source` against the model's declarations, then moves every tensor to the
    model's device in the dtype it is kept in and hands them to the parts."""
    check_tensors(model, source)
    have = source.entries()
    env = model.env
    tensors = {}
    for name, decl in model.expected_tensors().items():
        t = source.get(name)
        tensors[name] = t.to(device=env.device, dtype=kept_dtype(have[name][0], env.dtype, decl.use))
    model.bind(tensors)
