"""What a part is, and the registry parts are chosen from.

A model is put together from parts of five categories:

  mixer     mixes information across the positions of a sequence (attention here)
  ffn       position-wise feed-forward (dense here; a routed one would register the same way)
  norm      normalisation of one activation row
  position  position encoding applied by a mixer to its queries and keys
  block     the arrangement of a layer's sub-layers (a mixer or a feed-forward, each behind its
            norm) around the residual stream

plus the token embedding and the output head.  Every part is built from a `PartSpec` (its sizes
and constants) and a `BuildEnv` (activation dtype, device); it declares the tensors it wants by
local name, receives them from the loader, and knows nothing of the model it sits in.

Registering another part:  `@register_part("mixer", "my_kind") class MyMixer(Mixer): ...` and
name `"my_kind"` in a `PartSpec`.  Interfaces are the abstract classes below.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..config.spec import PartSpec

CATEGORIES = ("mixer", "ffn", "norm", "position", "block", "embedding", "head")
_REGISTRY: Dict[Tuple[str, str], type] = {}


def register_part(category: str, kind: str):
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; categories: {CATEGORIES}")

    def deco(cls):
        _REGISTRY[(category, kind)] = cls
        cls.category, cls.kind = category, kind
        return cls
    return deco


def known_parts(category: str):
    return sorted(k for c, k in _REGISTRY if c == category)


def part_class(category: str, kind: str) -> type:
    cls = _REGISTRY.get((category, kind))
    if cls is None:
        raise KeyError(f"no {category} part of kind {kind!r} is registered; known: {known_parts(category)}")
    return cls


def build_part(category: str, spec: PartSpec, env: "BuildEnv"):
    return part_class(category, spec.kind)(spec, env)


@dataclass(frozen=True)
class BuildEnv:
    """dtype: the activation dtype (torch.float32: everything in true 32-bit; torch.bfloat16:
    bfloat16 activations, weights and cache with float32 residual stream and reductions)."""
    dtype: torch.dtype
    device: torch.device


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part wants from the weights file.  kind: "float" or "int".  init: how the
    random-weights mode fills it ("normal": N(0, 0.02); "one_plus_normal": 1 + N(0, 0.02)).
    use: "matrix" for an operand of a matrix product or a table of rows (kept in the model's
    dtype, whatever the file stores, so that it can feed the tensor cores), "vector" for what
    enters 32-bit arithmetic only (a norm's weight, a bias: under a bfloat16 model such a tensor
    stays float32 if the file stores it in 32 bits)."""
    shape: Tuple[int, ...]
    kind: str = "float"
    init: str = "normal"
    use: str = "matrix"


@dataclass(frozen=True)
class KVNeed:
    """What a mixer keeps per token: `num_kv_heads` rows of `key_dim` elements in the key pool and
    of `value_dim` elements in the value pool (value_dim 0: no value pool, e.g. one latent row
    per token).  `window` None keeps every token, else the last `window`."""
    num_kv_heads: int
    key_dim: int
    value_dim: int
    window: Optional[int] = None


class Part:
    """Base of all parts."""
    category = kind = "?"
    capturable = False      # True: forward() only enqueues device work and may be captured in a CUDA graph

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec, self.env = spec, env

    def prepare(self, max_positions: int) -> None:
        """Called once before the first step with the longest sequence the cache can hold."""

    def tensors(self) -> Dict[str, TensorDecl]:
        """local tensor name -> declaration; the file's name is spec.prefix + "." + local name."""
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the declared tensors, on the device, in the dtype they are to be kept in."""


class Norm(Part):
    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual (float32 [T, H]) += delta (if given), then the normalised rows in the
        activation dtype.  With `rows` only those rows, and the residual is not written."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Encodes positions into the query and key heads.  It never touches the cache: storing keys
    and values is the mixer's business."""

    def apply(self, qkv: torch.Tensor, num_heads: int, num_kv_heads: int, ctx) -> None:
        """Encodes the positions ctx.tok_pos into the query and key heads of the packed
        projections [T, (num_heads + 2 num_kv_heads) head_dim], in place."""
        raise NotImplementedError

    def rotation_tables(self, positions: int) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        """An encoding that is a rotation of the pairs (j, j + head_dim / 2) by angles that depend
        on position and j alone may hand out its float32 tables (cos, sin), each
        [rows >= positions, head_dim / 2]: a mixer's kernels can then rotate on the fly (and store
        the rotated key in the same pass) instead of calling apply().  None: apply() is the only way."""
        return None


class Mixer(Part):
    def kv_need(self) -> Optional[KVNeed]:
        """Growing per-token storage this mixer needs, or None."""
        return None

    def state_size(self) -> int:
        """float32 elements of fixed-size state per sequence (zeroed when a sequence starts)."""
        return 0

    def forward(self, x: torch.Tensor, ctx, call: int) -> torch.Tensor:
        """x: normalised activations [T, H] of the step's packed tokens.  Returns what is to be
        added to the residual stream: [T, H] or [parts, T, H].  `call` is this mixer's index
        among the mixers of the run order: `ctx.kv(call)` is its cache view, `ctx.state(call)`
        its state rows [n_slots, state_size]."""
        raise NotImplementedError

    def forward_into(self, x: torch.Tensor, ctx, call: int, residual: torch.Tensor) -> bool:
        """A mixer whose last kernel can add its result to the float32 residual stream [T, H] itself does
        so and returns True; the block then has no delta to hand on.  False (the default): nothing was
        done, call forward()."""
        return False


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x: normalised activations [T, H].  Returns what is to be added to the residual stream."""
        raise NotImplementedError

    def forward_into(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> bool:
        """A feed-forward that can add its result to the float32 residual stream [T, H] itself (in its
        last kernel, which saves a pass over the activations) does so and returns True; the block
        then has no delta to hand on.  False (the default): nothing was done, call forward()."""
        return False


@dataclass
class SubLayer:
    """A built sub-layer: the part, its category ("mixer" or "ffn") and the norm before it (or None)."""
    category: str
    part: Part
    norm: Optional[Norm]


class Block(Part):
    """Arrangement of one layer.  Built with the layer's sub-layers instead of a PartSpec."""

    def __init__(self, sublayers, env: BuildEnv):
        self.sublayers, self.env = list(sublayers), env
        self.spec = None

    def forward(self, residual: torch.Tensor, pending: Optional[torch.Tensor], ctx, users):
        """residual: float32 [T, H]; pending: a delta not yet added to it (or None); users: for
        each mixer of the layer, in sub-layer order, its index for ctx.kv() / ctx.state().
        Returns (residual, pending) for the next block."""
        raise NotImplementedError
