"""Architecture-independent description of a decoder: which parts, with which sizes, in which order.

A configuration class of an architecture (see `qwen2.py`) turns its config.json keys into a
`ModelSpec`.  Everything below the configuration layer (parts, cache, engine, weights) reads
only the spec, so no part knows which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: the registry key of its implementation, its sizes and constants, and the
    prefix of its tensors' names in the weights file."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""

    def tensor_name(self, local: str) -> str:
        return f"{self.prefix}.{local}" if self.prefix else local


@dataclass(frozen=True)
class LayerSpec:
    """A layer is an arrangement (`block`) of a mixer and a feed-forward, each behind a norm."""
    block: str
    mixer: PartSpec
    mixer_norm: PartSpec
    ffn: PartSpec
    ffn_norm: PartSpec


@dataclass(frozen=True)
class CallSpec:
    """One entry of the run order.  `layer` indexes `ModelSpec.layers` and may repeat.
    `cache_of` names an earlier entry of the order whose cache this call reads instead of
    keeping one of its own (it then appends nothing)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[CallSpec, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()


class ConfigError(ValueError):
    """A config.json that cannot be used: a missing or inconsistent key, an unknown architecture."""
