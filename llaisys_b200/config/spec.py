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
class SubLayerSpec:
    """One step of a layer: a part of category `category` ("mixer" or "ffn") behind an optional norm."""
    category: str
    part: PartSpec
    norm: Optional[PartSpec] = None


@dataclass(frozen=True)
class LayerSpec:
    """A layer is an arrangement (`block`) of sub-layers around the residual stream: as many as
    the architecture has (mixer then feed-forward here; a mixer alone, or a mixer and two
    feed-forwards, are other layers of the same kind)."""
    block: str
    sublayers: Tuple[SubLayerSpec, ...]

    @classmethod
    def pair(cls, block: str, mixer: PartSpec, mixer_norm: PartSpec, ffn: PartSpec, ffn_norm: PartSpec) -> "LayerSpec":
        """The usual layer: norm, mixer, norm, feed-forward."""
        return cls(block, (SubLayerSpec("mixer", mixer, mixer_norm), SubLayerSpec("ffn", ffn, ffn_norm)))

    def mixers(self) -> Tuple[PartSpec, ...]:
        return tuple(s.part for s in self.sublayers if s.category == "mixer")


@dataclass(frozen=True)
class CallSpec:
    """One entry of the run order.  `layer` indexes `ModelSpec.layers` and may repeat.
    `cache_of` names an earlier entry of the order whose cache this call's mixers read instead of
    keeping one of their own (they then append nothing); the mixers of the two entries pair up in
    sub-layer order."""
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
