from .base import (Block, BuildEnv, FeedForward, KVNeed, Mixer, Norm, Part, PositionEncoding,
                   SubLayer, TensorDecl, build_part, known_parts, part_class, register_part)
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registers the built-in parts)

__all__ = ["Block", "BuildEnv", "FeedForward", "KVNeed", "Mixer", "Norm", "Part", "PositionEncoding",
           "SubLayer", "TensorDecl", "build_part", "known_parts", "part_class", "register_part"]
