"""A decoder put together from a ModelSpec: embedding, the calls of the run order, final norm, head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec
from ..parts.base import BuildEnv, KVNeed, Part, TensorDecl, build_part, part_class


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec, self.env = spec, env
        self.embedding = build_part("embedding", spec.embedding, env)
        self.blocks = []
        for ls in spec.layers:
            mixer = build_part("mixer", ls.mixer, env)
            ffn = build_part("ffn", ls.ffn, env)
            n1, n2 = build_part("norm", ls.mixer_norm, env), build_part("norm", ls.ffn_norm, env)
            self.blocks.append(part_class("block", ls.block)(mixer, n1, ffn, n2, env))
        for c, call in enumerate(spec.order):
            if not (0 <= call.layer < len(self.blocks)):
                raise ValueError(f"run order entry {c} names layer {call.layer}, which does not exist")
        self.final_norm = build_part("norm", spec.final_norm, env)
        self.head = build_part("head", spec.head, env)
        self._loaded = False

    # ---- what the cache has to provide, per call of the run order
    def kv_needs(self) -> List[Optional[KVNeed]]:
        return [self.blocks[c.layer].mixer.kv_need() for c in self.spec.order]

    def cache_of(self) -> List[Optional[int]]:
        return [c.cache_of for c in self.spec.order]

    def state_sizes(self) -> List[int]:
        return [self.blocks[c.layer].mixer.state_size() for c in self.spec.order]

    def capturable(self) -> bool:
        """True when every part's forward only enqueues device work (no host read-back), so that
        a decode step can be captured in a CUDA graph."""
        return all(getattr(p, "capturable", False) for p in self.parts())

    def prepare(self, max_positions: int) -> None:
        """Lets parts size what depends on the longest sequence the cache can hold."""
        for p in self.parts():
            p.prepare(max_positions)

    # ---- weights
    def parts(self) -> List[Part]:
        ps: List[Part] = [self.embedding]
        for b in self.blocks:
            ps += [b.mixer_norm, b.mixer, b.ffn_norm, b.ffn]
        return ps + [self.final_norm, self.head]

    def expected_tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for p in self.parts():
            for local, decl in p.tensors().items():
                name = p.spec.tensor_name(local)
                if name in out:
                    raise ValueError(f"two parts declare the tensor {name!r}")
                out[name] = decl
        return out

    def ignorable_tensors(self) -> List[str]:
        """Names a file may hold without their being used: the head's own matrix when it is tied."""
        tied = getattr(self.head, "tied_to", None)
        return [self.head.spec.tensor_name("weight")] if tied else []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load({local: tensors[p.spec.tensor_name(local)] for local in p.tensors()})
        tied = getattr(self.head, "tied_to", None)
        if tied:
            self.head.tie(tensors[tied])
        self._loaded = True

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for p in self.parts():
            for v in vars(p).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen and v.dim() >= 1:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total

    # ---- the forward pass of one step
    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Runs the step's tokens through every call of the run order and returns float32
        logits [len(out_rows), vocab] (None when no logits are wanted)."""
        if not self._loaded:
            raise RuntimeError("the model has no weights yet")
        residual = self.embedding.forward(ctx)
        pending = None
        for c, call in enumerate(self.spec.order):
            residual, pending = self.blocks[call.layer].forward(residual, pending, ctx, c)
        if ctx.out_rows.numel() == 0:
            return None
        h = self.final_norm.forward(residual, pending, rows=ctx.out_rows)
        return self.head.forward(h)
