"""A decoder put together from a ModelSpec: embedding, the calls of the run order, final norm, head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec
from ..parts.base import BuildEnv, KVNeed, Part, SubLayer, TensorDecl, build_part, part_class


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec, self.env = spec, env
        self.embedding = build_part("embedding", spec.embedding, env)
        self.blocks = []
        for ls in spec.layers:
            subs = []
            for sub in ls.sublayers:
                if sub.category not in ("mixer", "ffn"):
                    raise ValueError(f"a sub-layer is a 'mixer' or an 'ffn', not {sub.category!r}")
                norm = build_part("norm", sub.norm, env) if sub.norm is not None else None
                subs.append(SubLayer(sub.category, build_part(sub.category, sub.part, env), norm))
            self.blocks.append(part_class("block", ls.block)(subs, env))
        # Every mixer of every entry of the run order is a user of the cache with an index of its own.
        self.users: List[tuple] = []                 # user -> (order entry, layer, sub-layer index)
        self.call_users: List[tuple] = []            # order entry -> its users, in sub-layer order
        for c, call in enumerate(spec.order):
            if not (0 <= call.layer < len(self.blocks)):
                raise ValueError(f"run order entry {c} names layer {call.layer}, which does not exist")
            mine = []
            for i, sub in enumerate(self.blocks[call.layer].sublayers):
                if sub.category == "mixer":
                    mine.append(len(self.users))
                    self.users.append((c, call.layer, i))
            self.call_users.append(tuple(mine))
        self.final_norm = build_part("norm", spec.final_norm, env)
        self.head = build_part("head", spec.head, env)
        self._loaded = False

    def _mixer(self, user: int):
        _, layer, i = self.users[user]
        return self.blocks[layer].sublayers[i].part

    # ---- what the cache has to provide, per user (a mixer of an entry of the run order)
    def kv_needs(self) -> List[Optional[KVNeed]]:
        return [self._mixer(u).kv_need() for u in range(len(self.users))]

    def cache_of(self) -> List[Optional[int]]:
        out: List[Optional[int]] = []
        for u, (c, _, _) in enumerate(self.users):
            owner = self.spec.order[c].cache_of
            if owner is None:
                out.append(None)
                continue
            if not (0 <= owner < c):
                raise ValueError(f"run order entry {c} reads the cache of entry {owner}, which does not come before it")
            k = self.call_users[c].index(u)
            theirs = self.call_users[owner]
            if k >= len(theirs):
                raise ValueError(f"run order entry {c} reads the cache of entry {owner}, which has fewer mixers")
            out.append(theirs[k])
        return out

    def state_sizes(self) -> List[int]:
        return [self._mixer(u).state_size() for u in range(len(self.users))]

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
            for sub in b.sublayers:
                ps += ([sub.norm] if sub.norm is not None else []) + [sub.part]
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
            residual, pending = self.blocks[call.layer].forward(residual, pending, ctx, self.call_users[c])
        if ctx.out_rows.numel() == 0:
            return None
        h = self.final_norm.forward(residual, pending, rows=ctx.out_rows)
        return self.head.forward(h)
