"""A decoder on the CPU, put together from the plain float32 operators of `cpu_ops`: one sequence,
a contiguous cache per attention call, the prompt in one step and then one token per step,
greedy choice of the next token.

This is what xsmccc/llaisys' own model is (src/models/qwen2/qwen2.cpp:53-87: operators on the
CPU, float32, one sequence), and it serves here as the second implementation that the command
line's --test compares the engine's tokens with (test/test_infer.py:193-195 compares with a
second implementation too), and as the model behind --device cpu.  It reads the same `ModelSpec`
and the same tensors by name as the engine does, shares no code with the engine's parts or
kernels, and knows the built-in part kinds only.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np

from .. import cpu_ops
from ..config.spec import ModelSpec, PartSpec

_KNOWN = {"embedding": {"token_embedding"}, "norm": {"rms_norm"}, "mixer": {"gqa_attention"}, "ffn": {"swiglu_mlp"},
          "block": {"pre_norm_residual"}, "head": {"lm_head"}, "position": {"rope_half_split"}}


class CpuModel:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, np.ndarray]):
        """tensors: name -> float32 array, the names being those of the weights file."""
        self.spec, self.w = spec, tensors
        for kind, cat in [(spec.embedding.kind, "embedding"), (spec.final_norm.kind, "norm"), (spec.head.kind, "head")]:
            self._known(cat, kind)
        for layer in spec.layers:
            self._known("block", layer.block)
            for sub in layer.sublayers:
                self._known(sub.category, sub.part.kind)
                if sub.norm is not None:
                    self._known("norm", sub.norm.kind)
                pos = sub.part.params.get("position")
                if pos is not None:
                    self._known("position", pos.kind)
        self.reset()

    @staticmethod
    def _known(category: str, kind: str):
        if kind not in _KNOWN[category]:
            raise NotImplementedError(f"the CPU model knows the built-in parts only, not the {category} {kind!r}")

    @classmethod
    def from_folder(cls, folder) -> "CpuModel":
        from ..config.registry import load_config
        from ..weights.loader import FolderSource
        src = FolderSource(folder)
        return cls(load_config(folder).to_spec(), {n: src.get(n).float().numpy() for n in src.entries()})

    def reset(self) -> None:
        self.length = 0
        self.cache: List[dict] = [{} for _ in self.spec.order]       # per entry of the run order: mixer index -> (k, v)

    # ---- parts
    def _norm(self, p: PartSpec, x):
        return cpu_ops.rms_norm(x, self.w[p.tensor_name("weight")], p.params["eps"])

    def _attention(self, p: PartSpec, x, positions, store: dict, key, owner):
        a = p.params
        nh, nkvh, dh = a["num_heads"], a["num_kv_heads"], a["head_dim"]
        T = x.shape[0]
        bias = (lambda n: self.w[p.tensor_name(n)]) if a.get("qkv_bias") else (lambda n: None)
        q = cpu_ops.linear(x, self.w[p.tensor_name("q_proj.weight")], bias("q_proj.bias")).reshape(T, nh, dh)
        k = cpu_ops.linear(x, self.w[p.tensor_name("k_proj.weight")], bias("k_proj.bias")).reshape(T, nkvh, dh)
        v = cpu_ops.linear(x, self.w[p.tensor_name("v_proj.weight")], bias("v_proj.bias")).reshape(T, nkvh, dh)
        if a.get("position") is not None:
            theta = a["position"].params["theta"]
            q, k = cpu_ops.rope(q, positions, theta), cpu_ops.rope(k, positions, theta)
        if owner is None:
            old = store.get(key)
            store[key] = (k, v) if old is None else (np.concatenate([old[0], k]), np.concatenate([old[1], v]))
            ks, vs = store[key]
        else:
            ks, vs = owner[key]                       # an earlier entry's keys and values; nothing is appended
        o = cpu_ops.self_attention(q, ks, vs, a["scale"], a.get("window"))
        out_bias = self.w[p.tensor_name("o_proj.bias")] if a.get("out_bias") else None
        return cpu_ops.linear(o.reshape(T, nh * dh), self.w[p.tensor_name("o_proj.weight")], out_bias)

    def _mlp(self, p: PartSpec, x):
        g = cpu_ops.linear(x, self.w[p.tensor_name("gate_proj.weight")])
        u = cpu_ops.linear(x, self.w[p.tensor_name("up_proj.weight")])
        return cpu_ops.linear(cpu_ops.swiglu(g, u), self.w[p.tensor_name("down_proj.weight")])

    # ---- the model
    def step(self, tokens: Sequence[int]) -> np.ndarray:
        """Feeds the next tokens of the sequence; returns float32 logits [len(tokens), vocab]."""
        positions = np.arange(self.length, self.length + len(tokens))
        x = cpu_ops.embedding(np.asarray(tokens), self.w[self.spec.embedding.tensor_name("weight")]).astype(np.float32)
        for c, call in enumerate(self.spec.order):
            owner = self.cache[call.cache_of] if call.cache_of is not None else None
            m = 0
            for sub in self.spec.layers[call.layer].sublayers:
                h = self._norm(sub.norm, x) if sub.norm is not None else x
                if sub.category == "mixer":
                    x = cpu_ops.add(self._attention(sub.part, h, positions, self.cache[c], m, owner), x)
                    m += 1
                else:
                    x = cpu_ops.add(self._mlp(sub.part, h), x)
        self.length += len(tokens)
        x = self._norm(self.spec.final_norm, x)
        head = self.spec.head
        name = head.params.get("tied_to") or head.tensor_name("weight")
        return cpu_ops.linear(x, self.w[name])

    def generate(self, prompt: Sequence[int], max_new_tokens: int, stop_ids: Sequence[int] = ()) -> List[int]:
        """Greedy continuation: the new tokens (a stop token included)."""
        self.reset()
        logits = self.step(list(prompt))[-1]
        new: List[int] = []
        for _ in range(max_new_tokens):
            tok, _ = cpu_ops.argmax(logits)
            new.append(tok)
            if tok in stop_ids or len(new) == max_new_tokens:
                break
            logits = self.step([tok])[-1]
        return new
