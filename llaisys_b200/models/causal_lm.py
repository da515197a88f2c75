"""The Python entry point: a model folder in, generated tokens out."""
from __future__ import annotations

from enum import IntEnum
from pathlib import Path
from typing import List, Optional, Sequence

import torch

from ..cache.kv import CacheConfig
from ..config.registry import load_config
from ..engine.engine import Engine, StepEntry, build_engine
from ..engine.generate import GenerationLoop
from ..sampling.sampler import Sampler, SamplingParams
from ..weights.loader import FolderSource


class DeviceType(IntEnum):
    """Device names of xsmccc/llaisys (include/llaisys.h:23-30).  Only NVIDIA is served here."""
    CPU = 0
    NVIDIA = 1


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class CausalLM:
    """A decoder of whatever architecture the folder's config.json names.

    model_path: folder with config.json and *.safetensors.  dtype: "bfloat16" (the serving
    path) or "float32" (everything in true 32-bit).  max_tokens sizes the cache: the most
    tokens all live sequences hold together, each rounded up to a whole page of 64."""

    architecture: Optional[str] = None      # subclasses pin the architecture they stand for

    def __init__(self, model_path, device: DeviceType = DeviceType.NVIDIA, device_id: int = 0,
                 dtype="bfloat16", max_tokens: int = 8192, max_seqs: Optional[int] = None, seed: int = 0):
        self.model_path = Path(model_path)
        if DeviceType(device) != DeviceType.NVIDIA:
            raise RuntimeError("llaisys_b200 serves DeviceType.NVIDIA only; it has no CPU path")
        self.config = load_config(self.model_path)
        if self.architecture and self.config.architecture != self.architecture:
            raise ValueError(f"{self.model_path} holds a {self.config.architecture} model, not {self.architecture}")
        self.spec = self.config.to_spec()
        self.dtype = _DTYPES[dtype]
        self.seed = seed
        self.engine: Engine = build_engine(self.spec, self.dtype, f"cuda:{device_id}",
                                           CacheConfig(max_tokens=max_tokens, max_seqs=max_seqs),
                                           FolderSource(self.model_path))

    @property
    def stop_token_ids(self):
        return self.spec.stop_token_ids

    def generate_batch(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 128, top_k: int = 1,
                       top_p: float = 0.8, temperature: float = 0.8, stop_ids: Optional[Sequence[int]] = None,
                       seed: Optional[int] = None, max_batch: Optional[int] = None) -> List[List[int]]:
        """The new tokens of every prompt (a stop token included).  Prompts of unequal lengths
        start together in batches as large as the cache allows."""
        sampler = Sampler(SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p),
                          self.seed if seed is None else seed)
        loop = GenerationLoop(self.engine, sampler, self.stop_token_ids if stop_ids is None else stop_ids, max_batch)
        self.last_loop = loop
        out = [g.tokens for g in loop.run(prompts, max_new_tokens)]
        self.engine.check()
        return out

    def generate(self, inputs: Sequence[int], max_new_tokens: int = 128, top_k: int = 1, top_p: float = 0.8,
                 temperature: float = 0.8) -> List[int]:
        """Signature and defaults of xsmccc/llaisys' Qwen2.generate
        (python/llaisys/models/qwen2.py:212-219): returns the prompt followed by the new tokens;
        top_k == 1 is greedy."""
        new = self.generate_batch([list(inputs)], max_new_tokens, top_k, top_p, temperature)[0]
        return list(inputs) + new

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """float32 logits [len(tokens), vocab] of one whole sequence, on the device."""
        slot = self.engine.acquire()
        try:
            out = self.engine.step([StepEntry(slot, list(tokens), list(range(len(tokens))))])
            self.engine.check()
            return out
        finally:
            self.engine.release(slot)


class Qwen2(CausalLM):
    """`llaisys.models.Qwen2(model_path, device)` of xsmccc/llaisys
    (python/llaisys/models/qwen2.py:31-33), for the Qwen2 dense decoder."""
    architecture = "Qwen2ForCausalLM"
