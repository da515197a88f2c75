"""Choice of the next token from logits.

xsmccc/llaisys' generate() takes top_k, top_p and temperature (python/llaisys/models/qwen2.py:
212-219; defaults 1, 0.8, 0.8) but picks the arg-max in C++ (src/models/qwen2/qwen2.cpp:80-85).
Here the three are honoured, with that project's meaning of top_k == 1 (greedy):

  top_k == 1 or temperature == 0 -> the first maximum;
  else softmax(logits / temperature), the top_k most probable (0: all), of these the shortest
  descending prefix whose mass reaches top_p, and an inverse-CDF draw over what is kept.

The uniform of a draw is a function of (seed, request key, number of tokens the request has
drawn so far) alone, so a request's tokens do not depend on the batch it runs in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch

from .. import kernels


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 1
    top_p: float = 1.0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must not be negative, got {self.temperature}")
        if not (0 < self.top_p <= 1):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must not be negative (0 keeps every token), got {self.top_k}")

    @property
    def greedy(self) -> bool:
        return self.top_k == 1 or self.temperature == 0


class Sampler:
    """Callable: (logits [R, V] float32 on the device, keys, steps) -> R token ids on the host."""

    def __init__(self, params: SamplingParams = SamplingParams(), seed: int = 0):
        self.params, self.seed = params, int(seed)

    def on_device(self, logits: torch.Tensor, keys: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        p = self.params
        if p.greedy:
            return kernels.argmax(logits)
        k = torch.tensor(list(keys), dtype=torch.int32).to(logits.device, non_blocking=True)
        s = torch.tensor(list(steps), dtype=torch.int32).to(logits.device, non_blocking=True)
        return kernels.sample(logits, p.temperature, p.top_k, p.top_p, self.seed, k, s)

    def __call__(self, logits: torch.Tensor, keys: Sequence[int], steps: Sequence[int]) -> List[int]:
        return self.on_device(logits, keys, steps).tolist()
