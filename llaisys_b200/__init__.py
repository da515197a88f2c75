"""llaisys_b200: a small model library with generation of its own for one NVIDIA B200.

It takes a model folder (config.json and safetensors) of the Qwen2 dense decoder to generated
tokens: typed configuration and architecture registry (`config`), weights by tensor name
(`weights`), layers put together from parts (`parts`), a paged key/value cache with slots
(`cache`), one step function and a generation loop (`engine`), greedy / temperature / top-k /
top-p sampling (`sampling`), and hand-written CUDA kernels for sm_100a (`csrc`, `kernels`).
"""
from . import config, weights, parts, cache, engine  # noqa: F401

__version__ = "0.1.0"
