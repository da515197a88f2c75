"""llaisys_b200: a small model library with generation of its own for one NVIDIA B200.

It takes a model folder (config.json and safetensors) of the Qwen2 dense decoder to generated
tokens: typed configuration and architecture registry (`config`), weights by tensor name
(`weights`), layers put together from parts (`parts`), a paged key/value cache with slots
(`cache`), one step function and a generation loop (`engine`), greedy / temperature / top-k /
top-p sampling (`sampling`), and hand-written CUDA kernels for sm_100a (`csrc`, `kernels`).
"""
import importlib
import os

from . import config, weights, parts, cache, engine  # noqa: F401

__version__ = "0.2.0"

# Modules named in LLAISYS_PLUGINS (comma-separated, importable names) are imported with the package:
# this is how an architecture or a part defined outside the package reaches programs that are started
# as processes of their own (the command line, bin/trace_run).  Such a module registers what it
# defines with config.register_architecture and parts.register_part.
for _name in filter(None, (n.strip() for n in os.environ.get("LLAISYS_PLUGINS", "").split(","))):
    importlib.import_module(_name)
