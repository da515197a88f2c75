from __future__ import annotations

from .. import kernels
from .base import Norm, TensorDecl, register_part


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    """y = x * w / sqrt(mean(x^2) + eps): eps inside the root, plain weight
    (xsmccc/llaisys src/ops/rms_norm/cpu/rms_norm_cpu.cpp:15-34), fused with the residual add
    that precedes it (src/models/qwen2/layer.hpp:60-71).  params: size, eps."""
    capturable = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size, self.eps = int(spec.params["size"]), float(spec.params["eps"])
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.size,), init="one_plus_normal", use="vector")}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def forward(self, residual, delta=None, rows=None):
        return kernels.add_rmsnorm(residual, delta, self.weight, self.eps, self.env.dtype, rows=rows)
