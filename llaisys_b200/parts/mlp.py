from __future__ import annotations

import torch

from .. import kernels
from .base import FeedForward, TensorDecl, register_part


@register_part("ffn", "swiglu_mlp")
class SwiGLUMLP(FeedForward):
    """down(up(x) * silu(gate(x))), no biases (xsmccc/llaisys src/models/qwen2/mlp.hpp:18-39,
    src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21).  The gate and up matrices are kept as one
    [2I, H] matrix so that one product serves both.  params: hidden_size, intermediate_size."""
    capturable = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        self.gate_up = self.down = None

    def tensors(self):
        return {"gate_proj.weight": TensorDecl((self.inter, self.hidden)),
                "up_proj.weight": TensorDecl((self.inter, self.hidden)),
                "down_proj.weight": TensorDecl((self.hidden, self.inter))}

    def load(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        dt = torch.promote_types(g.dtype, u.dtype)
        self.gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, x, ctx):
        return kernels.linear(kernels.linear_swiglu(x, self.gate_up), self.down)

    def forward_into(self, x, ctx, residual):
        # a few tokens (decode): the three matrices stream through one launch that ends in the residual add
        if kernels.mlp_fused_ok(x, self.gate_up, self.down, residual):
            kernels.mlp_fused(x, self.gate_up, self.down, residual)
            return True
        # more tokens: the down projection's tiles are added to the stream as they are finished
        if x.dtype == torch.bfloat16 and self.gate_up.dtype == torch.bfloat16 and x.shape[0] > 0:
            act = kernels.linear_swiglu(x, self.gate_up)
            if kernels.linear_into_ok(act, self.down, None, residual):
                kernels.linear_into(act, self.down, None, residual)
                return True
            kernels.residual_add(residual, kernels.linear(act, self.down))
            return True
        return False
