from __future__ import annotations

from .base import Block, register_part


@register_part("block", "pre_norm_residual")
class PreNormResidual(Block):
    """x -> norm -> mixer -> +x -> norm -> feed-forward -> +   (xsmccc/llaisys
    src/models/qwen2/layer.hpp:47-84).  Each residual add is done by the norm that follows it,
    so the block hands its last delta on to the next block (or to the final norm)."""
    capturable = True


    def forward(self, residual, pending, ctx, call):
        h = self.mixer_norm.forward(residual, pending)
        d = self.mixer.forward(h, ctx, call)
        h = self.ffn_norm.forward(residual, d)
        return residual, self.ffn.forward(h, ctx)
