from __future__ import annotations

from .base import Block, register_part


@register_part("block", "pre_norm_residual")
class PreNormResidual(Block):
    """x -> norm -> part -> + for every sub-layer in turn; with a mixer and a feed-forward that is
    x -> norm -> mixer -> +x -> norm -> feed-forward -> +   (xsmccc/llaisys
    src/models/qwen2/layer.hpp:47-84).  A part that can add its result to the residual stream in its
    own last kernel does so (forward_into); otherwise the add is done by the norm that follows, so
    the block hands its last delta on to the next block (or to the final norm).  A sub-layer
    without a norm of its own gets the residual stream as it is (the pending delta added)."""
    capturable = True

    def forward(self, residual, pending, ctx, users):
        from .. import kernels
        mixers = iter(users)
        for sub in self.sublayers:
            if sub.norm is not None:
                h = sub.norm.forward(residual, pending)
            else:
                if pending is not None:
                    kernels.residual_add(residual, pending)
                h = residual.to(self.env.dtype)
            if sub.category == "mixer":
                call = next(mixers)
                pending = None if sub.part.forward_into(h, ctx, call, residual) else sub.part.forward(h, ctx, call)
            else:
                pending = None if sub.part.forward_into(h, ctx, residual) else sub.part.forward(h, ctx)
        return residual, pending
