from __future__ import annotations

from .. import kernels
from .base import Part, TensorDecl, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """x[t] = E[id[t]] (xsmccc/llaisys src/ops/embedding/cpu/embedding_cpu.cpp:16-22), written
    as the float32 residual stream.  An id outside the table is reported through ctx.err.
    params: vocab_size, hidden_size."""
    capturable = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.vocab, self.hidden))}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def forward(self, ctx):
        return kernels.embedding(ctx.tokens, self.weight, ctx.err)


@register_part("head", "lm_head")
class LMHead(Part):
    """logits = h W^T in float32, no bias (xsmccc/llaisys src/models/qwen2/qwen2.cpp:76-77).
    With params["tied_to"] set, W is the tensor of that name (the embedding table) and the part
    declares no tensor of its own.  params: vocab_size, hidden_size, tied_to."""
    capturable = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.tied_to = spec.params.get("tied_to")
        self.weight = None

    def tensors(self):
        return {} if self.tied_to else {"weight": TensorDecl((self.vocab, self.hidden))}

    def load(self, tensors):
        if not self.tied_to:
            self.weight = tensors["weight"].contiguous()

    def tie(self, weight):
        self.weight = weight

    def forward(self, h):
        import torch
        return kernels.linear(h, self.weight, out_dtype=torch.float32)
