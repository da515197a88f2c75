from __future__ import annotations

import torch

from .. import kernels
from .base import KVNeed, Mixer, TensorDecl, build_part, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Mixer):
    """Causal grouped-query attention with a paged key/value cache.

    q, k, v projections (+ bias) -> head view -> position encoding of q and k -> keys and values
    into the cache -> softmax attention over the cache -> output projection
    (xsmccc/llaisys src/models/qwen2/attention.hpp:24-81).  A `window` (not in that project)
    limits a query at position p to the keys p - window < j <= p.

    The three projections are kept as one [(nh + 2 nkvh) dh, H] matrix.  When every sequence
    brings one token (decode) the keys are appended first and attention reads the cache alone;
    otherwise attention reads the step's own keys from the projection output and the cache only
    for earlier positions, and the append follows (so a window layer's ring is never overwritten
    by keys that queries of the same step still need).

    params: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, out_bias, scale, window,
    position (a PartSpec of category "position").
    """

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.nh, self.nkvh, self.dh = (int(p["hidden_size"]), int(p["num_heads"]),
                                                    int(p["num_kv_heads"]), int(p["head_dim"]))
        if self.nh % self.nkvh:
            raise ValueError(f"{self.nh} query heads cannot share {self.nkvh} key/value heads")
        self.qkv_bias, self.out_bias = bool(p.get("qkv_bias", False)), bool(p.get("out_bias", False))
        self.scale = float(p["scale"])
        self.window = p.get("window")
        self.position = build_part("position", p["position"], env) if p.get("position") else None
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    @property
    def capturable(self):
        return self.position is None or self.position.capturable

    def prepare(self, max_positions):
        if self.position is not None:
            self.position.prepare(max_positions)

    def kv_need(self):
        return KVNeed(self.nkvh, self.dh, self.window)

    def tensors(self):
        q, kv = self.nh * self.dh, self.nkvh * self.dh
        t = {"q_proj.weight": TensorDecl((q, self.hidden)), "k_proj.weight": TensorDecl((kv, self.hidden)),
             "v_proj.weight": TensorDecl((kv, self.hidden)), "o_proj.weight": TensorDecl((self.hidden, q))}
        if self.qkv_bias:
            t.update({"q_proj.bias": TensorDecl((q,)), "k_proj.bias": TensorDecl((kv,)),
                      "v_proj.bias": TensorDecl((kv,))})
        if self.out_bias:
            t["o_proj.bias"] = TensorDecl((self.hidden,))
        return t

    def load(self, tensors):
        def fuse(names):
            ts = [tensors[n] for n in names]
            dt = ts[0].dtype
            for t in ts[1:]:
                dt = torch.promote_types(dt, t.dtype)
            return torch.cat([t.to(dt) for t in ts], dim=0).contiguous()

        self.w_qkv = fuse(["q_proj.weight", "k_proj.weight", "v_proj.weight"])
        self.b_qkv = fuse(["q_proj.bias", "k_proj.bias", "v_proj.bias"]) if self.qkv_bias else None
        self.w_o = tensors["o_proj.weight"].contiguous()
        self.b_o = tensors["o_proj.bias"].contiguous() if self.out_bias else None

    def forward(self, x, ctx, call):
        kv = ctx.kv(call)
        qkv = kernels.linear(x, self.w_qkv, self.b_qkv)
        append = None
        if kv.writable:
            append = dict(tok_seq=ctx.tok_seq, seq_start=ctx.seq_start, seq_len_before=ctx.seq_len_before,
                          kpool=kv.k, vpool=kv.v, page_table=kv.page_table, ring=kv.ring)
        decode = ctx.is_decode
        common = (qkv, self.nh, self.nkvh, self.dh, kv.k, kv.v, kv.page_table, kv.ring,
                  ctx.seq_start, ctx.seq_len_before, ctx.n_seqs)
        if decode:
            fused_tables = getattr(self.position, "fused_tables", None) if self.position is not None else None
            if kernels.decode_fusion_ok(qkv.dtype, self.dh) and (self.position is None or fused_tables is not None):
                # the attention kernel rotates the query and the new key itself and appends to the cache
                rope = fused_tables(ctx.max_position + 1) if fused_tables is not None else None
                out = kernels.attention_decode(*common, self.window, self.scale, n_splits=ctx.decode_splits(self.nkvh, kernels.decode_clusters16(qkv.dtype, self.dh)),
                                               rope=rope, append_new=kv.writable)
            else:
                # position encoding; the same kernel also appends to the cache
                if self.position is not None:
                    self.position.apply(qkv, self.nh, self.nkvh, ctx, append=append)
                elif append:
                    kernels.rope_append(qkv, self.nh, self.nkvh, self.dh, tok_pos=ctx.tok_pos, append=append, err=ctx.err)
                out = kernels.attention_decode(*common, self.window, self.scale, n_splits=ctx.decode_splits(self.nkvh))
        elif self.window is None and kernels.prefill_tc_ok(qkv.dtype, self.dh):
            # every key is kept: append first (in the rotation kernel), then attend over the cache alone
            if self.position is not None:
                self.position.apply(qkv, self.nh, self.nkvh, ctx, append=append)
            elif append:
                kernels.rope_append(qkv, self.nh, self.nkvh, self.dh, tok_pos=ctx.tok_pos, append=append, err=ctx.err)
            out = kernels.attention_prefill(*common, ctx.max_new, self.window, self.scale, all_from_cache=True)
        else:
            if self.position is not None:
                self.position.apply(qkv, self.nh, self.nkvh, ctx, append=None)
            out = kernels.attention_prefill(*common, ctx.max_new, self.window, self.scale,
                                            all_from_cache=not kv.writable)
            if append:
                kernels.rope_append(qkv, self.nh, self.nkvh, self.dh, tok_pos=ctx.tok_pos, append=append, err=ctx.err)
        return kernels.linear(out, self.w_o, self.b_o)
