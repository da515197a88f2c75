from __future__ import annotations

import torch

from .. import kernels
from .base import KVNeed, Mixer, TensorDecl, build_part, register_part


def decode_splits(ctx, n_kv_heads: int, clusters16: int = 0) -> int:
    """Slices of the key range in decode attention: enough blocks to fill the device, at most
    one slice per page the widest page table of the step can hold (a function of the step's
    shape alone, so a captured step stays valid as sequences grow).  clusters16: how many
    clusters of sixteen blocks of the kernel the device holds at once (0: none)."""
    pages = max(ctx.widths) if ctx.widths else 1
    # two blocks fit an SM; more blocks than that would run as a second, mostly empty wave
    want = (2 * ctx.sm_count) // max(1, ctx.n_seqs * n_kv_heads)
    splits = max(1, min(want, pages, 64))
    # Sixteen slices in one (non-portable) cluster for small batches: a block then walks three pages at most
    # at contexts up to 3,000 tokens, all of them requested before the step's earlier kernels have finished.
    # Only while the blocks leave every second place on the SMs free: at batch 8 (two blocks on every SM)
    # the step was measured 1.3 % slower than with eight slices, at batch 1 it is 2.3 % faster.
    n_clusters = ctx.n_seqs * n_kv_heads
    if splits >= 16 and pages > 16 and n_clusters <= clusters16 and n_clusters * 16 <= ctx.sm_count:
        return 16
    # up to eight slices merge inside a thread-block cluster (by pushing their partial sums to each other), which is
    # cheaper than a second kernel: prefer that while a block then has at most thirty-two pages to walk.  Measured
    # at batch 8: context 8,192 (table width 256) 1.401 ms a step with eight slices against 1.451 with eighteen and
    # the merge kernel; context 16,384 1.856 against 1.736; context 32,768 2.75 against 2.35.
    if splits > 8 and pages <= 8 * 32:
        splits = 8
    return splits


@register_part("mixer", "gqa_attention")
class GQAttention(Mixer):
    """Causal grouped-query attention with a paged key/value cache.

    q, k, v projections (+ bias) -> head view -> position encoding of q and k -> keys and values
    into the cache -> softmax attention over the cache -> output projection
    (xsmccc/llaisys src/models/qwen2/attention.hpp:24-81).  A `window` (not in that project)
    limits a query at position p to the keys p - window < j <= p.

    The three projections are kept as one [(nh + 2 nkvh) dh, H] matrix.  Storing keys and values
    in the cache is this part's business, not the position encoding's: an encoding that hands out
    rotation tables is applied by this part's kernels in the same pass that stores the keys (in
    decode inside the attention kernel itself); any other encoding is asked to apply() itself and
    the keys are stored by a pass of their own.  When every sequence brings one token (decode), and
    in a layer that keeps every key, the keys are appended first and attention reads the cache alone;
    a window layer's attention reads the step's own keys from the projection output and the cache
    only for earlier positions, and the append follows (so its ring is never overwritten by keys
    that queries of the same step still need).

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
        kernels.require_head_dim(self.dh)            # a head size no kernel takes is refused here, not at the first step
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
        return KVNeed(self.nkvh, self.dh, self.dh, self.window)

    def tensors(self):
        q, kv = self.nh * self.dh, self.nkvh * self.dh
        t = {"q_proj.weight": TensorDecl((q, self.hidden)), "k_proj.weight": TensorDecl((kv, self.hidden)),
             "v_proj.weight": TensorDecl((kv, self.hidden)), "o_proj.weight": TensorDecl((self.hidden, q))}
        if self.qkv_bias:
            t.update({"q_proj.bias": TensorDecl((q,), use="vector"), "k_proj.bias": TensorDecl((kv,), use="vector"),
                      "v_proj.bias": TensorDecl((kv,), use="vector")})
        if self.out_bias:
            t["o_proj.bias"] = TensorDecl((self.hidden,), use="vector")
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
        return kernels.linear(self._attend(x, ctx, call), self.w_o, self.b_o)

    def forward_into(self, x, ctx, call, residual):
        # the output projection's tiles are added to the residual stream as they are finished
        if not (x.dtype == torch.bfloat16 and self.w_o.dtype == torch.bfloat16
                and kernels.linear_into_ok(x.new_empty((x.shape[0], self.nh * self.dh)), self.w_o, self.b_o, residual)):
            return False
        kernels.linear_into(self._attend(x, ctx, call), self.w_o, self.b_o, residual)
        return True

    def _attend(self, x, ctx, call):
        """Projections, position encoding, cache append and attention: [T, nh * dh], before the output projection."""
        kv = ctx.kv(call)
        qkv = kernels.linear(x, self.w_qkv, self.b_qkv)
        append = None
        if kv.writable:
            append = dict(tok_seq=ctx.tok_seq, seq_start=ctx.seq_start, seq_len_before=ctx.seq_len_before,
                          kpool=kv.k, vpool=kv.v, page_table=kv.page_table, ring=kv.ring)
        tables = self.position.rotation_tables(ctx.max_position + 1) if self.position is not None else None
        by_kernel = self.position is None or tables is not None       # this part's kernels can do the rotation

        def rotate(store):
            """Position encoding of q and k; with `store` the keys and values also go into the cache."""
            cos, sin = tables if tables is not None else (None, None)
            if not by_kernel:
                self.position.apply(qkv, self.nh, self.nkvh, ctx)
            if (by_kernel and tables is not None) or store:
                kernels.rope_append(qkv, self.nh, self.nkvh, self.dh, cos=cos if by_kernel else None,
                                    sin=sin if by_kernel else None, tok_pos=ctx.tok_pos,
                                    append=append if store else None, err=ctx.err)

        common = (qkv, self.nh, self.nkvh, self.dh, kv.k, kv.v, kv.page_table, kv.ring,
                  ctx.seq_start, ctx.seq_len_before, ctx.n_seqs)
        if ctx.is_decode:
            if kernels.decode_fusion_ok(qkv.dtype, self.dh) and by_kernel:
                # the attention kernel rotates the query and the new key itself and appends to the cache
                splits = decode_splits(ctx, self.nkvh, kernels.decode_clusters16(qkv.dtype, self.dh))
                out = kernels.attention_decode(*common, self.window, self.scale, n_splits=splits,
                                               rope=tables, append_new=kv.writable)
            else:
                rotate(store=kv.writable)
                out = kernels.attention_decode(*common, self.window, self.scale, n_splits=decode_splits(ctx, self.nkvh))
        elif self.window is None and kernels.prefill_tc_ok(qkv.dtype, self.dh):
            # every key is kept: append first (in the rotation kernel), then attend over the cache alone
            rotate(store=kv.writable)
            out = kernels.attention_prefill(*common, ctx.max_new, self.window, self.scale, all_from_cache=True)
        else:
            rotate(store=False)
            out = kernels.attention_prefill(*common, ctx.max_new, self.window, self.scale,
                                            all_from_cache=not kv.writable)
            if append:
                kernels.rope_append(qkv, self.nh, self.nkvh, self.dh, tok_pos=ctx.tok_pos, append=append, err=ctx.err)
        return out
