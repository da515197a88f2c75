"""The operators one by one, with the names and argument order of xsmccc/llaisys' `llaisys.Ops`
(python/llaisys/ops.py:6-55): the result tensor comes first and is written in place.

Tensors are torch tensors (float32, bfloat16 or float16; indices int64 or int32).  Where the
operands live chooses the implementation, as that project's operators dispatch on the device
(src/ops/linear/op.cpp:48-58): on a CUDA device the kernels of this package run (float16 goes
through the float32 kernels and is rounded once at the end); on the CPU the plain float32
functions of `cpu_ops`.  All operands of a call must live on the same device.

    add, argmax, embedding, linear (bias may be None), rearrange, rms_norm, rope, self_attention, swiglu
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from . import cpu_ops

_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


def _same_device(*ts):
    devs = {t.device for t in ts if t is not None}
    if len(devs) != 1:
        raise ValueError(f"the operands of an operator must live on one device, got {sorted(map(str, devs))}")
    return devs.pop()


def _np(t: Optional[torch.Tensor]):
    if t is None:
        return None
    return t.detach().float().numpy() if t.dtype in _FLOATS else t.detach().numpy()


def _put(out: torch.Tensor, value: np.ndarray):
    out.copy_(torch.from_numpy(np.ascontiguousarray(value)).to(out.dtype).view(out.shape))


def _work(t: torch.Tensor) -> torch.Tensor:
    """The tensor in a dtype the kernels take (float16 -> float32), contiguous."""
    if t.dtype not in _FLOATS:
        raise TypeError(f"dtype {t.dtype} is not supported (float32, bfloat16, float16)")
    return (t.float() if t.dtype == torch.float16 else t).contiguous()


class Ops:
    @staticmethod
    def add(c: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> None:
        """c = a + b."""
        if _same_device(c, a, b).type == "cpu":
            return _put(c, cpu_ops.add(_np(a), _np(b)))
        from . import kernels
        wa, wb = _work(a), _work(b)
        out = c if (c.dtype == wa.dtype and c.is_contiguous()) else torch.empty_like(wa)
        kernels.dense_binary(out, wa, wb, "add")
        if out is not c:
            c.copy_(out)

    @staticmethod
    def argmax(max_idx: torch.Tensor, max_val: torch.Tensor, vals: torch.Tensor) -> None:
        """max_idx[0] = index of the first maximum of the 1-D `vals`, max_val[0] = that maximum."""
        if _same_device(max_idx, max_val, vals).type == "cpu":
            i, v = cpu_ops.argmax(_np(vals))
            max_idx.fill_(i)
            max_val.fill_(float(v))
            return
        from . import kernels
        idx = kernels.argmax(vals.reshape(1, -1).float().contiguous())          # exact for 16-bit inputs
        max_idx.copy_(idx.to(max_idx.dtype))
        max_val.copy_(vals.reshape(-1)[idx.long()])

    @staticmethod
    def embedding(out: torch.Tensor, index: torch.Tensor, weight: torch.Tensor) -> None:
        """out[t] = weight[index[t]]."""
        if _same_device(out, index, weight).type == "cpu":
            return _put(out, cpu_ops.embedding(_np(index), _np(weight)))
        from . import kernels
        err = torch.zeros(1, dtype=torch.int32, device=out.device)
        rows = kernels.embedding(index.to(torch.int32).contiguous(), _work(weight), err)
        if int(err.item()):
            raise IndexError(f"embedding: index outside the table of {weight.shape[0]} rows")
        out.copy_(rows)                                                          # float32 rows of 16-bit values: exact

    @staticmethod
    def linear(out: torch.Tensor, inp: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """out = inp weight^T + bias, weight [out features, in features]; bias may be None."""
        if _same_device(out, inp, weight, bias).type == "cpu":
            return _put(out, cpu_ops.linear(_np(inp), _np(weight), _np(bias)))
        from . import kernels
        y = kernels.linear(_work(inp), _work(weight), _work(bias) if bias is not None else None)
        out.copy_(y)

    @staticmethod
    def rearrange(out: torch.Tensor, inp: torch.Tensor) -> None:
        """out <- inp element by element, whatever the strides of the two."""
        if out.shape != inp.shape:
            raise ValueError(f"rearrange: shapes differ, {tuple(out.shape)} and {tuple(inp.shape)}")
        out.copy_(inp)

    @staticmethod
    def rms_norm(out: torch.Tensor, inp: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
        """out = inp * weight / sqrt(mean(inp^2) + eps) along the last dimension."""
        if _same_device(out, inp, weight).type == "cpu":
            return _put(out, cpu_ops.rms_norm(_np(inp), _np(weight), eps))
        from . import kernels
        x = inp.reshape(-1, inp.shape[-1]).float().contiguous()
        kdt = torch.bfloat16 if out.dtype == torch.bfloat16 else torch.float32
        y = kernels.add_rmsnorm(x, None, _work(weight), eps, kdt)
        out.copy_(y.view(inp.shape))

    @staticmethod
    def rope(out: torch.Tensor, inp: torch.Tensor, pos_ids: torch.Tensor, theta: float) -> None:
        """out = inp [seq, heads, d] rotated by its positions (half-split pairs)."""
        if _same_device(out, inp, pos_ids).type == "cpu":
            return _put(out, cpu_ops.rope(_np(inp), _np(pos_ids), theta))
        from . import kernels
        from .config.spec import PartSpec
        from .parts.base import BuildEnv
        from .parts.rope import RotaryHalfSplit
        seq, heads, d = inp.shape
        x = _work(inp).clone().view(seq, heads * d)
        table = RotaryHalfSplit(PartSpec("rope_half_split", {"head_dim": d, "theta": theta}), BuildEnv(x.dtype, x.device))
        cos, sin = table.table(int(pos_ids.max().item()) + 1 if seq else 1)
        err = torch.zeros(1, dtype=torch.int32, device=x.device)
        kernels.rope_append(x, heads, 0, d, cos=cos, sin=sin, tok_pos=pos_ids.to(torch.int32).contiguous(), err=err)
        if int(err.item()):
            raise IndexError("rope: a position is negative")
        out.copy_(x.view(seq, heads, d))

    @staticmethod
    def self_attention(attn_val: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> None:
        """attn_val [qlen, nh, d] = causal softmax(q k^T * scale) v for q [qlen, nh, d] and k, v [kvlen, nkvh, d],
        the queries being the last qlen of the kvlen positions (qlen <= kvlen)."""
        qlen, nh, d = q.shape
        kvlen, nkvh, _ = k.shape
        if qlen > kvlen or nh % nkvh or v.shape != k.shape:
            raise ValueError("self_attention: wants qlen <= kvlen, nh a multiple of nkvh, and k and v of one shape")
        if _same_device(attn_val, q, k, v).type == "cpu":
            return _put(attn_val, cpu_ops.self_attention(_np(q), _np(k), _np(v), scale))
        from . import kernels
        from .cache.kv import PAGE
        dev = q.device
        qw = _work(q).view(qlen, nh * d)
        pages = -(-kvlen // PAGE)

        def paged(t):                                   # [kvlen, nkvh, d] -> pages of [nkvh, PAGE, d]
            buf = torch.zeros((pages * PAGE, nkvh, d), dtype=qw.dtype, device=dev)
            buf[:kvlen] = t
            return buf.view(pages, PAGE, nkvh, d).permute(0, 2, 1, 3).contiguous()

        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        seq_start = torch.tensor([0, qlen], dtype=torch.int32, device=dev)
        before = torch.tensor([kvlen - qlen], dtype=torch.int32, device=dev)
        # the queries alone stand in the place of the packed projections: every key is read from the pages
        o = kernels.attention_prefill(qw, nh, nkvh, d, paged(_work(k)), paged(_work(v)), table, pages, seq_start, before,
                                      1, qlen, None, float(scale), all_from_cache=True)
        attn_val.copy_(o.view(qlen, nh, d))

    @staticmethod
    def swiglu(out: torch.Tensor, gate: torch.Tensor, up: torch.Tensor) -> None:
        """out = up * gate / (1 + exp(-gate))."""
        if _same_device(out, gate, up).type == "cpu":
            return _put(out, cpu_ops.swiglu(_np(gate), _np(up)))
        from . import kernels
        g, u = _work(gate), _work(up)
        y = out if (out.dtype == g.dtype and out.is_contiguous()) else torch.empty_like(g)
        kernels.dense_binary(y, g, u, "swiglu")
        if y is not out:
            out.copy_(y)


add, argmax, embedding, linear, rearrange = Ops.add, Ops.argmax, Ops.embedding, Ops.linear, Ops.rearrange
rms_norm, rope, self_attention, swiglu = Ops.rms_norm, Ops.rope, Ops.self_attention, Ops.swiglu
