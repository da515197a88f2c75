"""The operators on the CPU: plain float32 numpy, one function per operator, written from the
formulas of xsmccc/llaisys' CPU operators (src/ops/*/cpu/*.cpp: inputs of any supported dtype are
computed in float32 and rounded once at the output, README.md:156).

This is the reference beside each CUDA operator, as that project keeps one (src/ops/linear/op.cpp:48-58
dispatches on the device): `llaisys_b200.ops.Ops` runs these when its operands live on the CPU, the
op tests compare the CUDA kernels with them, and the command line's --test and --device cpu
generate with a model put together from them.  It is not a fallback of the engine: the engine
runs on a CUDA device only.
"""
from __future__ import annotations

import numpy as np


def add(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """c = a + b (src/ops/add/cpu/add_cpu.cpp:8-16)."""
    return a.astype(np.float32) + b.astype(np.float32)


def argmax(vals: np.ndarray):
    """(index of the first maximum, the maximum): strict > scan from index 0
    (src/ops/argmax/cpu/argmax_cpu.cpp:14-27)."""
    v = vals.astype(np.float32).reshape(-1)
    i = int(np.argmax(v))
    return i, v[i]


def embedding(index: np.ndarray, weight: np.ndarray) -> np.ndarray:
    """out[t] = weight[index[t]] (src/ops/embedding/cpu/embedding_cpu.cpp:16-22)."""
    idx = np.asarray(index, dtype=np.int64)
    if idx.size and (idx.min() < 0 or idx.max() >= weight.shape[0]):
        raise IndexError(f"embedding: index outside the table of {weight.shape[0]} rows")
    return weight[idx]


def linear(x: np.ndarray, weight: np.ndarray, bias=None) -> np.ndarray:
    """y = x W^T + b with W [out, in], float32 accumulation (src/ops/linear/cpu/linear_cpu.cpp:21-40)."""
    y = x.astype(np.float32) @ weight.astype(np.float32).T
    if bias is not None:
        y = y + bias.astype(np.float32)
    return y


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """y = (x * w) / sqrt(mean(x^2) + eps), eps inside the root (src/ops/rms_norm/cpu/rms_norm_cpu.cpp:15-34)."""
    x = x.astype(np.float32)
    ss = (x * x).sum(axis=-1, keepdims=True, dtype=np.float32)
    inv = np.float32(1.0) / np.sqrt(ss / np.float32(x.shape[-1]) + np.float32(eps))
    return (x * weight.astype(np.float32)) * inv


def rope(x: np.ndarray, pos_ids: np.ndarray, theta: float) -> np.ndarray:
    """Half-split rotation of x [seq, heads, d]: phi = p / theta^(2j/d) in double precision from theta
    held as a C float; (a, b) = (x[j], x[j + d/2]) -> (a cos - b sin, b cos + a sin)
    (src/ops/rope/cpu/rope_cpu.cpp:16-46)."""
    d = x.shape[-1]
    half = d // 2
    t = float(np.float32(theta))
    freq = 1.0 / np.power(t, 2.0 * np.arange(half, dtype=np.float64) / d)
    ang = np.asarray(pos_ids, dtype=np.float64)[:, None] * freq[None, :]
    cos, sin = np.cos(ang)[:, None, :].astype(np.float32), np.sin(ang)[:, None, :].astype(np.float32)
    x = x.astype(np.float32)
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1)


def self_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window=None) -> np.ndarray:
    """Causal grouped-query attention of q [qlen, nh, d] over k, v [kvlen, nkvh, d], the queries being
    the last qlen of the kvlen positions: query i sees keys t <= kvlen - qlen + i; head h reads kv head
    h // (nh / nkvh); softmax with the maximum subtracted (src/ops/self_attention/cpu/self_attention_cpu.cpp:28-112).
    window (not in that project): a query at position p sees only the keys p - window < t <= p."""
    qlen, nh, d = q.shape
    kvlen, nkvh, dv = v.shape
    group = nh // nkvh
    q, k, v = q.astype(np.float32), k.astype(np.float32), v.astype(np.float32)
    out = np.zeros((qlen, nh, dv), dtype=np.float32)
    t = np.arange(kvlen)
    cur = (kvlen - qlen + np.arange(qlen))[:, None]
    visible = t[None, :] <= cur
    if window is not None:
        visible &= t[None, :] > cur - window
    for h in range(nh):
        s = (q[:, h, :] @ k[:, h // group, :].T) * np.float32(scale)
        s = np.where(visible, s, -np.inf)
        e = np.where(visible, np.exp(s - s.max(axis=-1, keepdims=True)), 0.0).astype(np.float32)
        out[:, h, :] = (e / e.sum(axis=-1, keepdims=True)) @ v[:, h // group, :]
    return out


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """out = up * gate / (1 + exp(-gate)) (src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21)."""
    g, u = gate.astype(np.float32), up.astype(np.float32)
    return u * (g / (np.float32(1.0) + np.exp(-g)))
