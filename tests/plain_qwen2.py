"""Plain, slow Qwen2 decoder: the oracle the engine is compared with.

Whole sequences, no cache, one function for each part, float64 numpy throughout.
Nothing here imports the product package; even the safetensors reader is its own.

Written from the formulas of xsmccc/llaisys' CPU operators and model code (paths are
relative to that project's root).  It was compared once with that project's own
compiled CPU code on a tiny random model; the outputs of that run and the script
that produced them are under tests/golden/.

The sliding window, the tied head, temperature / top-k / top-p sampling and batching
are not in xsmccc/llaisys' code: those functions rest on the formulas stated in their
docstrings.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- files

_ST_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": None,
              "I64": np.int64, "I32": np.int32}


def read_safetensors(path) -> dict:
    """name -> float64 (or integer) numpy array.  Format: 8-byte little-endian header
    length, JSON header {name: {dtype, shape, data_offsets}}, raw little-endian data."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[base + lo: base + hi]
        if info["dtype"] == "BF16":
            u16 = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            arr = u16.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(buf, dtype=np.dtype(_ST_DTYPES[info["dtype"]]).newbyteorder("<"))
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = arr.reshape(info["shape"])
    return out


def load_model_folder(folder):
    """(config dict, weights dict) of a folder with config.json and *.safetensors
    (python/llaisys/models/qwen2.py:39-44, :99-112)."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = {}
    for f in sorted(folder.glob("*.safetensors")):
        weights.update(read_safetensors(f))
    return config, weights


# --------------------------------------------------------------------------- parts

def embedding(ids, table):
    """x[t,:] = E[id[t],:]  (src/ops/embedding/cpu/embedding_cpu.cpp:16-22)."""
    ids = np.asarray(ids, dtype=np.int64)
    assert ids.min() >= 0 and ids.max() < table.shape[0], "token id out of range"
    return table[ids].copy()


def rms_norm(x, weight, eps):
    """y = x * w / sqrt(mean(x^2) + eps), eps inside the root, plain weight
    (src/ops/rms_norm/cpu/rms_norm_cpu.cpp:15-34)."""
    ss = (x * x).sum(axis=-1, keepdims=True)
    inv = 1.0 / np.sqrt(ss / x.shape[-1] + eps)
    return x * weight * inv


def linear(x, weight, bias=None):
    """Y = X W^T + b, W stored [out, in]  (src/ops/linear/cpu/linear_cpu.cpp:21-40)."""
    y = x @ weight.T
    if bias is not None:
        y = y + bias
    return y


def rope(x, positions, theta):
    """Half-split rotation of x[T, heads, d]: for j < d/2, phi = p / theta^(2j/d),
    (a, b) = (x[j], x[j+d/2]) -> (a cos - b sin, b cos + a sin)
    (src/ops/rope/cpu/rope_cpu.cpp:16-46).  theta reaches that code as a C float
    (include/llaisys/models/qwen2.h:7-12), so it is rounded to float32 first."""
    T, _, d = x.shape
    half = d // 2
    theta = float(np.float32(theta))
    j = np.arange(half, dtype=np.float64)
    freq = 1.0 / np.power(theta, 2.0 * j / d)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]    # [T, half]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1)


def self_attention(q, k, v, scale, window=None):
    """Causal grouped-query softmax attention of q[S, nh, d] over k, v[L, nkvh, d],
    the queries being the last S of the L positions
    (src/ops/self_attention/cpu/self_attention_cpu.cpp:28-112): query i stands at
    position cur = L - S + i and sees keys t <= cur; head h reads kv head h // (nh/nkvh).

    window (not in xsmccc/llaisys): a query at position p sees only keys j with
    p - window < j <= p, i.e. `window` keys counting itself."""
    S, nh, d = q.shape
    L, nkvh, _ = k.shape
    group = nh // nkvh
    out = np.zeros((S, nh, v.shape[-1]), dtype=np.float64)
    t = np.arange(L)
    for h in range(nh):
        kh, vh = k[:, h // group, :], v[:, h // group, :]
        for i in range(S):
            cur = L - S + i
            s = (kh @ q[i, h]) * scale
            visible = t <= cur
            if window is not None:
                visible &= t > cur - window
            s = np.where(visible, s, -np.inf)
            e = np.where(visible, np.exp(s - s.max()), 0.0)
            out[i, h] = (e / e.sum()) @ vh
    return out


def swiglu(gate, up):
    """out = up * gate / (1 + exp(-gate))  (src/ops/swiglu/cpu/swiglu_cpu.cpp:13-21)."""
    return up * (gate / (1.0 + np.exp(-gate)))


def argmax(values):
    """Index of the first maximum (strict > scan from index 0,
    src/ops/argmax/cpu/argmax_cpu.cpp:14-27)."""
    return int(np.argmax(values))


# --------------------------------------------------------------------------- model

def layer_window(config, layer):
    """Window of a layer, or None.  Not in xsmccc/llaisys (its config reader takes no
    window key, python/llaisys/models/qwen2.py:50-64).  Rule: layer l is windowed iff
    use_sliding_window and l >= max_window_layers; the window is sliding_window keys."""
    if not config.get("use_sliding_window", False):
        return None
    if layer < config.get("max_window_layers", config["num_hidden_layers"]):
        return None
    return int(config["sliding_window"])


def attention_block(x, positions, config, w, prefix, window):
    """q/k/v projections with bias, head view, RoPE on q and k, attention over all
    positions, output projection  (src/models/qwen2/attention.hpp:24-81)."""
    nh, nkvh = config["num_attention_heads"], config["num_key_value_heads"]
    dh = config.get("head_dim") or config["hidden_size"] // nh
    T = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias")).reshape(T, nh, dh)
    k = linear(x, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias")).reshape(T, nkvh, dh)
    v = linear(x, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias")).reshape(T, nkvh, dh)
    q = rope(q, positions, config["rope_theta"])
    k = rope(k, positions, config["rope_theta"])
    o = self_attention(q, k, v, 1.0 / math.sqrt(dh), window)          # attention.hpp:67
    return linear(o.reshape(T, nh * dh), w[prefix + "o_proj.weight"])


def mlp_block(x, w, prefix):
    """down(swiglu(gate(x), up(x)))  (src/models/qwen2/mlp.hpp:18-39)."""
    g = linear(x, w[prefix + "gate_proj.weight"])
    u = linear(x, w[prefix + "up_proj.weight"])
    return linear(swiglu(g, u), w[prefix + "down_proj.weight"])


def decoder_layer(x, positions, config, w, layer):
    """x -> norm -> attention -> +x -> norm -> mlp -> +  (src/models/qwen2/layer.hpp:47-84)."""
    p = f"model.layers.{layer}."
    eps = config["rms_norm_eps"]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    x = attention_block(h, positions, config, w, p + "self_attn.", layer_window(config, layer)) + x
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    return mlp_block(h, w, p + "mlp.") + x


def forward_logits(tokens, config, w):
    """Logits [T, vocab] of one whole sequence starting at position 0
    (src/models/qwen2/qwen2.cpp:58-77, applied to every position instead of the last).
    The head is lm_head.weight; when tie_word_embeddings is set or that tensor is
    absent it is the embedding table (not in xsmccc/llaisys, which needs the tensor)."""
    positions = np.arange(len(tokens))
    x = embedding(tokens, w["model.embed_tokens.weight"])
    for layer in range(config["num_hidden_layers"]):
        x = decoder_layer(x, positions, config, w, layer)
    x = rms_norm(x, w["model.norm.weight"], config["rms_norm_eps"])
    head = w.get("lm_head.weight")
    if config.get("tie_word_embeddings", False) or head is None:
        head = w["model.embed_tokens.weight"]
    return linear(x, head)


# --------------------------------------------------------------------------- sampling

def sample(logits, temperature=1.0, top_k=0, top_p=1.0, u=0.0):
    """One token from one row of logits, with a given uniform draw u in [0, 1).

    Not in xsmccc/llaisys (its generate() accepts top_k, top_p and temperature and
    ignores them, python/llaisys/models/qwen2.py:212-219).  Order: top_k == 1 or
    temperature == 0 is the arg-max; otherwise p = softmax(logits / temperature);
    keep the top_k most probable (ties by lower index; 0 or >= vocab keeps all);
    of these, in descending order, keep the shortest prefix whose mass reaches
    top_p times the kept mass; draw by inverse CDF over the kept tokens in index order."""
    logits = np.asarray(logits, dtype=np.float64)
    V = logits.shape[0]
    if top_k == 1 or temperature == 0.0:
        return argmax(logits)
    z = logits / temperature
    p = np.exp(z - z.max())
    p /= p.sum()
    order = np.argsort(-p, kind="stable")
    keep = np.zeros(V, dtype=bool)
    k = V if (top_k <= 0 or top_k >= V) else top_k
    cand = order[:k]
    if top_p < 1.0:
        csum = np.cumsum(p[cand])
        before = csum - p[cand]
        cand = cand[before < top_p * csum[-1]]
    keep[cand] = True
    kept = np.where(keep, p, 0.0)
    cdf = np.cumsum(kept)
    idx = int(np.searchsorted(cdf, u * cdf[-1], side="right"))
    return min(idx, int(np.nonzero(keep)[0][-1]))


def generate_greedy(prompt, config, w, max_new_tokens, stop_ids=()):
    """Greedy continuation by re-running the whole sequence for every token.  The loop
    of python/llaisys/models/qwen2.py:234-283, except that the stop test also applies
    to the first generated token."""
    ids = list(prompt)
    new = []
    for _ in range(max_new_tokens):
        nxt = argmax(forward_logits(ids, config, w)[-1])
        ids.append(nxt)
        new.append(nxt)
        if nxt in stop_ids:
            break
    return new
