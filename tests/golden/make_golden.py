#!/usr/bin/env python3
"""Makes tests/golden/tiny_a_reference.json and tiny_b_reference.json from xsmccc/llaisys' own CPU code.

    python tests/golden/make_golden.py /path/to/llaisys-checkout

It copies the checkout to a temporary folder, compiles its C++ sources with g++ into
libllaisys.so (the project builds with xmake, which this does in its place), writes a
tiny random Qwen2 folder per case, and records

  * the greedy tokens of `llaisys.models.Qwen2(dir).generate(prompt, 8)` (that model knows no
    sliding window, so for case B these are the tokens of the same model without a window), and
  * the logits of one prompt, obtained by composing that project's own operators
    (`llaisys.Ops`) in the order of its model code, since its model API returns token ids only.

Case A is the first tiny configuration's shape (theta 1e4, eps 1e-6, head size 16, 9 tokens).
Case B is the second one's (three layers, 6 query heads on 2 key/value heads, head size 24,
theta 1e6, eps 1e-5, an untied head, a window of 8 keys from layer 1 on, 21 tokens).  That
project has no window; in a windowed layer its own self_attention is called once per query row
with the keys and values sliced to the row's window (Tensor.slice, zero-copy): with one query
and no more keys than the window its causal mask admits every key
(src/ops/self_attention/cpu/self_attention_cpu.cpp:66-75), so the softmax over exactly those
keys is that project's arithmetic.

The committed JSON files hold the configuration, the seed, the prompt and these outputs;
tests/test_plain.py rebuilds the same weights and compares the plain implementation
with them.  The model folders have an explicit lm_head.weight because that code has no
tied-head path.
"""
import ctypes
import glob
import json
import os
import shutil
import struct
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

CONFIG_A = {
    "architectures": ["Qwen2ForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "intermediate_size": 160, "vocab_size": 256,
    "max_position_embeddings": 128, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
    "tie_word_embeddings": False, "eos_token_id": 255,
}
CONFIG_B = {
    "architectures": ["Qwen2ForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 144, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 24, "intermediate_size": 232, "vocab_size": 384,
    "max_position_embeddings": 256, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 8, "max_window_layers": 1,
    "eos_token_id": 383,
}
# name -> (config, seed, prompt, gain on the query and key projections: case B's scores are spread out so
# that the window's edge shows in the logits)
CASES = {
    "tiny_a": (CONFIG_A, 0, [17, 201, 5, 99, 42, 7, 130, 64, 250], 1.0),
    "tiny_b": (CONFIG_B, 1, [311, 4, 77, 150, 9, 263, 88, 301, 12, 45, 199, 230, 6, 371, 54, 120, 33, 280, 91, 2, 160], 12.0),
}


def tiny_weights(config, seed, gain=1.0):
    """float32 weights: matrices N(0, 0.02), norm weights 1 + N(0, 0.02), biases N(0, 0.02),
    drawn in sorted-name order from numpy's default_rng(seed); the query and key projections
    (weights and biases) are then multiplied by `gain`."""
    L, H = config["num_hidden_layers"], config["hidden_size"]
    nh, nkvh = config["num_attention_heads"], config["num_key_value_heads"]
    dh, I, V = H // nh, config["intermediate_size"], config["vocab_size"]
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,), "lm_head.weight": (V, H)}
    for l in range(L):
        p = f"model.layers.{l}."
        shapes.update({
            p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
            p + "self_attn.q_proj.weight": (nh * dh, H), p + "self_attn.q_proj.bias": (nh * dh,),
            p + "self_attn.k_proj.weight": (nkvh * dh, H), p + "self_attn.k_proj.bias": (nkvh * dh,),
            p + "self_attn.v_proj.weight": (nkvh * dh, H), p + "self_attn.v_proj.bias": (nkvh * dh,),
            p + "self_attn.o_proj.weight": (H, nh * dh),
            p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H),
            p + "mlp.down_proj.weight": (H, I),
        })
    rng = np.random.default_rng(seed)
    out = {}
    for name in sorted(shapes):
        x = rng.normal(0.0, 0.02, size=shapes[name]).astype(np.float32)
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            x = (1.0 + x).astype(np.float32)
        if ".q_proj." in name or ".k_proj." in name:
            x = (x * np.float32(gain)).astype(np.float32)
        out[name] = x
    return out


def write_safetensors(path, tensors):
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        b = np.ascontiguousarray(arr.astype("<f4")).tobytes()
        header[name] = {"dtype": "F32", "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def build_reference(src: Path, work: Path) -> Path:
    ref = work / "ref"
    shutil.copytree(src, ref, ignore=shutil.ignore_patterns(".git"))
    srcs = []
    for pat in ["src/utils/*.cpp", "src/device/*.cpp", "src/device/cpu/*.cpp", "src/core/*/*.cpp",
                "src/tensor/*.cpp", "src/ops/*/*.cpp", "src/ops/*/cpu/*.cpp", "src/llaisys/*.cc",
                "src/models/qwen2/*.cpp"]:
        srcs += sorted(glob.glob(str(ref / pat)))
    out = ref / "python/llaisys/libllaisys/libllaisys.so"
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", f"-I{ref / 'include'}",
                           *srcs, "-o", str(out)])
    return ref / "python"


def layer_window(config, layer):
    if not config.get("use_sliding_window", False) or layer < config.get("max_window_layers", config["num_hidden_layers"]):
        return None
    return int(config["sliding_window"])


def run_case(llaisys, work: Path, name: str):
    from llaisys import DataType, DeviceType, Ops, Tensor
    CONFIG, SEED, PROMPT, GAIN = CASES[name]
    weights = tiny_weights(CONFIG, SEED, GAIN)
    folder = work / name
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(CONFIG))
    write_safetensors(folder / "model.safetensors", weights)

    model = llaisys.models.Qwen2(str(folder), DeviceType.CPU)
    generated = [int(t) for t in model.generate(PROMPT, max_new_tokens=8, top_k=1)]

    # ---- logits by composing the project's operators in its model's order
    keep = []

    def T(arr, dtype=DataType.F32):
        arr = np.ascontiguousarray(arr)
        t = Tensor(arr.shape, dtype, DeviceType.CPU)
        t.load(ctypes.c_void_p(arr.ctypes.data))
        keep.append(arr)
        return t

    def new(*shape):
        return Tensor(shape, DataType.F32, DeviceType.CPU)

    def read(t):
        n = int(np.prod(t.shape()))
        buf = (ctypes.c_float * n).from_address(t.data_ptr())
        return np.array(buf, dtype=np.float32).reshape(t.shape())

    def lin(x, name, bias_name=None):
        W = weights[name]
        b = weights[bias_name] if bias_name else np.zeros(W.shape[0], np.float32)
        out = new(x.shape()[0], W.shape[0])
        Ops.linear(out, x, T(W), T(b))
        return out

    L, H = CONFIG["num_hidden_layers"], CONFIG["hidden_size"]
    nh, nkvh = CONFIG["num_attention_heads"], CONFIG["num_key_value_heads"]
    dh, n = H // nh, len(PROMPT)
    eps, theta = CONFIG["rms_norm_eps"], CONFIG["rope_theta"]
    scale = 1.0 / float(np.sqrt(np.float32(dh)))
    ids = T(np.array(PROMPT, np.int64), DataType.I64)
    pos = T(np.arange(n, dtype=np.int64), DataType.I64)
    x = new(n, H)
    Ops.embedding(x, ids, T(weights["model.embed_tokens.weight"]))
    for l in range(L):
        p = f"model.layers.{l}."
        h = new(n, H)
        Ops.rms_norm(h, x, T(weights[p + "input_layernorm.weight"]), eps)
        q = lin(h, p + "self_attn.q_proj.weight", p + "self_attn.q_proj.bias").view(n, nh, dh)
        k = lin(h, p + "self_attn.k_proj.weight", p + "self_attn.k_proj.bias").view(n, nkvh, dh)
        v = lin(h, p + "self_attn.v_proj.weight", p + "self_attn.v_proj.bias").view(n, nkvh, dh)
        qr, kr = new(n, nh, dh), new(n, nkvh, dh)
        Ops.rope(qr, q, pos, theta)
        Ops.rope(kr, k, pos, theta)
        a = new(n, nh, dh)
        W = layer_window(CONFIG, l)
        if W is None:
            Ops.self_attention(a, qr, kr, v, scale)
        else:
            # one call per query row over the keys and values of its window, sliced without a copy
            for i in range(n):
                lo = max(0, i - W + 1)
                Ops.self_attention(a.slice(0, i, i + 1), qr.slice(0, i, i + 1), kr.slice(0, lo, i + 1), v.slice(0, lo, i + 1), scale)
        o = lin(a.view(n, H), p + "self_attn.o_proj.weight")
        x1 = new(n, H)
        Ops.add(x1, o, x)
        h = new(n, H)
        Ops.rms_norm(h, x1, T(weights[p + "post_attention_layernorm.weight"]), eps)
        g = lin(h, p + "mlp.gate_proj.weight")
        u = lin(h, p + "mlp.up_proj.weight")
        s = new(n, CONFIG["intermediate_size"])
        Ops.swiglu(s, g, u)
        d = lin(s, p + "mlp.down_proj.weight")
        x = new(n, H)
        Ops.add(x, d, x1)
    h = new(n, H)
    Ops.rms_norm(h, x, T(weights["model.norm.weight"]), eps)
    logits = read(lin(h, "lm_head.weight"))

    out = {
        "source": "xsmccc/llaisys CPU code compiled with g++ -O2 (see make_golden.py)",
        "config": CONFIG, "seed": SEED, "gain": GAIN, "prompt": PROMPT,
        "generated": generated,
        "generated_note": "tokens of that project's model, which applies no sliding window",
        "logits_shape": list(logits.shape),
        "logits": [float(f"{v:.9g}") for v in logits.reshape(-1)],
    }
    dst = Path(__file__).with_name(f"{name}_reference.json")
    dst.write_text(json.dumps(out))
    print("wrote", dst, "generated:", generated, "max|logit|", float(np.abs(logits).max()))


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of xsmccc/llaisys>")
    src = Path(sys.argv[1])
    with tempfile.TemporaryDirectory() as tmp:
        work = Path(tmp)
        sys.path.insert(0, str(build_reference(src, work)))
        import llaisys
        for name in CASES:
            run_case(llaisys, work, name)


if __name__ == "__main__":
    main()
