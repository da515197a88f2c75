"""Each part of a layer alone, against the plain function of the same part.  (Parts that are not in
the package, and a whole architecture made of them, are in test_gpu_toy_arch.py.)"""
import math

import numpy as np
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _env(dtype):
    from llaisys_b200.parts import BuildEnv
    return BuildEnv(dtype, DEV)


def _ctx(cache, slots, n_new, tokens=None, want=()):
    from llaisys_b200.engine import StepContext
    for s, n in zip(slots, n_new):
        cache.book.reserve(s, n)
    tokens = tokens if tokens is not None else [0] * sum(n_new)
    shape = StepContext.shape_of(cache, slots, n_new, list(want), bucket=False)
    ctx = StepContext(cache, DEV, *shape, torch.zeros(1, dtype=torch.int32, device=DEV))
    ctx.load(slots, n_new, tokens, list(want))
    return ctx


def _commit(cache, slots, n_new):
    for s, n in zip(slots, n_new):
        cache.book.commit(s, n)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    norm = build_part("norm", PartSpec("rms_norm", {"size": 50, "eps": 1e-3}, prefix="n"), _env(dtype))
    assert {k: v.shape for k, v in norm.tensors().items()} == {"weight": (50,)}
    rng = np.random.default_rng(0)
    w, x, d = 1 + rng.normal(size=50) * 0.1, rng.normal(size=(4, 50)), rng.normal(size=(4, 50))
    norm.load({"weight": torch.from_numpy(w).to(dtype).to(DEV)})
    res = torch.from_numpy(x).float().to(DEV)
    out = norm.forward(res, torch.from_numpy(d).to(dtype).to(DEV))
    wr, dr = (torch.from_numpy(a).to(dtype).double().numpy() for a in (w, d))
    want = plain.rms_norm(torch.from_numpy(x).float().double().numpy() + dr, wr, 1e-3)
    assert out.dtype == dtype and np.abs(out.double().cpu().numpy() - want).max() < (1e-5 if dtype == torch.float32 else 0.03)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    ffn = build_part("ffn", PartSpec("swiglu_mlp", {"hidden_size": 40, "intermediate_size": 56}, prefix="f"), _env(dtype))
    rng = np.random.default_rng(1)
    ws = {n: rng.normal(size=d.shape) * 0.3 for n, d in ffn.tensors().items()}
    ffn.load({n: torch.from_numpy(w).to(dtype).to(DEV) for n, w in ws.items()})
    x = rng.normal(size=(9, 40))
    got = ffn.forward(torch.from_numpy(x).to(dtype).to(DEV), None)
    r = {n: torch.from_numpy(w).to(dtype).double().numpy() for n, w in ws.items()}
    xr = torch.from_numpy(x).to(dtype).double().numpy()
    want = plain.linear(plain.swiglu(plain.linear(xr, r["gate_proj.weight"]), plain.linear(xr, r["up_proj.weight"])),
                        r["down_proj.weight"])
    assert np.abs(got.double().cpu().numpy() - want).max() < (1e-4 if dtype == torch.float32 else 0.15)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 6])
def test_attention_part_prefill_then_decode(dtype, window):
    """The mixer alone over its own cache: 70 tokens at once, then 5 one by one, against the
    plain attention block over the whole 75."""
    from llaisys_b200.cache import CacheConfig, PagedCache
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    H, nh, nkvh, dh, theta = 48, 6, 3, 8, 3000.0
    spec = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkvh, "head_dim": dh,
                                      "qkv_bias": True, "scale": 1 / math.sqrt(dh), "window": window,
                                      "position": PartSpec("rope_half_split", {"head_dim": dh, "theta": theta})}, prefix="a")
    att = build_part("mixer", spec, _env(dtype))
    rng = np.random.default_rng(2)
    # sharp scores under float32; milder under bfloat16, where a score's rounding error grows with its size
    qk = 0.6 if dtype == torch.float32 else 0.15
    ws = {n: rng.normal(size=d.shape) * (qk if "q_proj" in n or "k_proj" in n else 0.2) for n, d in att.tensors().items()}
    att.load({n: torch.from_numpy(w).to(dtype).to(DEV) for n, w in ws.items()})
    cache = PagedCache([att.kv_need()], [None], [0], CacheConfig(max_tokens=128), dtype, DEV)
    x = rng.normal(size=(75, H))
    xt = torch.from_numpy(x).to(dtype).to(DEV)
    slot = cache.acquire()
    ctx = _ctx(cache, [slot], [70])
    outs = [att.forward(xt[:70], ctx, 0)]
    _commit(cache, [slot], [70])
    for t in range(70, 75):
        ctx = _ctx(cache, [slot], [1])
        outs.append(att.forward(xt[t:t + 1], ctx, 0))
        _commit(cache, [slot], [1])
    got = torch.cat(outs).double().cpu().numpy()
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkvh, "head_dim": dh, "hidden_size": H, "rope_theta": theta}
    r = {"a." + n: torch.from_numpy(w).to(dtype).double().numpy() for n, w in ws.items()}
    want = plain.attention_block(torch.from_numpy(x).to(dtype).double().numpy(), np.arange(75), cfg, r, "a.", window)
    # bfloat16: four roundings on the way (projections, rotation, attention output, output projection)
    bound = 2e-5 if dtype == torch.float32 else 8 * 2.0 ** -9 * 2 * float(np.sqrt(np.mean(want ** 2)))
    assert np.abs(got - want).max() < bound


def test_rope_part_table_grows():
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import build_part
    rope = build_part("position", PartSpec("rope_half_split", {"head_dim": 16, "theta": 1e4}), _env(torch.float32))
    c1, _ = rope.table(10)
    c2, s2 = rope.table(500)
    assert c2.shape[0] >= 500 and torch.equal(c2[:10], c1[:10])
    j = np.arange(8)
    ang = 499 / np.power(1e4, 2 * j / 16)
    assert np.abs(c2[499].double().cpu().numpy() - np.cos(ang)).max() < 1e-7
    assert np.abs(s2[499].double().cpu().numpy() - np.sin(ang)).max() < 1e-7
