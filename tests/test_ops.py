"""The op-level interface `llaisys_b200.ops.Ops` at the shapes and tolerances of xsmccc/llaisys' own
op tests (test/ops/add.py:48-54, argmax.py:49-50, embedding.py:45-54, linear.py:55-64,
rms_norm.py:54-60, rope.py:69-77, self_attention.py:70-80, swiglu.py:48-54), against the plain
float64 functions of plain_qwen2: on the CPU (the package's numpy operators) without a device,
and on the GPU (the package's kernels) under -m gpu.  A few more shapes exercise the tensor-core
kernels, which those tests' sizes do not reach."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from llaisys_b200.ops import Ops

DTYPES = [(torch.float32, 1e-5, 1e-5), (torch.float16, 1e-3, 1e-3), (torch.bfloat16, 1e-2, 1e-2)]
DEVICES = ["cpu", pytest.param("cuda:0", marks=pytest.mark.gpu)]


def _rand(shape, dtype, dev, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    t = (torch.rand(shape, generator=g) * scale).to(dtype)
    return t.to(dev), t.double().numpy()


def _close(got: torch.Tensor, want: np.ndarray, atol, rtol):
    g = got.double().cpu().numpy()
    assert g.shape == want.shape
    bad = np.abs(g - want) > atol + rtol * np.abs(want)
    assert not bad.any(), f"{int(bad.sum())} of {bad.size} elements differ; worst {np.abs(g - want).max():.3e}"


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("dtype,atol,rtol", [(torch.float32, 1e-5, 1e-5), (torch.float16, 1e-3, 1e-3), (torch.bfloat16, 1e-3, 1e-3)])
@pytest.mark.parametrize("shape", [(2, 3), (512, 4096)])
def test_add(dev, dtype, atol, rtol, shape):
    a, ar = _rand(shape, dtype, dev, 1)
    b, br = _rand(shape, dtype, dev, 2)
    c = torch.zeros(shape, dtype=dtype, device=dev)
    Ops.add(c, a, b)
    # the sum of two 16-bit values is rounded once: half a unit in the last place of the result
    want = (torch.from_numpy(ar + br)).to(dtype).double().numpy()
    _close(c, want, atol, rtol)


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n", [4, 4096])
def test_argmax(dev, dtype, n):
    vals, ref = _rand((n,), dtype, dev, 3)
    vals[n // 2] = vals.max()                          # a tie: the first maximum wins
    ref = vals.double().cpu().numpy()
    idx = torch.zeros(1, dtype=torch.int64, device=dev)
    val = torch.zeros(1, dtype=dtype, device=dev)
    Ops.argmax(idx, val, vals)
    assert int(idx) == plain.argmax(ref) and float(val) == float(ref.max())


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n_idx,table", [(1, (2, 3)), (50, (512, 4096))])
def test_embedding(dev, dtype, n_idx, table):
    w, wr = _rand(table, dtype, dev, 4)
    index = torch.randint(0, table[0], (n_idx,), generator=torch.Generator().manual_seed(5)).to(dev)
    out = torch.zeros((n_idx, table[1]), dtype=dtype, device=dev)
    Ops.embedding(out, index, w)
    assert np.array_equal(out.double().cpu().numpy(), plain.embedding(index.cpu().numpy(), wr))
    with pytest.raises(IndexError):
        Ops.embedding(out, torch.full((n_idx,), table[0], dtype=torch.int64, device=dev), w)


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("dtype,atol,rtol", DTYPES)
@pytest.mark.parametrize("out_shape,x_shape,w_shape,bias", [((2, 3), (2, 4), (3, 4), True), ((512, 4096), (512, 4096), (4096, 4096), True),
                                                           ((7, 40), (7, 24), (40, 24), False)])
def test_linear(dev, dtype, atol, rtol, out_shape, x_shape, w_shape, bias):
    # the reference's tests draw operands from [0, 1) too; scaled so that sums over 4096 terms stay near 1
    s = (1.0 / x_shape[1]) ** 0.5
    x, xr = _rand(x_shape, dtype, dev, 6, 2 * s)
    w, wr = _rand(w_shape, dtype, dev, 7, 2 * s)
    b, br = _rand((w_shape[0],), dtype, dev, 8) if bias else (None, None)
    out = torch.zeros(out_shape, dtype=dtype, device=dev)
    Ops.linear(out, x, w, b)
    _close(out, plain.linear(xr, wr, br), atol, rtol)


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("dtype,atol,rtol", DTYPES)
@pytest.mark.parametrize("shape", [(1, 4), (512, 4096)])
def test_rms_norm(dev, dtype, atol, rtol, shape):
    x, xr = _rand(shape, dtype, dev, 9)
    w, wr = _rand((shape[1],), dtype, dev, 10)
    out = torch.zeros(shape, dtype=dtype, device=dev)
    Ops.rms_norm(out, x, w, 1e-5)
    _close(out, plain.rms_norm(xr, wr, 1e-5), atol, rtol)


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("dtype,atol,rtol", [(torch.float32, 1e-4, 1e-4), (torch.float16, 1e-3, 1e-3), (torch.bfloat16, 1e-2, 1e-2)])
@pytest.mark.parametrize("shape,span", [((2, 1, 4), (0, 2)), ((512, 4, 4096), (512, 1024)), ((9, 3, 48), (100, 109))])
def test_rope(dev, dtype, atol, rtol, shape, span):
    x, xr = _rand(shape, dtype, dev, 11)
    pos = torch.arange(span[0], span[1], dtype=torch.int64, device=dev)
    out = torch.zeros(shape, dtype=dtype, device=dev)
    Ops.rope(out, x, pos, 10000.0)
    _close(out, plain.rope(xr, np.arange(*span), 10000.0), atol, rtol)


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("dtype,atol,rtol", DTYPES)
@pytest.mark.parametrize("qlen,kvlen,nh,nkvh,hd", [(2, 2, 1, 1, 4), (5, 11, 4, 2, 8), (1, 200, 6, 2, 64), (150, 330, 4, 1, 128)])
def test_self_attention(dev, dtype, atol, rtol, qlen, kvlen, nh, nkvh, hd):
    q, qr = _rand((qlen, nh, hd), dtype, dev, 12)
    k, kr = _rand((kvlen, nkvh, hd), dtype, dev, 13)
    v, vr = _rand((kvlen, nkvh, hd), dtype, dev, 14)
    out = torch.zeros((qlen, nh, hd), dtype=dtype, device=dev)
    Ops.self_attention(out, q, k, v, hd ** -0.5)
    _close(out, plain.self_attention(qr, kr, vr, hd ** -0.5), atol, rtol)


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("dtype,atol,rtol", DTYPES)
@pytest.mark.parametrize("shape", [(2, 3), (512, 4096)])
def test_swiglu(dev, dtype, atol, rtol, shape):
    g, gr = _rand(shape, dtype, dev, 15)
    u, ur = _rand(shape, dtype, dev, 16)
    out = torch.zeros(shape, dtype=dtype, device=dev)
    Ops.swiglu(out, g, u)
    _close(out, plain.swiglu(gr, ur), atol, rtol)


@pytest.mark.parametrize("dev", DEVICES)
def test_rearrange_and_mixed_devices(dev):
    src = torch.arange(24, dtype=torch.float32, device=dev).view(2, 3, 4)
    out = torch.zeros((4, 3, 2), dtype=torch.float32, device=dev).permute(2, 1, 0)       # another stride order
    Ops.rearrange(out, src)
    assert torch.equal(out, src) and not out.is_contiguous()
    if dev != "cpu":
        with pytest.raises(ValueError, match="one device"):
            Ops.add(torch.zeros(2, device=dev), torch.zeros(2), torch.zeros(2, device=dev))
