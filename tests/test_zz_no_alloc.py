"""The allocation-free entry point of the tensor-core matrix product (csrc/gemm_tc_noalloc.h),
called through its exported C symbol and compared with the regular entry point.

This file sorts last on purpose: a run that stops at the first failure has then run every other test.
"""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOO_LARGE = -3001


def _entry():
    from llaisys_b200.csrc.build import load_module
    f = load_module("gemm_tc.cu").llb_gemm_tc_noalloc
    f.restype = c_int
    f.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    return f


def _status():
    from llaisys_b200.csrc.build import load_module
    f = load_module("gemm_tc.cu").llb_gemm_tc_noalloc_status
    f.restype, f.argtypes = c_int, [c_void_p]
    return f(torch.cuda.current_stream().cuda_stream)


def _call(f, x, w, bias, out, bn, splits):
    return f(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None, 1, out.data_ptr(),
             0 if out.dtype == torch.float32 else 1, x.shape[0], w.shape[0], x.shape[1], x.stride(0), out.stride(0),
             bn, splits, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("T,N,K,bn,splits", [(8, 1536, 1536, 16, 6), (5, 200, 712, 16, 3), (40, 300, 1000, 64, 4), (8, 1536, 8960, 16, 12)])
def test_same_result_as_the_regular_entry_point_twice_in_a_row(T, N, K, bn, splits):
    from llaisys_b200 import kernels
    f = _entry()
    g = torch.Generator(device="cpu").manual_seed(T + N + K)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    want = kernels.linear(x, w, b, out_dtype=torch.float32, plan=(bn, splits)).clone()
    import plain_qwen2 as plain
    exact = torch.from_numpy(plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy(), b.double().cpu().numpy())).to(DEV)
    for call in range(2):                     # the second call meets the scratch and the counters the first one left
        out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
        torch.cuda.synchronize()
        before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(DEV)
        assert _call(f, x, w, b, out, bn, splits) == 0
        torch.cuda.synchronize()
        if call == 1:                         # (the first call may load the kernel's code onto the device)
            assert (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(DEV)) == before, "the call took device memory"
        # both entry points run the same kernel with the same split of the reduction: the tolerance is that of
        # the kernel tests (float32 accumulation of bfloat16 products), and in fact the results are identical
        err = (out - want).abs()
        bound = 5e-4 * (K / 64) ** 0.5 + 2e-3 * want.abs()
        assert torch.isfinite(out).all() and bool((err <= bound).all()), f"call {call}: max error {float(err.max())}"
        # and against the plain product, which shares nothing with either entry point
        err = (out.double() - exact).abs()
        assert bool((err <= 5e-4 * (K / 64) ** 0.5 + 2e-3 * exact.abs()).all()), f"call {call}: {float(err.max())} from the plain product"
        assert _status() == 0                 # no block gave up a wait
    out_bf = torch.empty((T, N), dtype=torch.bfloat16, device=DEV)
    assert _call(f, x, w, None, out_bf, bn, 1) == 0                  # no bias, bfloat16 out, no split
    ref = kernels.linear(x, w)
    torch.cuda.synchronize()
    assert float((out_bf.float() - ref.float()).abs().max()) <= 2.0 ** -7 * float(ref.float().abs().max()) + 1e-3


def test_sizes_beyond_the_built_in_scratch_are_refused():
    f = _entry()
    x = torch.zeros(256, 1536, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(17920, 1536, dtype=torch.bfloat16, device=DEV)
    out = torch.full((256, 17920), 7.0, dtype=torch.float32, device=DEV)
    assert _call(f, x, w, None, out, 256, 8) == TOO_LARGE            # 140 tiles * 8 splits * 256 * 128 floats > 4 MiB
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0                                   # nothing was launched
    assert _call(f, x, w, None, out, 100, 1) != 0                    # a tile size the kernel does not have
    assert _status() == 0
