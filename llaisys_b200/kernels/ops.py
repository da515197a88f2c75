from __future__ import annotations

import ctypes
import functools
from ctypes import c_double, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from ..csrc.build import load_module, page_tokens
from .. import diagnostics
from ..diagnostics import timers

PAGE = page_tokens()           # tokens of a cache page (LLB_PAGE in csrc/common.cuh)
DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    try:
        return DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    # the raw handle of torch's current stream on the current device, without the Python layers in between
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels of llaisys_b200 run on a CUDA device only; got a CPU tensor")


_basic = None


def _lib_basic():
    global _basic
    if _basic is None:
        _basic = load_module("basic.cu")
        _basic.llb_error_string.restype = ctypes.c_char_p
        _basic.llb_error_string.argtypes = [c_int]
    return _basic


_launches = 0

# LLAISYS_STAMPS=1: the kernels that can record cycle stamps (see csrc/common.cuh: the decode step's three short ones and
# the paired-SM product) are built with them; set_stamps() then switches them on for launches of a given grid size.  Off by default: the product's
# builds contain no stamp.
_STAMPS = {"LLB_STAMPS": 1} if __import__("os").environ.get("LLAISYS_STAMPS", "0") not in ("", "0") else {}
_stamp_libs = {}


def _stamped(source: str, defines: Optional[dict] = None):
    lib = load_module(source, {**(defines or {}), **_STAMPS} or None)
    if _STAMPS:
        _stamp_libs[source] = lib
    return lib


def set_stamps(source: str, buf: Optional[torch.Tensor], blocks: int = 0) -> None:
    """Cycle stamps of the kernels of `source` ("gemm_tc.cu", "gemm_tc2.cu", "attention_mma.cu", "mlp_tc.cu") into `buf` (int64
    [blocks, 16] on the device) for launches of exactly `blocks` blocks; None switches them off.  Needs
    LLAISYS_STAMPS=1 in the environment before the package is imported, and the module in use already."""
    lib = _stamp_libs.get(source)
    if lib is None:
        raise KernelError(f"no stamped build of {source} is loaded (LLAISYS_STAMPS=1, and run a step first)")
    lib.llb_set_stamps.argtypes = [c_void_p, ctypes.c_uint]
    lib.llb_set_stamps.restype = c_int
    rc = lib.llb_set_stamps(_ptr(buf), blocks)
    if rc:
        raise KernelError(f"llb_set_stamps: CUDA error {rc}")


def launch_count() -> int:
    """Kernels of this package launched so far by this process (a captured launch counts once,
    at capture; replays are counted by whoever replays)."""
    return _launches


def _check(rc: int, what: str, n: int = 1):
    global _launches
    _launches += n
    if timers.enabled:
        timers.mark(what)
    if rc <= -2000:
        raise KernelError(f"{what}: the kernel's shared-memory size was refused (CUDA error {-rc - 2000})")
    if rc <= -1000:
        raise KernelError(f"{what}: a tensor map could not be encoded (driver error {-rc - 1000})")
    if rc != 0:
        msg = _lib_basic().llb_error_string(rc)
        raise KernelError(f"{what}: CUDA error {rc} ({msg.decode() if msg else '?'})")


_configured = set()


def _fn(lib, name, argtypes):
    f = getattr(lib, name)
    if (id(lib), name) not in _configured:
        f.argtypes = argtypes
        f.restype = c_int
        _configured.add((id(lib), name))
    return f


# ------------------------------------------------------------------ row-wise kernels
def embedding(ids: torch.Tensor, table: torch.Tensor, err: torch.Tensor) -> torch.Tensor:
    """float32 [T, H] rows of `table` (float32 or bfloat16) for int32 `ids`; an id outside the
    table sets err[0] = 1 and yields a zero row."""
    _need_cuda(ids, table)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    f = _fn(_lib_basic(), "llb_embedding", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(out), _ptr(table), _dt(table), _ptr(ids), T, H, V, _ptr(err), _stream()), "embedding")
    return out


def gather_i32(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor):
    """dst[i] = src[idx[i]] (int32, on the device)."""
    _need_cuda(dst, src, idx)
    assert dst.dtype == src.dtype == idx.dtype == torch.int32 and dst.numel() == idx.numel()
    f = _fn(_lib_basic(), "llb_gather_i32", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(dst), _ptr(src), _ptr(idx), idx.numel(), _stream()), "gather_i32")


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, src: torch.Tensor):
    """dst[idx[i]] = src[i] (int32, on the device; idx without repeats)."""
    _need_cuda(dst, src, idx)
    assert dst.dtype == src.dtype == idx.dtype == torch.int32 and src.numel() == idx.numel()
    f = _fn(_lib_basic(), "llb_scatter_i32", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(dst), _ptr(idx), _ptr(src), idx.numel(), _stream()), "scatter_i32")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, want_out: bool = True):
    """residual (float32 [T, H]) += delta, then out = residual * weight / sqrt(mean(residual^2) + eps).

    delta is [T, H] or [parts, T, H] (partial sums, added in order).  With `rows` (int32) only those
    rows are normalised, into an [len(rows), H] output, and the residual is left as it was."""
    _need_cuda(residual, delta, weight, rows)
    T, H = residual.shape
    n_part, stride = 1, 0
    if delta is not None:
        if delta.dim() == 3:
            n_part, stride = delta.shape[0], delta.stride(0)
        assert delta.shape[-2:] == residual.shape and delta.is_contiguous()
    R = T if rows is None else rows.numel()
    out = torch.empty((R, H), dtype=out_dtype, device=residual.device) if want_out else None
    f = _fn(_lib_basic(), "llb_add_rmsnorm", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_int,
                                              c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), _dt(delta) if delta is not None else 0, n_part, stride,
             _ptr(weight), _dt(weight), _ptr(out), DT[out_dtype], _ptr(rows), R, H, eps,
             0 if rows is not None else 1, _stream()), "add_rmsnorm")
    return out


def residual_add(residual: torch.Tensor, delta: torch.Tensor):
    _need_cuda(residual, delta)
    n_part, stride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
    f = _fn(_lib_basic(), "llb_residual_add", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_void_p])
    _check(f(_ptr(residual), _ptr(delta), _dt(delta), n_part, stride, residual.numel(), _stream()), "residual_add")


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] (gate columns first) -> [T, I]: up * gate / (1 + exp(-gate))."""
    _need_cuda(gate_up)
    T, I2 = gate_up.shape
    out = torch.empty((T, I2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn(_lib_basic(), "llb_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(gate_up), _dt(gate_up), T, I2 // 2, _stream()), "swiglu")
    return out


def dense_binary(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, op: str):
    """out = a + b (op "add") or out = b * a / (1 + exp(-a)) (op "swiglu": a the gate, b the up
    projection) on contiguous tensors of one dtype and one shape."""
    _need_cuda(out, a, b)
    assert out.dtype == a.dtype == b.dtype and out.shape == a.shape == b.shape
    assert out.is_contiguous() and a.is_contiguous() and b.is_contiguous()
    f = _fn(_lib_basic(), "llb_dense_binary", [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(a), _ptr(b), _dt(out), out.numel(), {"add": 0, "swiglu": 1}[op], _stream()), op)


def rope_append(qkv: torch.Tensor, nh: int, nkvh: int, dh: int, *, cos=None, sin=None, tok_pos=None,
                append=None, err=None):
    """In place on the packed projections [T, (nh + 2 nkvh) dh]: rotate the query and key heads
    (when cos/sin tables are given) and/or write keys and values to the paged cache.

    append = dict(tok_seq, seq_start, seq_len_before, kpool, vpool, page_table, ring)."""
    _need_cuda(qkv, tok_pos)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1
    if tok_pos is None or tok_pos.numel() != T or err is None:
        raise KernelError("rope_append needs tok_pos (one position per packed token) and an error word")
    do_rope, do_app = cos is not None, append is not None
    a = append or {}
    pt = a.get("page_table")
    f = _fn(_lib_basic(), "llb_rope_append",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
             c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(qkv), _dt(qkv), T, qkv.stride(0), nh, nkvh, dh, int(do_rope), _ptr(cos), _ptr(sin),
             cos.shape[0] if do_rope else 0, _ptr(tok_pos), int(do_app), _ptr(a.get("tok_seq")),
             _ptr(a.get("seq_start")), _ptr(a.get("seq_len_before")), _ptr(a.get("kpool")), _ptr(a.get("vpool")),
             _ptr(pt), pt.shape[1] if do_app else 0, a.get("ring", 1), _ptr(err), _stream()), "rope_append")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float, first: int = 0):
    """out (contiguous, float32 or bfloat16) <- mean + std * z(key, first + i): the counter-based
    normal numbers of csrc/random_init.cu, whose host twin is weights/rng.py."""
    _need_cuda(out)
    assert out.is_contiguous()
    f = _fn(load_module("random_init.cu"), "llb_fill_normal",
            [c_void_p, c_int, c_longlong, c_longlong, c_ulonglong, c_double, c_double, c_void_p])
    with torch.cuda.device(out.device):
        _check(f(_ptr(out), _dt(out), out.numel(), first, key & 0xFFFFFFFFFFFFFFFF, mean, std, _stream()), "fill_normal")


# ------------------------------------------------------------------ matrix products
_TC_SCRATCH_ELEMS = 16 * 1024 * 1024        # float32 partial tiles of split-K launches (64 MB)
_TC_COUNTERS = 1 << 16
_tc_res = {}
TC_ENABLED = True                            # tests switch the tensor-core path off to compare


def _tc_resources(device):
    """Per device: the scratch of split-K partial tiles, the tile counters (zero between
    launches) and the error word of the tensor-core kernels.  Allocated once, so launches inside
    a CUDA graph capture allocate nothing."""
    device = _dev_key(device)
    r = _tc_res.get(device)
    if r is None:
        if diagnostics.CANARY:
            scratch, raw_s = diagnostics.guarded((_TC_SCRATCH_ELEMS,), torch.float32, device, fill_zero=False)
            counters, raw_c = diagnostics.guarded((_TC_COUNTERS,), torch.int32, device)
            _tc_guards[device] = [("tensor-core scratch", raw_s), ("tensor-core tile counters", raw_c)]
        else:
            scratch = torch.empty(_TC_SCRATCH_ELEMS, dtype=torch.float32, device=device)
            counters = torch.zeros(_TC_COUNTERS, dtype=torch.int32, device=device)
        r = (scratch, counters, torch.zeros(1, dtype=torch.int32, device=device))
        _tc_res[device] = r
    return r


_tc_guards = {}


def check_guards(device) -> None:
    """Raises KernelError if the guard words around the tensor-core scratch or counters of `device` were
    overwritten (they exist only under LLAISYS_CANARY=1)."""
    broken = [what for what, raw in _tc_guards.get(_dev_key(device), []) if not diagnostics.guards_intact(raw)]
    if broken:
        raise KernelError("guard words overwritten around: " + ", ".join(broken))


def _dev_key(device) -> torch.device:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def tc_error(device, clear: bool = True) -> int:
    """Error word of the tensor-core kernels on `device` (0: none; 101-104, 111-114, 121-122, 131-136, 141: a bounded
    wait ran out).  Reading it waits for the device; a code that was found is cleared, so that it is
    reported once."""
    r = _tc_res.get(_dev_key(device))
    if not r:
        return 0
    code = int(r[2].item())
    if code and clear:
        r[2].zero_()
    return code


_sm_counts = {}


def _sm_count(device) -> int:
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


_TC_STAGES = {False: {16: 5, 32: 4, 64: 4, 128: 6, 256: 4}, True: {16: 3, 32: 3, 64: 4, 128: 4, 256: 3}}


@functools.lru_cache(maxsize=4096)
def tc_plan(T: int, rows_out: int, K: int, sms: int, dual: bool = False):
    """(tokens per tile, K splits) of a tensor-core launch.

    The tile is the smallest that holds the tokens.  When the weight has fewer row blocks than
    the device can run CTAs (decode), K is split 2, 4, 8 or 16 ways over a thread-block cluster that
    reduces through shared memory.  The split minimises a cost fitted to measurements on a B200
    (microseconds): k-blocks per CTA times 0.0155 per KB of a pipeline stage, plus, when split,
    1.2 + 0.0015 * tile tokens * accumulators * splits for the cluster reduction; the CTAs must
    all be resident at once (two per SM while a CTA's shared memory stays under 113 KB; with one
    per SM, clusters of eight fill a GPC unevenly, so fewer CTAs are allowed)."""
    bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256
    tiles = -(-rows_out // 128) * -(-T // bn)
    kblocks = -(-K // 64)
    accs = 2 if dual else 1
    stage_kb = accs * 16 + bn / 8
    recv_kb = bn / 2 if bn <= 32 and not dual else 0          # the push reduction's receive buffer
    two_per_sm = stage_kb * _TC_STAGES[dual][bn] + recv_kb <= 112
    capacity = (sms * 2 * 280) // 296 if two_per_sm else (sms * 112) // 148
    best, best_cost = 1, kblocks * stage_kb * 0.0155
    if bn <= 128:
        # sixteen (a cluster of non-portable size) for 64-token tiles and for up to four tokens: measured in the
        # whole step, +2.7 % at batch 64, +1.5 % at batch 1 and 2, +4 % at batch 4, nothing at batch 6, but -1 % at
        # batch 8 and 32, although the product alone is faster there too
        for s in (2, 4, 8, 16):
            if s > kblocks // 2 or tiles * s > capacity or (s == 16 and bn != 64 and T > 4):
                break
            if (s - 1) * -(-kblocks // s) >= kblocks:      # a CTA of the cluster would be left without a k-block
                continue
            cost = -(-kblocks // s) * stage_kb * 0.0155 + 1.2 + 0.0015 * bn * accs * s
            if cost < best_cost:
                best, best_cost = s, cost
    return bn, best


def _tc_ok(x, weight, bias) -> bool:
    return (TC_ENABLED and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _pair_ok(out, rows_out) -> bool:
    return out.dtype == torch.bfloat16 and rows_out % 8 == 0 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0


def _gemm_tc_pair(x, weight, bias, out, dual_offset=0):
    """The product on pairs of SMs (csrc/gemm_tc2.cu): persistent, for many tokens, bfloat16 output."""
    M, K = x.shape
    N = weight.shape[0]
    err = _tc_resources(x.device)[2]
    f = _fn(_stamped("gemm_tc2.cu"), "llb_gemm_tc2",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(weight), _ptr(bias), _dt(bias) if bias is not None else 0, _ptr(out), M, N, K,
             x.stride(0), out.stride(0), dual_offset, _sm_count(x.device) // 2, _ptr(err), _stream()),
           "linear (tensor cores, paired SMs)")


def _gemm_tc(x, weight, bias, out, dual_offset=0, plan=None):
    M, K = x.shape
    N = weight.shape[0]
    if plan is None and M > 256 and _pair_ok(out, dual_offset or N):
        plan = ("pair",)
    if plan is not None and plan[0] == "pair":
        return _gemm_tc_pair(x, weight, bias, out, dual_offset)
    scratch, counters, err = _tc_resources(x.device)
    # gate/up for 17 to 64 tokens: a block per 64 outputs (gate and up rows side by side in one accumulator), twice as
    # many blocks as with a tile of 128 gate rows, which without a K split leaves half of the SMs idle at these sizes
    side_by_side = plan is not None and plan[0] == "gateup"
    if plan is None and dual_offset and 16 < M <= 64:
        side_by_side = True
    if side_by_side and dual_offset and bias is None and _pair_ok(out, dual_offset):
        bn = plan[1] if plan is not None else (32 if M <= 32 else 64)
        f = _fn(_stamped("gemm_tc.cu"), "llb_gemm_tc_gateup",
                [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
        _check(f(_ptr(x), _ptr(weight), _ptr(out), M, dual_offset, K, x.stride(0), out.stride(0), bn, _ptr(err), _stream()),
               "gate/up (tensor cores, rows side by side)")
        return
    if side_by_side:
        plan = None
    plan = plan or tc_plan(M, dual_offset or N, K, _sm_count(x.device), bool(dual_offset))
    bn, splits = plan[0], plan[1]
    cluster = plan[2] if len(plan) > 2 else 1            # (bn, splits, 0) forces the reduction through scratch
    f = _fn(_stamped("gemm_tc.cu"), "llb_gemm_tc",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(weight), _ptr(bias), _dt(bias) if bias is not None else 0, _ptr(out), _dt(out),
             M, N, K, x.stride(0), out.stride(0), bn, splits, cluster, dual_offset, _ptr(scratch), scratch.numel(),
             _ptr(counters), counters.numel(), _ptr(err), _stream()), "linear (tensor cores)")


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, plan=None) -> torch.Tensor:
    """x [M, K] (row stride free) times weight [N, K] transposed, plus bias [N]; float32 accumulation.

    bfloat16 operands with K a multiple of 8 run on the tensor cores (csrc/gemm_tc.cu); everything
    else (float32, a 32-bit weight under 16-bit activations, odd K) on the CUDA cores (csrc/gemm_simt.cu)."""
    _need_cuda(x, weight, bias)
    M, K = x.shape
    N, K2 = weight.shape
    if K != K2:
        raise KernelError(f"linear: x has {K} columns but the weight has {K2}")
    assert x.stride(1) == 1 and weight.is_contiguous()
    out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    if M == 0:
        return out
    if _tc_ok(x, weight, bias):
        _gemm_tc(x, weight, bias, out, plan=plan)
        return out
    lib = load_module("gemm_simt.cu")
    f = _fn(lib, "llb_gemm_simt", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                   c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _dt(x), _ptr(weight), _dt(weight), _ptr(bias), _dt(bias) if bias is not None else 0,
             _ptr(out), _dt(out), M, N, K, x.stride(0), out.stride(0), _stream()), "linear")
    return out


def linear_into_ok(x: torch.Tensor, weight: torch.Tensor, bias, stream: torch.Tensor) -> bool:
    """True when linear_into() takes these operands: bfloat16 on the tensor cores, a float32 stream with 16-byte
    aligned rows."""
    return (_tc_ok(x, weight, bias) and x.shape[0] > 0 and stream.dtype == torch.float32 and stream.stride(1) == 1
            and stream.stride(0) % 4 == 0 and stream.data_ptr() % 16 == 0 and stream.shape == (x.shape[0], weight.shape[0]))


def into_plan(T: int, N: int, K: int, sms: int):
    """(tokens per tile, K ranges) of linear_into() for up to 256 tokens: the smallest tile that holds the tokens, and as
    many K ranges as keep every block at two k-blocks or more and all blocks resident at once (two per SM while a
    block's ring stays under half of an SM's shared memory)."""
    bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256
    tiles = -(-N // 128) * -(-T // bn)
    kblocks = -(-K // 64)
    room = 2 * sms if bn <= 64 else sms
    return bn, max(1, min(kblocks // 2, room // tiles))


def linear_into(x: torch.Tensor, weight: torch.Tensor, bias, stream: torch.Tensor, ksplit: int = 0) -> None:
    """stream [T, N] (float32) += x weight^T + bias in place: a projection that ends in the residual add.  Up to 256
    tokens: csrc/gemm_tc.cu (INTO), the K range divided over blocks that each add their partial tile by a TMA
    reduction; more: the paired-SM kernel (csrc/gemm_tc2.cu, INTO).  ksplit: K ranges per tile (0: chosen)."""
    _need_cuda(x, weight, bias, stream)
    T, K = x.shape
    N = weight.shape[0]
    err = _tc_resources(x.device)[2]
    if T <= 256:
        bn, splits = into_plan(T, N, K, _sm_count(x.device))
        f = _fn(_stamped("gemm_tc.cu"), "llb_gemm_tc_into",
                [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
        _check(f(_ptr(x), _ptr(weight), _ptr(bias), _dt(bias) if bias is not None else 0, _ptr(stream), T, N, K, x.stride(0),
                 stream.stride(0), bn, ksplit or splits, _ptr(err), _stream()), "linear into the residual stream (tensor cores)")
        return
    f = _fn(_stamped("gemm_tc2.cu"), "llb_gemm_tc2_into",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), _ptr(weight), _ptr(bias), _dt(bias) if bias is not None else 0, _ptr(stream), T, N, K, x.stride(0),
             stream.stride(0), ksplit, _sm_count(x.device) // 2, _ptr(err), _stream()), "linear into the residual stream (tensor cores, paired SMs)")


def linear_swiglu(x: torch.Tensor, gate_up: torch.Tensor, plan=None) -> torch.Tensor:
    """up(x) * silu(gate(x)) for the fused [2I, K] matrix (gate rows first): [M, I].  On the
    tensor cores the two products share one kernel and the [M, 2I] intermediate is never written."""
    _need_cuda(x, gate_up)
    I = gate_up.shape[0] // 2
    if _tc_ok(x, gate_up, None) and x.shape[0] > 0:
        out = torch.empty((x.shape[0], I), dtype=x.dtype, device=x.device)
        _gemm_tc(x, gate_up, None, out, dual_offset=I, plan=plan)
        return out
    return swiglu(linear(x, gate_up))


FUSED_MLP = __import__("os").environ.get("LLAISYS_FUSED_MLP", "1") != "0"     # tests switch the one-launch feed-forward off to compare
_MLP_STAGES = int(__import__("os").environ.get("LLAISYS_MLP_STAGES", "0"))     # depth of its TMA ring (0: the kernel's choice)
# LLAISYS_MLP_WAIT_LIMIT: a build of that kernel whose bounded waits give up after this many tries (for trying out changes)
_MLP_DEFINES = ({"LLB_WAIT_LIMIT": int(__import__("os").environ["LLAISYS_MLP_WAIT_LIMIT"])}
                if __import__("os").environ.get("LLAISYS_MLP_WAIT_LIMIT") else None)


def mlp_fused_ok(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, residual: torch.Tensor) -> bool:
    """True when the whole SwiGLU feed-forward of these tokens can run as one launch (csrc/mlp_tc.cu):
    bfloat16 operands, at most 32 tokens, widths that are multiples of 8 and an output width whose
    accumulators fit tensor memory."""
    if not (FUSED_MLP and TC_ENABLED and x.is_cuda and x.dtype == gate_up.dtype == down.dtype == torch.bfloat16
            and residual.dtype == torch.float32 and residual.is_contiguous() and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and not ((x.data_ptr() | gate_up.data_ptr() | down.data_ptr()) & 15)):
        return False
    T, H = x.shape
    I = down.shape[1]
    if gate_up.shape != (2 * I, H) or down.shape != (H, I) or residual.shape != (T, H):
        return False
    f = _stamped("mlp_tc.cu", _MLP_DEFINES).llb_mlp_fused_ok
    f.argtypes, f.restype = [c_int, c_int, c_int], c_int
    return bool(f(T, H, I))


def mlp_fused(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, residual: torch.Tensor, stages: int = 0) -> None:
    """residual [T, H] (float32) += down(up(x) * silu(gate(x))) in one launch; gate_up is [2I, H] with the gate rows
    first, down [H, I].  See mlp_fused_ok() for what it takes."""
    _need_cuda(x, gate_up, down, residual)
    T, H = x.shape
    I = down.shape[1]
    err = _tc_resources(x.device)[2]
    stages = stages or _MLP_STAGES
    f = _fn(_stamped("mlp_tc.cu", _MLP_DEFINES), "llb_mlp_fused",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(gate_up), _ptr(down), _ptr(residual), T, H, I, _sm_count(x.device), stages,
             _ptr(err), _stream()), "feed-forward (one launch, tensor cores)")


# ------------------------------------------------------------------ attention
class _AttnParams(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p), ("row_stride", c_int),
                ("out", c_void_p), ("kpool", c_void_p), ("vpool", c_void_p), ("page_table", c_void_p),
                ("table_stride", c_int), ("ring", c_int), ("seq_start", c_void_p),
                ("seq_len_before", c_void_p), ("nh", c_int), ("nkvh", c_int), ("window", c_int),
                ("scale", c_float), ("all_from_cache", c_int), ("n_splits", c_int), ("part_o", c_void_p), ("part_ml", c_void_p)]


class _MmaAttnParams(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k_new", c_void_p), ("v_new", c_void_p), ("row_stride", c_int),
                ("out", c_void_p), ("kpool", c_void_p), ("vpool", c_void_p), ("page_table", c_void_p),
                ("table_stride", c_int), ("ring", c_int), ("seq_start", c_void_p),
                ("seq_len_before", c_void_p), ("nh", c_int), ("nkvh", c_int), ("window", c_int),
                ("scale", c_float), ("all_from_cache", c_int), ("n_splits", c_int), ("part_o", c_void_p),
                ("part_ml", c_void_p), ("rope_cos", c_void_p), ("rope_sin", c_void_p), ("rope_rows", c_int),
                ("append_new", c_int), ("cluster", c_int), ("err", c_void_p)]


MMA_ATTENTION = True                         # tests switch the tensor-core attention off to compare


def _mma_ok(qkv, dh) -> bool:
    return MMA_ATTENTION and qkv.dtype == torch.bfloat16 and dh % 16 == 0 and dh <= 128 and qkv.stride(0) % 8 == 0


_decode16 = {}


def decode_clusters16(dtype: torch.dtype, dh: int) -> int:
    """Clusters of sixteen blocks of the decode attention kernel that the device holds at once
    (0 where that kernel or that cluster size does not apply)."""
    if not (MMA_ATTENTION and dtype == torch.bfloat16 and dh % 16 == 0 and dh <= 128):
        return 0
    if dh not in _decode16:
        f = _mma_lib(dh).llb_attn_mma_decode_max_clusters
        f.argtypes, f.restype = [c_int], c_int
        _decode16[dh] = int(f(16))
    return _decode16[dh]


def decode_fusion_ok(dtype: torch.dtype, dh: int) -> bool:
    """True when decode attention can itself rotate the query and the new key and append the
    new key and value to the cache (the tensor-core kernel), so that no kernel has to do it before."""
    return MMA_ATTENTION and dtype == torch.bfloat16 and dh % 16 == 0 and dh <= 128


class _TcAttnParams(ctypes.Structure):
    _fields_ = [("out", c_void_p), ("page_table", c_void_p), ("table_stride", c_int), ("seq_start", c_void_p),
                ("seq_len_before", c_void_p), ("nh", c_int), ("nkvh", c_int), ("window", c_int), ("scale", c_float),
                ("err", c_void_p), ("n_split", c_int)]


TC_ATTENTION = True                          # tests switch the tcgen05 prefill attention off to compare


def prefill_tc_ok(dtype: torch.dtype, dh: int) -> bool:
    """True when prefill attention can run on tcgen05 (csrc/attention_tc.cu): bfloat16, head size 64
    or 128.  That kernel reads every key, those of the step included, from the cache."""
    return TC_ATTENTION and dtype == torch.bfloat16 and dh in (64, 128)


def require_head_dim(dh: int) -> None:
    """Raises unless some attention kernel of this package takes heads of `dh` elements: the CUDA-core
    kernel (both precisions) takes any even size up to 256; the tensor-core kernels take multiples of
    16 up to 128 (mma.sync) and 64 or 128 (tcgen05) and are chosen where they apply."""
    if dh <= 0 or dh % 2 or dh > 256:
        raise KernelError(f"attention: head size {dh} is not supported (even, at most 256)")


def _mma_lib(dh: int):
    lib = _stamped("attention_mma.cu", {"LLB_HEAD_DIM": dh})
    return lib


def _attn_lib(dh: int):
    require_head_dim(dh)
    return load_module("attention_simt.cu", {"LLB_HEAD_DIM": dh})


def _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before,
                 window, scale, cls=None):
    es = qkv.element_size()
    p = (cls or _AttnParams)()
    p.q = qkv.data_ptr()
    p.k_new = qkv.data_ptr() + nh * dh * es
    p.v_new = qkv.data_ptr() + (nh + nkvh) * dh * es
    p.row_stride = qkv.stride(0)
    p.out = out.data_ptr()
    p.kpool, p.vpool = kpool.data_ptr(), vpool.data_ptr()
    p.page_table, p.table_stride, p.ring = page_table.data_ptr(), page_table.shape[1], ring
    p.seq_start, p.seq_len_before = seq_start.data_ptr(), seq_len_before.data_ptr()
    p.nh, p.nkvh, p.window, p.scale = nh, nkvh, int(window or 0), scale
    p.all_from_cache, p.n_splits, p.part_o, p.part_ml = 0, 1, None, None
    return p


def attention_prefill(qkv, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before,
                      n_seqs: int, max_new: int, window, scale, all_from_cache: bool = False,
                      tc_split: int = 0) -> torch.Tensor:
    """Attention of the new tokens of each sequence over its cached keys (positions before the
    step) and the step's own keys, read from the packed projections `qkv` [T, (nh + 2 nkvh) dh]
    whose query and key heads are already rotated.  With all_from_cache the step's keys are
    read from the cache too (they were put there by an earlier call).  Returns [T, nh * dh].
    tc_split: CTAs per row block of the tcgen05 kernel (1, 2 or 4; 0: chosen by the number of row blocks)."""
    _need_cuda(qkv, kpool, vpool, page_table)
    assert qkv.dtype == kpool.dtype == vpool.dtype
    out = torch.empty((qkv.shape[0], nh * dh), dtype=qkv.dtype, device=qkv.device)
    if all_from_cache and prefill_tc_ok(qkv.dtype, dh) and ring >= page_table.shape[1] and qkv.stride(0) % 8 == 0:
        p = _TcAttnParams()
        p.out, p.page_table, p.table_stride = out.data_ptr(), page_table.data_ptr(), page_table.shape[1]
        p.seq_start, p.seq_len_before = seq_start.data_ptr(), seq_len_before.data_ptr()
        p.nh, p.nkvh, p.window, p.scale = nh, nkvh, int(window or 0), scale
        p.err = _tc_resources(qkv.device)[2].data_ptr()
        # few row blocks (up to one and a half per SM): two CTAs share each block's key range, so that the longest
        # CTA gets shorter (measured at 12 heads: 30.5 vs 33.7 us at 2,048 tokens, 73 vs 64 us at 4,096; four CTAs
        # per block always lost to the cost of the merge)
        ctas = -(-max_new // 128) * nh * n_seqs
        p.n_split = tc_split if tc_split else (2 if ctas * 2 <= 3 * _sm_count(qkv.device) and dh >= 64 else 1)
        f = _fn(load_module("attention_tc.cu", {"LLB_HEAD_DIM": dh}), "llb_attn_tc_prefill",
                [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, _TcAttnParams, c_int, c_int, c_void_p])
        _check(f(qkv.data_ptr(), qkv.shape[0], qkv.stride(0), kpool.data_ptr(), vpool.data_ptr(), kpool.shape[0],
                 p, n_seqs, max_new, _stream()), "attention_prefill (tcgen05)")
        return out
    if _mma_ok(qkv, dh):
        p = _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, window,
                         scale, _MmaAttnParams)
        p.all_from_cache = int(all_from_cache)
        f = _fn(_mma_lib(dh), "llb_attn_mma_prefill", [_MmaAttnParams, c_int, c_int, c_void_p])
        _check(f(p, n_seqs, max_new, _stream()), "attention_prefill (tensor cores)")
        return out
    p = _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, window, scale)
    p.all_from_cache = int(all_from_cache)
    f = _fn(_attn_lib(dh), "llb_attn_prefill", [_AttnParams, c_int, c_int, c_int, c_void_p])
    _check(f(p, _dt(qkv), n_seqs, max_new, _stream()), "attention_prefill")
    return out


def attention_decode(qkv, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before,
                     n_seqs: int, window, scale, n_splits: int = 1, rope=None, append_new: bool = False) -> torch.Tensor:
    """Attention of one new token per sequence over the cache.

    By default the new token's (rotated) key and value are already in the cache.  Where
    decode_fusion_ok() holds, the kernel can do that work itself: rope = (cos, sin) tables makes it
    rotate the query heads (and the new key), append_new makes it take the new key and value from
    `qkv`, use them and write them to the cache."""
    _need_cuda(qkv, kpool, vpool, page_table)
    assert qkv.dtype == kpool.dtype == vpool.dtype
    out = torch.empty((qkv.shape[0], nh * dh), dtype=qkv.dtype, device=qkv.device)
    mma = _mma_ok(qkv, dh)
    p = _attn_params(qkv, out, nh, nkvh, dh, kpool, vpool, page_table, ring, seq_start, seq_len_before, window, scale,
                     _MmaAttnParams if mma else None)
    if (rope is not None or append_new) and not mma:
        raise KernelError("attention_decode: the fused rotation / append needs the tensor-core kernel (see decode_fusion_ok)")
    keep = None
    if mma:
        n_splits = min(n_splits, 64)
        if rope is not None:
            p.rope_cos, p.rope_sin, p.rope_rows = rope[0].data_ptr(), rope[1].data_ptr(), rope[0].shape[0]
        p.append_new = int(append_new)
        p.cluster = int(1 < n_splits <= 8 or n_splits == 16)      # few slices merge inside a cluster, through shared memory
        p.err = _tc_resources(qkv.device)[2].data_ptr()           # a bounded wait of that merge that runs out says so here
    p.n_splits = n_splits
    if n_splits > 1 and not (mma and p.cluster):
        part_o = torch.empty((n_seqs, nh, n_splits, dh), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n_seqs, nh, n_splits, 2), dtype=torch.float32, device=qkv.device)
        p.n_splits, p.part_o, p.part_ml = n_splits, part_o.data_ptr(), part_ml.data_ptr()
        keep = (part_o, part_ml)
    if mma:
        f = _fn(_mma_lib(dh), "llb_attn_mma_decode", [_MmaAttnParams, c_int, c_void_p])
        _check(f(p, n_seqs, _stream()), "attention_decode (tensor cores)", 2 if (n_splits > 1 and not p.cluster) else 1)
    else:
        f = _fn(_attn_lib(dh), "llb_attn_decode", [_AttnParams, c_int, c_int, c_void_p])
        _check(f(p, _dt(qkv), n_seqs, _stream()), "attention_decode", 2 if n_splits > 1 else 1)
    del keep
    return out


# ------------------------------------------------------------------ choice of the next token
_argmax_counters = {}          # device -> int32 [4096], zero between launches (the split arg-max's per-row counters)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """int32 index of the first maximum of every row of float32 logits [R, V]."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    # few rows of a wide vocabulary: several blocks share a row, so that the device's SMs all read
    parts = min(64, (2 * _sm_count(logits.device)) // max(R, 1), V // 2048)
    if parts >= 2 and R <= 4096:
        counters = _argmax_counters.get(logits.device)
        if counters is None:
            counters = _argmax_counters[logits.device] = torch.zeros(4096, dtype=torch.int32, device=logits.device)
        part = torch.empty((R * parts, 2), dtype=torch.int32, device=logits.device)
        f = _fn(load_module("sampling.cu"), "llb_argmax_split",
                [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
        _check(f(_ptr(logits), logits.stride(0), R, V, parts, _ptr(part), _ptr(counters), _ptr(out), _stream()), "argmax")
        return out
    f = _fn(load_module("sampling.cu"), "llb_argmax", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int,
           keys: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V]; see csrc/sampling.cu for the rule.  keys and
    steps (int32 [R]) are the request number and the number of tokens the request has drawn."""
    _need_cuda(logits, keys, steps)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _fn(load_module("sampling.cu"), "llb_sample",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_float, c_int, c_float, c_ulonglong,
             c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(out), temperature, top_k, top_p,
             seed & 0xFFFFFFFFFFFFFFFF, _ptr(keys), _ptr(steps), _stream()), "sample")
    return out


def uniform(seed: int, key: int, step: int) -> float:
    """The uniform in [0, 1) that `sample` uses for (seed, key, step) (splitmix64 finaliser)."""
    mask, G = 0xFFFFFFFFFFFFFFFF, 0x9E3779B97F4A7C15

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)

    z = mix((mix((seed + G * (key + 1)) & mask) + G * (step + 1)) & mask)
    return (z >> 11) / 9007199254740992.0
