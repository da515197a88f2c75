"""Each kernel alone against the plain formulas, at sizes other than the tiny models'."""
import math

import numpy as np
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 2.0 ** -7) * scale


def _close(got, want, dtype, atol=None):
    """The kernel computes in float32 from the same rounded inputs as the plain formula, so what
    remains is float32 summation error and, for bfloat16, the rounding of the output itself
    (half a unit in the last place: 2^-9 relative; 2^-8 is allowed)."""
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else got
    if dtype == torch.float32:
        bound = (atol or 2e-5) + 1e-5 * np.abs(want)
    else:
        bound = (atol or 1e-3) + 2.0 ** -8 * np.abs(want)
    err = np.abs(got - want)
    assert np.isfinite(got).all(), "non-finite output"
    worst = np.unravel_index(np.argmax(err - bound), err.shape)
    assert (err <= bound).all(), f"worst at {worst}: got {got[worst]}, want {want[worst]}"


def _rt(x, dtype):
    """float64 numpy values as the kernel sees them after rounding to dtype."""
    return torch.from_numpy(np.asarray(x)).to(dtype).double().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    from llaisys_b200 import kernels
    rng = np.random.default_rng(0)
    table = torch.from_numpy(rng.normal(size=(301, 72))).to(dtype).to(DEV)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = kernels.embedding(ids, table, err)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float()) and int(err) == 0
    bad = torch.tensor([3, 301], dtype=torch.int32, device=DEV)
    out = kernels.embedding(bad, table, err)
    assert int(err) == 1 and float(out[1].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H", [(1, 8), (5, 200), (37, 1536), (3, 5000), (4, 3584), (2, 8192), (3, 1001),
                                 (300, 1536), (257, 256), (261, 3584), (256, 4096), (300, 5120)])       # many rows: a warp per row where the width allows
def test_add_rmsnorm(dtype, T, H):
    from llaisys_b200 import kernels
    rng = np.random.default_rng(T * H)
    res, delta, w = rng.normal(size=(T, H)), rng.normal(size=(T, H)), 1 + 0.1 * rng.normal(size=H)
    res_t = torch.from_numpy(res).float().to(DEV)
    delta_t = torch.from_numpy(delta).to(dtype).to(DEV)
    w_t = torch.from_numpy(w).to(dtype).to(DEV)
    x = res_t.double().cpu().numpy() + _rt(delta, dtype)
    want = plain.rms_norm(x, _rt(w, dtype), 1e-5)
    out = kernels.add_rmsnorm(res_t, delta_t, w_t, 1e-5, dtype)
    assert np.abs(res_t.double().cpu().numpy() - x).max() < 1e-6          # the sum is kept in float32
    _close(out, want, dtype)
    # no delta; a float32 weight under a bfloat16 model; a gather that leaves the residual alone
    keep = res_t.clone()
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    out = kernels.add_rmsnorm(res_t, None, torch.from_numpy(w).float().to(DEV), 1e-5, dtype, rows=rows)
    want = plain.rms_norm(keep.double().cpu().numpy()[[T - 1, 0]], _rt(w, torch.float32), 1e-5)
    assert torch.equal(res_t, keep)
    _close(out, want, dtype)
    # partial sums are added in order
    parts = torch.from_numpy(rng.normal(size=(3, T, H))).float().to(DEV)
    kernels.add_rmsnorm(res_t, parts, w_t, 1e-5, dtype)
    assert np.abs(res_t.double().cpu().numpy() - (keep.double().cpu().numpy() + parts.double().sum(0).cpu().numpy())).max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 33, 70), (7, 130, 257), (8, 64, 64), (9, 100, 48), (70, 200, 300), (130, 67, 1000)])
def test_linear(dtype, M, N, K):
    from llaisys_b200 import kernels
    rng = np.random.default_rng(M + N + K)
    x, w, b = rng.normal(size=(M, K)), rng.normal(size=(N, K)) * 0.1, rng.normal(size=N)
    xt, wt, bt = (torch.from_numpy(a).to(dtype).to(DEV) for a in (x, w, b))
    want = plain.linear(_rt(x, dtype), _rt(w, dtype), _rt(b, dtype))
    got = kernels.linear(xt, wt, bt, out_dtype=torch.float32)
    assert np.abs(got.double().cpu().numpy() - want).max() < 1e-4 * math.sqrt(K)
    got = kernels.linear(xt, wt)                      # no bias, activation dtype out
    want = plain.linear(_rt(x, dtype), _rt(w, dtype))
    # bfloat16 runs on the tensor cores, where the probabilities are rounded to bfloat16 as the operand of P*V:
    # a further 2^-9 relative on top of the output's own rounding
    _close(got, want, dtype, atol=1e-4 if dtype == torch.float32 else 6e-3)
    # a strided view as input, a float32 weight under bfloat16 activations
    wide = torch.zeros((M, K + 24), dtype=dtype, device=DEV)
    wide[:, 8:8 + K] = xt
    got = kernels.linear(wide[:, 8:8 + K], torch.from_numpy(w).float().to(DEV), out_dtype=torch.float32)
    want = plain.linear(_rt(x, dtype), _rt(w, torch.float32))
    assert np.abs(got.double().cpu().numpy() - want).max() < 1e-4 * math.sqrt(K)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    from llaisys_b200 import kernels
    rng = np.random.default_rng(4)
    gu = rng.normal(size=(11, 2 * 136)) * 3
    got = kernels.swiglu(torch.from_numpy(gu).to(dtype).to(DEV))
    r = _rt(gu, dtype)
    _close(got, plain.swiglu(r[:, :136], r[:, 136:]), dtype)


def _paged(kv, page_ids, dtype):
    """kv: [L, nkvh, d] numpy -> pool [pages, nkvh, 64, d] with the sequence's pages at page_ids."""
    L, nkvh, d = kv.shape
    pool = torch.full((max(page_ids) + 2, nkvh, 64, d), float("nan"), dtype=dtype)
    for lp, pid in enumerate(page_ids):
        chunk = torch.from_numpy(kv[lp * 64:(lp + 1) * 64]).to(dtype)          # [n, nkvh, d]
        pool[pid, :, :chunk.shape[0]] = chunk.permute(1, 0, 2)
    return pool.to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("theta,dh", [(1e4, 32), (1e6, 48)])
def test_rope_and_append(dtype, theta, dh):
    from llaisys_b200 import kernels
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import BuildEnv, build_part
    nh, nkvh = 3, 1
    rope = build_part("position", PartSpec("rope_half_split", {"head_dim": dh, "theta": theta}),
                      BuildEnv(dtype, torch.device(DEV)))
    rng = np.random.default_rng(5)
    # two sequences: 70 cached + 3 new, 0 cached + 66 new
    lens, news = [70, 0], [3, 66]
    T = sum(news)
    qkv = rng.normal(size=(T, (nh + 2 * nkvh) * dh))
    qkv_t = torch.from_numpy(qkv).to(dtype).to(DEV)
    tok_seq = torch.tensor([0] * 3 + [1] * 66, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([70, 71, 72] + list(range(66)), dtype=torch.int32, device=DEV)
    seq_start = torch.tensor([0, 3, 69], dtype=torch.int32, device=DEV)
    len_before = torch.tensor(lens, dtype=torch.int32, device=DEV)
    table = torch.tensor([[4, 1], [0, 3]], dtype=torch.int32, device=DEV)
    kpool = torch.zeros((5, nkvh, 64, dh), dtype=dtype, device=DEV)
    vpool = torch.zeros_like(kpool)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    cos, sin = rope.table(73)
    kernels.rope_append(qkv_t, nh, nkvh, dh, cos=cos, sin=sin, tok_pos=tok_pos, err=err,
                        append=dict(tok_seq=tok_seq, seq_start=seq_start, seq_len_before=len_before,
                                    kpool=kpool, vpool=vpool, page_table=table, ring=2))
    assert int(err) == 0
    r = _rt(qkv, dtype).reshape(T, nh + 2 * nkvh, dh)
    pos = tok_pos.cpu().numpy()
    want_qk = plain.rope(r[:, :nh + nkvh], pos, theta)
    got = qkv_t.double().cpu().numpy().reshape(T, nh + 2 * nkvh, dh)
    _close(got[:, :nh + nkvh], want_qk, dtype)
    assert np.array_equal(got[:, nh + nkvh:], r[:, nh + nkvh:])               # values untouched
    kp, vp = kpool.double().cpu().numpy(), vpool.double().cpu().numpy()
    pages = table.cpu().numpy()
    for t in range(T):
        s, p = int(tok_seq[t]), int(pos[t])
        page = pages[s][p // 64]
        assert np.array_equal(kp[page, 0, p % 64], got[t, nh]) and np.array_equal(vp[page, 0, p % 64], r[t, nh + 1])
    assert float(kpool[2].abs().sum()) == 0.0                                 # a page of no one stays untouched
    # a position beyond the table is reported, not read
    kernels.rope_append(qkv_t, nh, nkvh, dh, cos=cos[:10], sin=sin[:10], tok_pos=tok_pos, err=err)
    assert int(err) == 2


def _attention_case(dtype, nh, nkvh, dh, lens_before, news, window, seed, ring=None, gain=3.0):
    """Random q, k, v with sharp scores; returns device inputs and the plain outputs."""
    rng = np.random.default_rng(seed)
    B, T = len(news), sum(news)
    width = nh + 2 * nkvh
    qkv = rng.normal(size=(T, width, dh))
    qkv[:, :nh + nkvh] *= gain
    n_pages_seq = [-(-(l + n) // 64) for l, n in zip(lens_before, news)]
    perm = rng.permutation(sum(n_pages_seq) + 3).tolist()
    past_k = [rng.normal(size=(l, nkvh, dh)) * gain for l in lens_before]
    past_v = [rng.normal(size=(l, nkvh, dh)) for l in lens_before]
    tables, outs, t0 = [], [], 0
    P = max(n_pages_seq)
    kpool = torch.full((len(perm), nkvh, 64, dh), float("nan"), dtype=dtype)
    vpool = torch.full_like(kpool, float("nan"))
    for b in range(B):
        ids = [perm.pop() for _ in range(n_pages_seq[b])]
        tables.append(ids + [0] * (P - len(ids)))
        for lp, pid in enumerate(ids):
            for pool, past in ((kpool, past_k[b]), (vpool, past_v[b])):
                chunk = torch.from_numpy(past[lp * 64:(lp + 1) * 64]).to(dtype)
                if chunk.shape[0]:
                    pool[pid, :, :chunk.shape[0]] = chunk.permute(1, 0, 2)
        new = _rt(qkv[t0:t0 + news[b]], dtype)
        k = np.concatenate([_rt(past_k[b], dtype), new[:, nh:nh + nkvh]])
        v = np.concatenate([_rt(past_v[b], dtype), new[:, nh + nkvh:]])
        outs.append(plain.self_attention(new[:, :nh], k, v, 1 / math.sqrt(dh), window))
        t0 += news[b]
    dev = dict(
        qkv=torch.from_numpy(qkv.reshape(T, width * dh)).to(dtype).to(DEV), kpool=kpool.to(DEV), vpool=vpool.to(DEV),
        table=torch.tensor(tables, dtype=torch.int32, device=DEV),
        seq_start=torch.tensor(np.concatenate([[0], np.cumsum(news)]), dtype=torch.int32, device=DEV),
        len_before=torch.tensor(lens_before, dtype=torch.int32, device=DEV))
    return dev, np.concatenate(outs).reshape(T, nh * dh)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkvh,dh,window", [(4, 2, 32, None), (6, 1, 48, 70), (3, 3, 64, 5), (8, 2, 128, None), (2, 1, 16, 64)])
def test_attention_prefill(dtype, nh, nkvh, dh, window):
    from llaisys_b200 import kernels
    lens_before, news = [0, 130, 64, 5], [100, 37, 1, 200]
    d, want = _attention_case(dtype, nh, nkvh, dh, lens_before, news, window, seed=nh * dh)
    got = kernels.attention_prefill(d["qkv"], nh, nkvh, dh, d["kpool"], d["vpool"], d["table"], d["table"].shape[1],
                                    d["seq_start"], d["len_before"], len(news), max(news), window, 1 / math.sqrt(dh))
    # bfloat16 runs on the tensor cores, where the probabilities are rounded to bfloat16 as the operand of P*V:
    # a further 2^-9 relative on top of the output's own rounding
    _close(got, want, dtype, atol=1e-4 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkvh,dh,window", [(4, 2, 32, None), (6, 1, 48, 70), (12, 2, 128, None), (5, 5, 64, 3), (40, 1, 16, 129)])
@pytest.mark.parametrize("splits", [1, 3, 8, 11, 16])
def test_attention_decode(dtype, nh, nkvh, dh, window, splits):
    from llaisys_b200 import kernels
    lens_before, news = [0, 129, 63, 64, 500], [1, 1, 1, 1, 1]
    d, want = _attention_case(dtype, nh, nkvh, dh, lens_before, news, window, seed=nh + dh + splits)
    # decode reads the cache alone: put the new keys and values there first
    tok = torch.arange(5, dtype=torch.int32, device=DEV)
    kernels.rope_append(d["qkv"], nh, nkvh, dh, tok_pos=d["len_before"], append=dict(
        tok_seq=tok, seq_start=d["seq_start"], seq_len_before=d["len_before"], kpool=d["kpool"], vpool=d["vpool"],
        page_table=d["table"], ring=d["table"].shape[1]), err=torch.zeros(1, dtype=torch.int32, device=DEV))
    got = kernels.attention_decode(d["qkv"], nh, nkvh, dh, d["kpool"], d["vpool"], d["table"], d["table"].shape[1],
                                   d["seq_start"], d["len_before"], 5, window, 1 / math.sqrt(dh), n_splits=splits)
    # bfloat16 runs on the tensor cores, where the probabilities are rounded to bfloat16 as the operand of P*V:
    # a further 2^-9 relative on top of the output's own rounding
    _close(got, want, dtype, atol=1e-4 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key(dtype):
    """One key among several hundred matches the query; the output must be its value."""
    from llaisys_b200 import kernels
    nh, nkvh, dh, L = 2, 1, 32, 700
    for far in (0, 63, 64, 401, 698):
        rng = np.random.default_rng(far)
        k = rng.normal(size=(L + 1, nkvh, dh)) * 0.1
        v = rng.normal(size=(L + 1, nkvh, dh))
        q = np.zeros((1, nh + 2, dh))
        q[0, :nh] = 20.0 * np.sign(rng.normal(size=dh))
        k[far, 0] = q[0, 0] * 1.0
        q[0, nh], q[0, nh + 1] = k[L, 0], v[L, 0]
        pages = list(range(11, 0, -1))
        kpool, vpool = _paged(k[:L], pages, dtype), _paged(v[:L], pages, dtype)
        qkv = torch.from_numpy(q.reshape(1, -1)).to(dtype).to(DEV)
        table = torch.tensor([pages], dtype=torch.int32, device=DEV)
        ss = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
        lb = torch.tensor([L], dtype=torch.int32, device=DEV)
        kernels.rope_append(qkv, nh, nkvh, dh, tok_pos=lb, append=dict(tok_seq=torch.zeros(1, dtype=torch.int32, device=DEV),
                            seq_start=ss, seq_len_before=lb, kpool=kpool, vpool=vpool, page_table=table, ring=11),
                            err=torch.zeros(1, dtype=torch.int32, device=DEV))
        for splits in (1, 4):
            out = kernels.attention_decode(qkv, nh, nkvh, dh, kpool, vpool, table, 11, ss, lb, 1, None, 1.0, n_splits=splits)
            assert np.abs(out[0, :dh].double().cpu().numpy() - _rt(v[far, 0], dtype)).max() < 1e-2
        out = kernels.attention_prefill(qkv, nh, nkvh, dh, kpool, vpool, table, 11, ss, lb, 1, 1, None, 1.0)
        assert np.abs(out[0, :dh].double().cpu().numpy() - _rt(v[far, 0], dtype)).max() < 1e-2


def test_argmax_first_maximum():
    from llaisys_b200 import kernels
    rng = np.random.default_rng(1)
    x = rng.normal(size=(6, 5003)).astype(np.float32)
    x[1, 4000] = x[1, 77] = 9.0
    x[2, :] = -np.inf
    x[3, 5002] = 50.0
    x[4, 0] = 50.0
    got = kernels.argmax(torch.from_numpy(x).to(DEV)).tolist()
    assert got == [plain.argmax(r) for r in x] and got[1] == 77 and got[2] == 0


@pytest.mark.parametrize("R,V,pad", [(8, 151936, 0), (1, 151937, 3), (3, 40001, 1), (64, 20000, 0), (300, 4100, 2)])
def test_argmax_of_few_wide_rows(R, V, pad):
    """Few rows of a wide vocabulary go to several blocks per row: the first maximum, also where the maxima of a tie
    lie in different blocks' parts, at a part's first and last place, and with rows that start off 16-byte boundaries."""
    from llaisys_b200 import kernels
    rng = np.random.default_rng(R + V)
    x = rng.normal(size=(R, V + pad)).astype(np.float32)
    x[0, V - 1] = 40.0                                   # the very last place
    if R > 1:
        x[1, 5] = x[1, V // 2] = x[1, V - 2] = 30.0      # a tie across parts: the first wins
    if R > 2:
        x[2, :V] = -np.inf                               # nothing but -inf: index 0
    wide = torch.from_numpy(x).to(DEV)
    for _ in range(2):                                   # the counters are back at zero after a launch
        got = kernels.argmax(wide[:, :V]).tolist()
        assert got == [plain.argmax(r[:V]) for r in x]
    assert got[0] == V - 1 and (R < 2 or got[1] == 5) and (R < 3 or got[2] == 0)


@pytest.mark.parametrize("V", [257, 5000, 151936])
@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.7, 0, 1.0), (1.0, 50, 1.0), (1.0, 0, 0.8),
                                                     (0.8, 50, 0.8), (1.3, 7, 0.3), (1.0, 1, 1.0), (0.0, 0, 1.0)])
def test_sampling_follows_the_rule(V, temperature, top_k, top_p):
    from llaisys_b200 import kernels
    rng = np.random.default_rng(V + top_k)
    R = 24
    logits = (rng.normal(size=(R, V)) * 3).astype(np.float32)
    logits[0, 5:9] = logits[0].max() + 1.0                  # ties at the top
    logits[1, :] = 0.25                                     # all equal
    lt = torch.from_numpy(logits).to(DEV)
    keys = torch.arange(R, dtype=torch.int32, device=DEV) + 100
    steps = torch.arange(R, dtype=torch.int32, device=DEV) * 3
    got = kernels.sample(lt, temperature, top_k, top_p, 1234, keys, steps).tolist()
    miss = 0
    for r in range(R):
        u = kernels.uniform(1234, 100 + r, 3 * r)
        want = plain.sample(logits[r], temperature, top_k, top_p, u)
        if got[r] != want:
            # float32 exp against float64: a draw that lands within rounding of a boundary may fall to
            # the neighbour; it must still be a kept token right next to the boundary
            lo, hi = plain.sample(logits[r], temperature, top_k, top_p, max(0.0, u - 1e-5)), \
                plain.sample(logits[r], temperature, top_k, top_p, min(1 - 1e-12, u + 1e-5))
            assert got[r] in (lo, hi), (r, got[r], want)
            miss += 1
    assert miss <= 1


def test_sampling_statistics_and_reproducibility():
    from llaisys_b200 import kernels
    p = np.array([0.5, 0.25, 0.125, 0.125])
    logits = torch.from_numpy(np.log(p)).float().to(DEV).repeat(4000, 1)
    keys = torch.arange(4000, dtype=torch.int32, device=DEV)
    steps = torch.zeros(4000, dtype=torch.int32, device=DEV)
    a = kernels.sample(logits, 1.0, 0, 1.0, 7, keys, steps)
    assert torch.equal(a, kernels.sample(logits, 1.0, 0, 1.0, 7, keys, steps))
    assert not torch.equal(a, kernels.sample(logits, 1.0, 0, 1.0, 8, keys, steps))
    freq = np.bincount(a.cpu().numpy(), minlength=4) / 4000
    assert np.abs(freq - p).max() < 0.03
    b = kernels.sample(logits, 1.0, 2, 1.0, 7, keys, steps).cpu().numpy()
    assert set(b.tolist()) == {0, 1} and abs((b == 0).mean() - 2 / 3) < 0.03
    # the device's uniform is the documented function of (seed, key, step)
    import ctypes
    from llaisys_b200.csrc.build import load_module
    f = load_module("sampling.cu").llb_uniform_host
    f.restype, f.argtypes = ctypes.c_double, [ctypes.c_ulonglong] * 3
    for s, k, t in [(0, 0, 0), (7, 3, 9), (2 ** 40 + 5, 2 ** 31 - 1, 12345)]:
        assert f(s, k, t) == kernels.uniform(s, k, t)


# ----------------------------------------------------------------------------- tensor-core matrix product
def _tc_case(T, N, K, seed, bias=None):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.normal(size=(T, K))).to(torch.bfloat16).to(DEV)
    w = torch.from_numpy(rng.normal(size=(N, K)) * 0.05).to(torch.bfloat16).to(DEV)
    b = None if bias is None else torch.from_numpy(rng.normal(size=N)).to(bias).to(DEV)
    return x, w, b


def _tc_check(got, want, K):
    got = got.double().cpu().numpy()
    bound = 5e-4 * math.sqrt(K / 64) + 2e-3 * np.abs(want)
    err = np.abs(got - want)
    assert np.isfinite(got).all(), "non-finite output"
    worst = np.unravel_index(np.argmax(err - bound), err.shape)
    assert (err <= bound).all(), f"worst at {worst}: got {got[worst]}, want {want[worst]}"


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (8, 2048, 1536), (5, 200, 72), (16, 1536, 8960), (33, 130, 520),
                                   (64, 256, 128), (100, 384, 1000), (300, 500, 776), (1000, 1536, 256), (17, 151936, 64)])
def test_linear_tensor_cores(T, N, K):
    from llaisys_b200 import kernels
    x, w, b = _tc_case(T, N, K, T + N + K, bias=torch.bfloat16)
    want = plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy(), b.double().cpu().numpy())
    _tc_check(kernels.linear(x, w, b, out_dtype=torch.float32), want, K)
    got = kernels.linear(x, w, b.float())                          # bfloat16 out, float32 bias
    _close(got, want, torch.bfloat16, atol=5e-3)
    assert kernels.tc_error(DEV) == 0
    # the CUDA-core path gives the same numbers up to summation order
    kernels.ops.TC_ENABLED = False
    try:
        ref = kernels.linear(x, w, b, out_dtype=torch.float32)
    finally:
        kernels.ops.TC_ENABLED = True
    _tc_check(ref, want, K)


@pytest.mark.parametrize("T,N,K", [(257, 256, 64), (300, 520, 200), (700, 1000, 776), (1030, 136, 96), (2048, 1536, 1536)])
def test_linear_on_paired_sms_and_on_single_ones(T, N, K):
    """More than 256 tokens run on pairs of SMs (csrc/gemm_tc2.cu); a plan sends them to the one-CTA kernel."""
    from llaisys_b200 import kernels
    x, w, b = _tc_case(T, N, K, T + N + K, bias=torch.bfloat16)
    want = plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy(), b.double().cpu().numpy())
    outs = [kernels.linear(x, w, b, plan=plan) for plan in (None, ("pair",), (256, 1))]
    for got in outs:
        _close(got, want, torch.bfloat16, atol=5e-3)
    assert torch.equal(outs[0], outs[1])
    wide = torch.zeros((T, K + 16), dtype=torch.bfloat16, device=DEV)
    wide[:, 8:8 + K] = x
    _close(kernels.linear(wide[:, 8:8 + K], w, None, plan=("pair",)), plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy()),
           torch.bfloat16, atol=5e-3)
    assert kernels.tc_error(DEV) == 0


@pytest.mark.parametrize("T,I,K", [(300, 264, 200), (257, 128, 64), (1000, 136, 96), (1500, 1000, 520), (300, 264, 2112)])
@pytest.mark.parametrize("plan", [None, ("pair",), (256, 1)])
def test_linear_swiglu_on_paired_sms_and_on_single_ones(T, I, K, plan):
    """(The paired kernel has two gate/up variants: gate and up rows side by side in one accumulator up to K = 2,048,
    two accumulators beyond; the last case takes the second.)"""
    from llaisys_b200 import kernels
    x, w, _ = _tc_case(T, 2 * I, K, T + I)
    w = (w.float() * 4).to(torch.bfloat16)
    gu = plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy())
    want = plain.swiglu(gu[:, :I], gu[:, I:])
    got = kernels.linear_swiglu(x, w, plan=plan)
    assert got.shape == (T, I)
    _close(got, want, torch.bfloat16, atol=5e-3)
    assert kernels.tc_error(DEV) == 0


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("splits,cluster", [(1, 0), (2, 0), (5, 0), (2, 1), (4, 1), (8, 1)])
def test_linear_tensor_cores_every_tile_and_split(bn, splits, cluster):
    """cluster = 1: the splits reduce through distributed shared memory (a tile of 256 tokens falls back to
    the scratch buffer); cluster = 0: through the scratch buffer and the last-arriver fix-up."""
    from llaisys_b200 import kernels
    T, N, K = bn + 3, 300, 1096                 # two token tiles, three row tiles, eighteen k-blocks (the last one partial)
    x, w, b = _tc_case(T, N, K, bn * splits, bias=torch.float32)
    want = plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy(), b.double().cpu().numpy())
    for _ in range(2):                          # twice: the tile counters must be back at zero
        _tc_check(kernels.linear(x, w, b, out_dtype=torch.float32, plan=(bn, splits, cluster)), want, K)
    wide = torch.zeros((T, K + 16), dtype=torch.bfloat16, device=DEV)
    wide[:, 8:8 + K] = x
    _tc_check(kernels.linear(wide[:, 8:8 + K], w, b, out_dtype=torch.float32, plan=(bn, splits, cluster)), want, K)
    assert kernels.tc_error(DEV) == 0


@pytest.mark.parametrize("bn,T", [(16, 9), (64, 50), (128, 70)])
def test_linear_tensor_cores_sixteen_splits_in_one_cluster(bn, T):
    from llaisys_b200 import kernels
    N, K = 300, 4096                            # 64 k-blocks: four for each of sixteen CTAs
    x, w, b = _tc_case(T, N, K, bn + T, bias=torch.float32)
    want = plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy(), b.double().cpu().numpy())
    for _ in range(2):
        _tc_check(kernels.linear(x, w, b, out_dtype=torch.float32, plan=(bn, 16, 1)), want, K)
    assert kernels.tc_error(DEV) == 0


@pytest.mark.parametrize("T,I,K,plan", [(8, 8960, 1536, None), (3, 200, 72, None), (70, 136, 96, None), (300, 264, 200, None),
                                        (20, 300, 712, (32, 3)), (20, 300, 712, (256, 2)), (130, 300, 712, (128, 4)),
                                        (130, 300, 712, (128, 4, 0)), (9, 300, 1096, (16, 8)), (40, 136, 520, (64, 2)),
                                        (17, 8960, 1536, None), (64, 8960, 1536, None), (40, 136, 520, (64, 1)),
                                        (20, 72, 200, ("gateup", 32)), (33, 200, 72, ("gateup", 64)), (100, 328, 1096, ("gateup", 64)),
                                        (64, 64, 64, ("gateup", 64)), (70, 1000, 520, ("gateup", 32)), (50, 264, 2112, ("gateup", 64))])
def test_linear_swiglu_tensor_cores(T, I, K, plan):
    from llaisys_b200 import kernels
    x, w, _ = _tc_case(T, 2 * I, K, T + I)
    w = (w.float() * 4).to(torch.bfloat16)
    gu = plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy())
    want = plain.swiglu(gu[:, :I], gu[:, I:])
    got = kernels.linear_swiglu(x, w, plan=plan)
    assert got.shape == (T, I)
    _close(got, want, torch.bfloat16, atol=5e-3)
    assert kernels.tc_error(DEV) == 0


def test_linear_falls_back_where_tensor_cores_do_not_apply():
    from llaisys_b200 import kernels
    x, w, _ = _tc_case(5, 40, 36, 1)             # K = 36 is no multiple of 8
    want = plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy())
    _tc_check(kernels.linear(x, w, out_dtype=torch.float32), want, 36)


@pytest.mark.parametrize("nh,nkvh,dh,window", [(12, 2, 128, None), (6, 1, 48, 70), (40, 1, 16, 129), (4, 4, 64, 3)])
@pytest.mark.parametrize("splits", [1, 5, 13, 16])
def test_attention_decode_fused_rotation_and_append(nh, nkvh, dh, window, splits):
    """The tensor-core decode kernel can rotate the query and the new key and append to the cache
    itself; that must give what the separate rotation/append kernel followed by attention gives,
    in the output and in the cache."""
    from llaisys_b200 import kernels
    from llaisys_b200.config import PartSpec
    from llaisys_b200.parts import BuildEnv, build_part
    dtype = torch.bfloat16
    lens_before, news = [0, 129, 63, 64, 500], [1, 1, 1, 1, 1]
    d, _ = _attention_case(dtype, nh, nkvh, dh, lens_before, news, window, seed=nh + dh + splits)
    rope = build_part("position", PartSpec("rope_half_split", {"head_dim": dh, "theta": 1e4}), BuildEnv(dtype, torch.device(DEV)))
    cos, sin = rope.table(600)
    width = d["table"].shape[1]
    args = lambda q, k, v: (q, nh, nkvh, dh, k, v, d["table"], width, d["seq_start"], d["len_before"], 5, window, 1 / math.sqrt(dh))
    # separate kernels
    q1, k1, v1 = d["qkv"].clone(), d["kpool"].clone(), d["vpool"].clone()
    tok = torch.arange(5, dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.rope_append(q1, nh, nkvh, dh, cos=cos, sin=sin, tok_pos=d["len_before"], err=err, append=dict(
        tok_seq=tok, seq_start=d["seq_start"], seq_len_before=d["len_before"], kpool=k1, vpool=v1,
        page_table=d["table"], ring=width))
    want = kernels.attention_decode(*args(q1, k1, v1), n_splits=splits)
    # one kernel
    q2, k2, v2 = d["qkv"].clone(), d["kpool"].clone(), d["vpool"].clone()
    got = kernels.attention_decode(*args(q2, k2, v2), n_splits=splits, rope=(cos, sin), append_new=True)
    assert torch.equal(q2, d["qkv"])                                   # the projections are left as they were
    assert torch.isfinite(got).all() and float((got.float() - want.float()).abs().max()) <= 2.0 ** -7 * float(want.float().abs().max())
    written = torch.isfinite(k1)                                       # untouched rows of the test pool are NaN
    assert torch.equal(written, torch.isfinite(k2)) and torch.equal(k1[written], k2[written])
    assert torch.equal(torch.isfinite(v1), torch.isfinite(v2)) and torch.equal(v1[torch.isfinite(v1)], v2[torch.isfinite(v2)])
    # the same kernel twice more: the counters of the slice merge must be back at zero
    got2 = kernels.attention_decode(*args(q1, k1, v1), n_splits=splits)
    assert torch.equal(got2, want)


@pytest.mark.parametrize("nh,nkvh,dh,window", [(4, 2, 64, None), (12, 2, 128, None), (3, 3, 64, 70), (8, 1, 128, 5), (2, 1, 128, 200)])
def test_attention_prefill_from_cache_tcgen05(nh, nkvh, dh, window):
    """Prefill attention with every key read from the cache (the tcgen05 kernel for head sizes 64
    and 128): sequences of unequal lengths, some with cached history, against the plain formula."""
    from llaisys_b200 import kernels
    dtype = torch.bfloat16
    lens_before, news = [0, 130, 64, 5, 0], [100, 37, 1, 200, 300]
    d, want = _attention_case(dtype, nh, nkvh, dh, lens_before, news, window, seed=nh * dh + 1)
    T = sum(news)
    tok_seq = torch.tensor(np.repeat(np.arange(5), news), dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(np.concatenate([np.arange(l, l + n) for l, n in zip(lens_before, news)]), dtype=torch.int32, device=DEV)
    width = d["table"].shape[1]
    kernels.rope_append(d["qkv"], nh, nkvh, dh, tok_pos=tok_pos, err=torch.zeros(1, dtype=torch.int32, device=DEV), append=dict(
        tok_seq=tok_seq, seq_start=d["seq_start"], seq_len_before=d["len_before"], kpool=d["kpool"], vpool=d["vpool"],
        page_table=d["table"], ring=width))
    args = (d["qkv"], nh, nkvh, dh, d["kpool"], d["vpool"], d["table"], width, d["seq_start"], d["len_before"], 5, max(news),
            window, 1 / math.sqrt(dh))
    got = kernels.attention_prefill(*args, all_from_cache=True)
    assert kernels.tc_error(DEV) == 0
    _close(got, want, dtype, atol=6e-3)
    # every way of sharing a row block's keys among the CTAs of a cluster
    for split in (1, 2, 4):
        if dh // split >= 32:
            _close(kernels.attention_prefill(*args, all_from_cache=True, tc_split=split), want, dtype, atol=6e-3)
            assert kernels.tc_error(DEV) == 0
    # and the same through the mma.sync kernel
    kernels.ops.TC_ATTENTION = False
    try:
        _close(kernels.attention_prefill(*args, all_from_cache=True), want, dtype, atol=6e-3)
    finally:
        kernels.ops.TC_ATTENTION = True


@pytest.mark.parametrize("splits", [1, 3])
def test_a_bounded_wait_that_runs_out_is_reported_and_the_next_launch_is_right(splits, tmp_path):
    """A test build of the tensor-core product (a small wait limit, and a switch that arms one stage barrier for
    sixteen bytes that nothing ever brings: no fault, no copy left in flight) makes the issuing thread's wait run
    out.  The block must record its code, free its tensor memory and return; the tile counters must be back at
    zero; Engine.check() must raise; and the launches that follow must be right.  The code is 101 (the wait for a
    full stage) or, where the K range is longer than the ring, 102 (the copying thread's wait for the same stage to
    be freed, which starves with it): whichever of the two runs out first reports, the other sees the flag and leaves."""
    from ctypes import c_int, c_longlong, c_void_p
    from helpers import TINY_A, build_engine, make_folder
    from llaisys_b200 import kernels
    from llaisys_b200.csrc.build import load_module
    from llaisys_b200.engine import StepError
    from llaisys_b200.kernels import ops
    lib = load_module("gemm_tc.cu", {"LLB_WAIT_LIMIT": 4096, "LLB_TEST_STALL": 1})
    f = lib.llb_gemm_tc
    f.restype = c_int
    f.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                  c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p]
    T, N, K = 8, 300, 1096
    x, w, b = _tc_case(T, N, K, 77, bias=torch.float32)
    want = plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy(), b.double().cpu().numpy())
    scratch, counters, err = ops._tc_resources(torch.device(DEV))
    engine = build_engine(make_folder(tmp_path, TINY_A, 0), torch.bfloat16, max_tokens=64)

    def launch():
        out = torch.zeros((T, N), dtype=torch.float32, device=DEV)
        rc = f(x.data_ptr(), w.data_ptr(), b.data_ptr(), 0, out.data_ptr(), 0, T, N, K, x.stride(0), out.stride(0), 16, splits, 0, 0,
               scratch.data_ptr(), scratch.numel(), counters.data_ptr(), counters.numel(), err.data_ptr(),
               torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        return out

    assert kernels.tc_error(DEV) == 0
    _tc_check(launch(), want, K)                       # the test build is the same kernel when the switch is off
    err.fill_(-7)                                      # the switch: this launch's first stage never fills
    launch()
    code = kernels.tc_error(DEV, clear=False)          # a wait ran out, and said so
    assert code == 101 or (code == 102 and -(-K // 64) // splits > 5)
    assert int(counters.abs().sum()) == 0              # blocks that gave up still arrived at their tile's counter
    with pytest.raises(StepError, match=str(code)):
        engine.check()
    engine.check()                                     # reported once
    _tc_check(launch(), want, K)                       # the context is whole: the same launch is right again
    _tc_check(kernels.linear(x, w, b, out_dtype=torch.float32, plan=(16, splits, 0)), want, K)
    assert kernels.tc_error(DEV) == 0


@pytest.mark.parametrize("T,H,I,stages", [(8, 1536, 8960, 0), (1, 1536, 8960, 4), (16, 1536, 8960, 10), (17, 1536, 8960, 0),
                                          (32, 256, 520, 6), (5, 144, 232, 0), (9, 64, 72, 8), (3, 3584, 18944, 0),
                                          (20, 3584, 1096, 0), (2, 5120, 640, 0)])
def test_feed_forward_in_one_launch(T, H, I, stages):
    """gate/up + SwiGLU + down + residual add as one kernel: slices of the intermediate dimension per block, the
    down projection's partial sums added to the float32 residual.  Sizes: the benchmark shapes' (one and two
    slices per block, 12 and 28 output tiles), widths that are no multiple of the tiles, both token tiles."""
    from llaisys_b200 import kernels
    rng = np.random.default_rng(T + H + I)
    x = torch.from_numpy(rng.normal(size=(T, H))).to(torch.bfloat16).to(DEV)
    gu = torch.from_numpy(rng.normal(size=(2 * I, H)) * (2.0 / math.sqrt(H))).to(torch.bfloat16).to(DEV)
    wd = torch.from_numpy(rng.normal(size=(H, I)) * (1.0 / math.sqrt(I))).to(torch.bfloat16).to(DEV)
    res0 = torch.from_numpy(rng.normal(size=(T, H))).float().to(DEV)
    if not kernels.mlp_fused_ok(x, gu, wd, res0):
        bn = 16 if T <= 16 else 32
        assert 2 * bn + -(-H // 128) * bn > 512          # refused only where tensor memory cannot hold the accumulators
        return
    pre = plain.linear(x.double().cpu().numpy(), gu.double().cpu().numpy())
    act = torch.from_numpy(plain.swiglu(pre[:, :I], pre[:, I:])).to(torch.bfloat16).double().numpy()      # the kernel rounds it once too
    want = res0.double().cpu().numpy() + plain.linear(act, wd.double().cpu().numpy())
    for turn in range(2):
        res = res0.clone()
        kernels.mlp_fused(x, gu, wd, res, stages=stages)
        torch.cuda.synchronize()
        got = res.double().cpu().numpy()
        # float32 sums of bfloat16 products; an activation next to a rounding boundary may round the other way
        bound = 2e-3 * math.sqrt(I / 64) * float(np.abs(want - res0.double().cpu().numpy()).std()) + 1e-4 + 1e-5 * np.abs(want)
        err = np.abs(got - want)
        assert np.isfinite(got).all() and (err <= bound).all(), f"turn {turn}: worst {err.max():.3e} against {bound.min():.3e}"
    assert kernels.tc_error(DEV) == 0
    # and the unfused pair of launches agrees (its output is rounded to bfloat16 before the add)
    two = kernels.linear(kernels.linear_swiglu(x, gu), wd).float() + res0
    assert float((two - res).abs().max()) <= 2.0 ** -7 * float((res - res0).abs().max()) + 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_weights_are_the_same_numbers_on_the_device_and_on_the_host(dtype):
    """The device kernel and its numpy twin perform the same IEEE operations in the same order: a tensor made on
    the GPU (what the benchmark's 3 GB of weights are) equals the tensor that write_random_model puts in a file."""
    from llaisys_b200 import kernels
    from llaisys_b200.parts import TensorDecl
    from llaisys_b200.weights import RandomSource
    from llaisys_b200.weights.rng import normal, tensor_key
    decls = {"model.layers.3.mlp.up_proj.weight": TensorDecl((301, 517)), "n.weight": TensorDecl((1000,), init="one_plus_normal", use="vector")}
    host, dev = RandomSource(decls, 7, dtype), RandomSource(decls, 7, dtype, device=DEV)
    for name in decls:
        a, b = host.get(name), dev.get(name)
        assert b.is_cuda and b.dtype == dtype and torch.equal(a, b.cpu()), name
    # a piece in the middle of a long tensor, and the far tails of the distribution
    key = tensor_key(7, "big")
    out = torch.empty(4096, dtype=torch.float32, device=DEV)
    kernels.fill_normal(out, key, 0.0, 1.0, first=3_000_000_000)
    assert np.array_equal(out.cpu().numpy(), normal(key, 4096, first=3_000_000_000))
    big = torch.empty(1 << 22, dtype=torch.float32, device=DEV)
    kernels.fill_normal(big, key, 0.0, 1.0)
    assert abs(float(big.mean())) < 2e-3 and abs(float(big.std()) - 1) < 2e-3 and float(big.abs().max()) > 4.5
    assert np.array_equal(big[-100000:].cpu().numpy(), normal(key, 100000, first=(1 << 22) - 100000))


@pytest.mark.parametrize("T,N,K,ksplit", [(2048, 1536, 1536, 0), (2048, 1536, 8960, 0), (300, 520, 1096, 3), (700, 200, 72, 1),
                                          (257, 1536, 8960, 4), (1000, 3584, 512, 2),
                                          (8, 1536, 1536, 0), (1, 1536, 8960, 0), (64, 1536, 8960, 0), (64, 1536, 1536, 5), (20, 144, 200, 0),
                                          (100, 300, 1096, 7), (200, 520, 72, 0), (33, 3584, 3584, 1)])
def test_linear_into_the_residual_stream_on_paired_sms(T, N, K, ksplit):
    """A projection that ends in the residual add: K ranges of a tile as separate units (of the paired-SM kernel above
    256 tokens, blocks of the one-CTA kernel up to there), their partial tiles added to the float32 stream by TMA
    reductions."""
    from llaisys_b200 import kernels
    x, w, b = _tc_case(T, N, K, T + N + K, bias=torch.bfloat16)
    rng = np.random.default_rng(3)
    s0 = torch.from_numpy(rng.normal(size=(T, N))).float().to(DEV)
    prod = plain.linear(x.double().cpu().numpy(), w.double().cpu().numpy())
    for bias in (b, None):
        stream = s0.clone()
        assert kernels.linear_into_ok(x, w, bias, stream)
        for turn in range(2):                                    # adding twice adds twice
            kernels.linear_into(x, w, bias, stream, ksplit=ksplit)
        torch.cuda.synchronize()
        want = s0.double().cpu().numpy() + 2 * (prod + (b.double().cpu().numpy() if bias is not None else 0.0))
        _tc_check(stream, want, 4 * K)
    assert kernels.tc_error(DEV) == 0


def test_stamped_build_gives_the_same_product_and_ordered_stamps(monkeypatch):
    """A build with cycle stamps (the tool behind `bench.py --stamps`) is the same kernel: equal results, and the
    stamps that one thread of a block takes rise in the order of their places."""
    from llaisys_b200 import kernels
    from llaisys_b200.kernels import ops
    x, w, b = _tc_case(8, 2048, 1536, 5, bias=torch.bfloat16)
    plain_out = kernels.linear(x, w, b)
    monkeypatch.setattr(ops, "_STAMPS", {"LLB_STAMPS": 1})
    bn, splits = ops.tc_plan(8, 2048, 1536, ops._sm_count(DEV))
    blocks = 16 * splits
    buf = torch.zeros((blocks, 16), dtype=torch.int64, device=DEV)
    with pytest.raises(kernels.KernelError):
        ops.set_stamps("mlp_tc.cu", buf)                      # no stamped build of that module is loaded
    out0 = kernels.linear(x, w, b)                            # loads the stamped build; stamps still off
    ops.set_stamps("gemm_tc.cu", buf, blocks)
    out1 = kernels.linear(x, w, b)
    kernels.linear(x[:, :512].contiguous(), w[:, :512].contiguous(), b)      # another grid: leaves the stamps alone
    torch.cuda.synchronize()
    ops.set_stamps("gemm_tc.cu", None)
    st = buf.cpu().numpy()
    kernels.linear(x, w, b)
    torch.cuda.synchronize()
    assert torch.equal(out0, plain_out) and torch.equal(out1, plain_out)
    assert (st[:, :8] > 0).all()
    # places stamped by one and the same thread come in order: the epilogue's thread (0, 1, 4, 5, 6, 7), the issuing lane (2, 3)
    assert (np.diff(st[:, [0, 1, 4, 5, 6, 7]], axis=1) > 0).all() and (st[:, 3] > st[:, 2]).all()
    assert np.array_equal(buf.cpu().numpy(), st)              # switched off: nothing is written any more
    assert kernels.tc_error(DEV) == 0
