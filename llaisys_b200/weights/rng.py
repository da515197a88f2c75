"""Counter-based normal random numbers: element i of a tensor with 64-bit key k is a function of
(k, i) alone.  This is the host twin of csrc/random_init.cu: the same operations in the same order
in IEEE double precision (additions, multiplications, divisions and square roots only, which
round the same way everywhere), so a tensor filled on the host and the same tensor filled by the
device kernel hold the same values.  The formula is stated at the top of that file.
"""
from __future__ import annotations

import hashlib

import numpy as np

_G = np.uint64(0x9E3779B97F4A7C15)
_LN2 = np.float64(0.69314718055994530942)
_HALF_PI = np.float64(1.57079632679489661923)
_SQRT_HALF = np.float64(0.70710678118654752440)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of tensor `name` under `seed`."""
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _ln(x: np.ndarray) -> np.ndarray:
    m, e = np.frexp(x)
    small = m < _SQRT_HALF
    m = np.where(small, m * 2.0, m)
    e = np.where(small, e - 1, e).astype(np.float64)
    s = (m + (-1.0)) / (m + 1.0)
    s2 = s * s
    acc = np.full_like(s, np.float64(1.0) / np.float64(25.0))
    for k in range(23, 0, -2):
        acc = acc * s2 + np.float64(1.0) / np.float64(k)
    return e * _LN2 + (2.0 * s) * acc


def _cos_sin(t: np.ndarray):
    t2 = t * t
    ca = np.zeros_like(t)
    sa = np.zeros_like(t)
    for k in range(13, 0, -1):
        ca = (1.0 + (-ca)) * (t2 / np.float64((2 * k - 1) * (2 * k)))
        sa = (1.0 + (-sa)) * (t2 / np.float64((2 * k) * (2 * k + 1)))
    return 1.0 + (-ca), t * (1.0 + (-sa))


def normal(key: int, n: int, first: int = 0, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    """float32 values of elements first .. first + n - 1 of the tensor with key `key`."""
    out = np.empty(n, dtype=np.float32)
    with np.errstate(over="ignore"):
        for lo in range(0, n, 1 << 20):
            hi = min(n, lo + (1 << 20))
            i = np.arange(first + lo, first + hi, dtype=np.uint64)
            k = np.uint64(key & 0xFFFFFFFFFFFFFFFF)
            b1 = _mix64(k + (np.uint64(2) * i + np.uint64(1)) * _G) >> np.uint64(11)
            b2 = _mix64(k + (np.uint64(2) * i + np.uint64(2)) * _G) >> np.uint64(11)
            u1 = (b1.astype(np.float64) + 0.5) * np.float64(1.1102230246251565e-16)
            quadrant = (b2 >> np.uint64(51)).astype(np.int64)
            frac = (b2 & np.uint64((1 << 51) - 1)).astype(np.float64) * np.float64(4.440892098500626e-16)
            c, s = _cos_sin(frac * _HALF_PI)
            cosv = np.choose(quadrant, [c, -s, -c, s])
            r = np.sqrt(-2.0 * _ln(u1))
            out[lo:hi] = (np.float64(mean) + np.float64(std) * (r * cosv)).astype(np.float32)
    return out
