"""The library's own random numbers for random weights: a counter-based generator whose
element ``i`` of tensor ``name`` under ``seed`` is one fixed number, whoever computes it.

The host (this file, NumPy) and the device (``csrc/random_fill.cu``) run the same
arithmetic, and only operations that IEEE 754 rounds correctly (add, multiply, divide,
square root, integer work), each on its own (the device code uses the explicitly rounded
intrinsics, so nothing is contracted into a fused multiply-add). The two therefore agree
bit for bit, which lets a model of any size that was drawn on the device be spot-checked on
the CPU. The reference has random weights only in tests, from a linear congruential
generator written out there (src/cuda_resident/tests.rs:537-553, norms at :217-224).

    key   = splitmix64(fnv1a64(name) ^ splitmix64(seed))
    z     = splitmix64(key + (i + 1) * 0x9E3779B97F4A7C15)          (wrapping, 64 bits)
    u1    = ((z >> 32) + 1) / 2^32 in (0, 1],  angle = 2 pi (z & 0xffffffff) / 2^32
    value = float32(mean + std * sqrt(-2 ln u1) * cos(angle))        (Box-Muller)

``ln`` is (e - 32) ln 2 + 2 s (1 + s^2/3 + ... + s^20/21) with the mantissa brought into
[sqrt(1/2), sqrt(2)) and s = (m - 1) / (m + 1); the cosine is folded into an eighth of
the circle by the top three bits of the angle and evaluated by the Taylor polynomials of
sine and cosine up to t^17; both are exact to about 1e-16, far below the float32 result.
"""
from __future__ import annotations

import math

import numpy as np

GOLDEN = 0x9E3779B97F4A7C15
_M64 = (1 << 64) - 1
LN2 = 0.6931471805599453
SQRT_HALF = 0.7071067811865476
PI_4 = 0.7853981633974483
LOG_TERMS = [1.0 / (2 * k + 1) for k in range(11)]                  # 1, 1/3, ..., 1/21
COS_TERMS = [(-1.0) ** k / math.factorial(2 * k) for k in range(9)]         # 1, -1/2!, ..., 1/16!
SIN_TERMS = [(-1.0) ** k / math.factorial(2 * k + 1) for k in range(9)]     # 1, -1/3!, ..., 1/17!
CHUNK = 1 << 15             # elements per pass: the temporaries of a pass stay in the cache


def splitmix64(z: int) -> int:
    z &= _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def fnv1a64(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & _M64
    return h


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor: its values depend on the seed and on its own name only,
    not on which other tensors the model has."""
    return splitmix64(fnv1a64(name.encode("utf-8")) ^ splitmix64(int(seed) & _M64))


def _splitmix64_np(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _horner(terms, w: np.ndarray) -> np.ndarray:
    p = np.full_like(w, terms[-1])
    for c in reversed(terms[:-1]):
        p = p * w + c                 # two roundings: NumPy never fuses them
    return p


def standard_normals(key: int, first: int, count: int) -> np.ndarray:
    """float64 standard normal deviates of elements ``first .. first + count`` under ``key``."""
    with np.errstate(over="ignore"):
        i = np.arange(first + 1, first + count + 1, dtype=np.uint64)
        z = _splitmix64_np(np.uint64(key) + i * np.uint64(GOLDEN))
    n = (z >> np.uint64(32)).astype(np.float64) + 1.0                  # 1 .. 2^32, exact
    b = (z & np.uint64(0xFFFFFFFF)).astype(np.int64)
    mant, ex = np.frexp(n)                                             # n = mant * 2^ex, mant in [0.5, 1)
    low = mant < SQRT_HALF
    mant = np.where(low, mant * 2.0, mant)
    ex = np.where(low, ex - 1, ex).astype(np.float64)
    s = (mant - 1.0) / (mant + 1.0)
    ln_u = (ex - 32.0) * LN2 + (2.0 * s) * _horner(LOG_TERMS, s * s)
    r = np.sqrt(-2.0 * ln_u)
    octant = b >> 29
    f = (b & 0x1FFFFFFF).astype(np.float64) * (1.0 / (1 << 29))
    g = np.where(octant & 1, 1.0 - f, f)
    t = g * PI_4
    w = t * t
    cos_t = _horner(COS_TERMS, w)
    sin_t = t * _horner(SIN_TERMS, w)
    use_sin = ((octant + 1) & 2) != 0                                  # octants 1, 2, 5, 6
    negative = ((octant + 2) & 4) != 0                                 # octants 2, 3, 4, 5
    trig = np.where(use_sin, sin_t, cos_t)
    trig = np.where(negative, -trig, trig)
    return r * trig


def fill_host(key: int, first: int, count: int, mean: float, std: float) -> np.ndarray:
    """float32 values ``mean + std * normal`` of elements ``first .. first + count``."""
    out = np.empty(count, dtype=np.float32)
    for lo in range(0, count, CHUNK):
        n = min(CHUNK, count - lo)
        out[lo:lo + n] = (mean + std * standard_normals(key, first + lo, n)).astype(np.float32)
    return out
