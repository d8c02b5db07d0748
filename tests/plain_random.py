"""Plain restatement of the random-weights generator, one element at a time.

The recipe (litinfer_b200/csrc/fill_random.cu states it; LitInfer itself has no random
mode): pair p of a tensor draws z = mix(key + (p + 1) * 0x9E3779B97F4A7C15) with the
finaliser of splitmix64; k = top 24 bits + 1, j = the next 24 bits;
r = sqrt(-2 ln(k / 2^24)); elements 2p and 2p + 1 are mean + std * r * cos(2 pi j / 2^24)
and the same with sin.  Logarithm, sine and cosine are series of single float32
operations.  Written with Python integers and NumPy float32 scalars, sharing no code
with the package.
"""

from __future__ import annotations

import hashlib
import math

import numpy as np

F = np.float32
MASK = (1 << 64) - 1


def tensor_key(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def mix64(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


def bits(key: int, counter: int) -> int:
    return mix64((key + (counter + 1) * 0x9E3779B97F4A7C15) & MASK)


def ln_u24(k: int) -> np.float32:
    e = k.bit_length() - 1
    m = F(k) * F(2.0 ** -e)
    t = (m - F(1)) / (m + F(1))
    t2 = t * t
    s = F(1) / F(11)
    for d in (9, 7, 5, 3):
        s = s * t2 + F(1) / F(d)
    s = s * t2 + F(1)
    return F(e - 24) * F(0.693147180559945309) + (F(2) * t) * s


def sincos_u24(j: int):
    q = j >> 22
    th = (F(j & 0x3FFFFF) * (F(1) / F(4194304))) * F(1.57079632679489662)
    x2 = th * th
    s = F(-1) / F(39916800)
    for c in (F(1) / F(362880), F(-1) / F(5040), F(1) / F(120), F(-1) / F(6), F(1)):
        s = s * x2 + c
    s = s * th
    c = F(1) / F(479001600)
    for d in (F(-1) / F(3628800), F(1) / F(40320), F(-1) / F(720), F(1) / F(24), F(-0.5), F(1)):
        c = c * x2 + d
    return [(s, c), (c, -s), (-s, -c), (-c, s)][q]          # (sin, cos) by quadrant


def normal(key: int, n: int, mean: float, std: float) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    for p in range((n + 1) // 2):
        z = bits(key, p)
        k, j = (z >> 40) + 1, (z >> 16) & 0xFFFFFF
        r = np.sqrt(F(-2) * ln_u24(k))
        sn, cs = sincos_u24(j)
        out[2 * p] = F(mean) + F(std) * (r * cs)
        if 2 * p + 1 < n:
            out[2 * p + 1] = F(mean) + F(std) * (r * sn)
    return out


def randint(key: int, n: int, high: int) -> np.ndarray:
    return np.asarray([(bits(key, i) >> 33) % high for i in range(n)], dtype=np.int32)


def series_errors():
    """Largest error of the three series against the library functions in float64, over a sweep."""
    worst_ln = max(abs(float(ln_u24(k)) - math.log(k / 2.0 ** 24)) for k in list(range(1, 3000)) + list(range(2 ** 24 - 3000, 2 ** 24 + 1, 7)))
    worst_sc = 0.0
    for j in range(0, 1 << 24, 4099):
        s, c = sincos_u24(j)
        a = 2 * math.pi * j / 2.0 ** 24
        worst_sc = max(worst_sc, abs(float(s) - math.sin(a)), abs(float(c) - math.cos(a)))
    return worst_ln, worst_sc
