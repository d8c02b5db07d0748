"""Random-weights mode: tensors from a declaration and a seed, and a model
folder (config.json, model.safetensors) written from a configuration.

LitInfer has no such mode (python/llaisys/models/qwen2.py:25-208 loads files
only).  Distributions: matrices and biases N(0, std) with the declared std
(0.02 unless a part says otherwise), norm weights 1 + N(0, 0.1), so that a
wrong norm weight or bias shows in the logits.

One generator serves the device and the host.  It is counter-based: element
``i`` of a tensor is a pure function of ``(key, i)`` with ``key`` made of the
seed and the tensor's name, so the values of one tensor do not depend on which
other tensors exist, in which order they are drawn, or where.  On a CUDA
device the library's own kernel fills the tensor (``csrc/fill_random.cu``:
a 28 GB model is drawn in place, without a copy from the host); on the host
the NumPy restatement below gives the same bits, because every step of the
recipe is a single IEEE float32 operation: splitmix64's finaliser on
``key + (pair + 1) * 0x9E3779B97F4A7C15``, 24 bits each for the radius and the
angle of Box-Muller, logarithm / sine / cosine as short series of additions,
multiplications and divisions, and a correctly rounded square root.  So a
model folder written on a machine without a GPU and a model drawn on the
device from the same configuration and seed hold the same weights.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Sequence

import numpy as np
import torch

from .loader import ParamSpec
from .safetensors_io import write_file

_STORE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}
_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
RANDINT_RANGE = 1 << 15


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's stream: the first 8 bytes of SHA-256 of ``"<seed>:<name>"``."""
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _bits(key: int, first: int, count: int) -> np.ndarray:
    """The 64 random bits of counters first .. first + count - 1."""
    with np.errstate(over="ignore"):
        c = np.arange(first + 1, first + count + 1, dtype=np.uint64)
        return _mix64(np.uint64(key) + c * np.uint64(_GOLDEN))


def _f(x) -> np.float32:
    return np.float32(x)


def normal_pairs(key: int, first_pair: int, pairs: int) -> np.ndarray:
    """Standard normals of the pairs first_pair .. first_pair + pairs - 1, float32 ``[pairs, 2]`` (elements 2p, 2p + 1).
    Every line is one IEEE float32 operation per element, as in ``csrc/fill_random.cu``."""
    f32 = np.float32
    z = _bits(key, first_pair, pairs)
    k = ((z >> np.uint64(40)) + np.uint64(1)).astype(f32)                      # 1 .. 2^24, exact in float32
    j = ((z >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.int32)
    del z
    # ln(k / 2^24): k = m 2^e with m in [1, 2); ln m = 2 t (1 + t^2/3 + ... + t^10/11), t = (m - 1) / (m + 1)
    m, e = np.frexp(k)                                                         # k = m 2^e, m in [0.5, 1): exact
    m *= f32(2.0)
    t = (m - f32(1.0)) / (m + f32(1.0))
    t2 = t * t
    s = np.full(pairs, f32(1.0) / f32(11.0), dtype=f32)
    for d in (9.0, 7.0, 5.0, 3.0):
        s *= t2
        s += f32(1.0) / f32(d)
    s *= t2
    s += f32(1.0)
    t *= f32(2.0)
    t *= s                                                                     # ln m
    ln = (e - 25).astype(f32)                                                  # e - 1 - 24
    ln *= f32(0.693147180559945309)
    ln += t
    ln *= f32(-2.0)
    r = np.sqrt(ln, out=ln)
    # cos and sin of 2 pi j / 2^24: quadrant from the top two bits, series on [0, pi / 2)
    q = j >> 22
    th = (j & 0x3FFFFF).astype(f32)
    th *= f32(1.0) / f32(4194304.0)
    th *= f32(1.57079632679489662)
    x2 = th * th
    sn = np.full(pairs, f32(-1.0) / f32(39916800.0), dtype=f32)
    for c in (f32(1.0) / f32(362880.0), f32(-1.0) / f32(5040.0), f32(1.0) / f32(120.0), f32(-1.0) / f32(6.0), f32(1.0)):
        sn *= x2
        sn += c
    sn *= th
    cs = np.full(pairs, f32(1.0) / f32(479001600.0), dtype=f32)
    for c in (f32(-1.0) / f32(3628800.0), f32(1.0) / f32(40320.0), f32(-1.0) / f32(720.0), f32(1.0) / f32(24.0), f32(-0.5), f32(1.0)):
        cs *= x2
        cs += c
    odd = (q & 1).astype(bool)
    cos = np.where(odd, sn, cs)                                                # quadrants: (c, s), (-s, c), (-c, -s), (s, -c)
    sin = np.where(odd, cs, sn)
    np.negative(cos, where=(q == 1) | (q == 2), out=cos)
    np.negative(sin, where=q >= 2, out=sin)
    out = np.empty((pairs, 2), dtype=f32)
    np.multiply(r, cos, out=out[:, 0])
    np.multiply(r, sin, out=out[:, 1])
    return out


def _host_normal(key: int, n: int, mean: float, std: float) -> torch.Tensor:
    from concurrent.futures import ThreadPoolExecutor
    import os

    total = (n + 1) // 2
    out = np.empty(2 * total, dtype=np.float32)
    slab = 1 << 18                                                             # pairs per round: scratch that stays in the caches

    def fill(p0: int) -> None:
        cnt = min(slab, total - p0)
        v = normal_pairs(key, p0, cnt).reshape(-1)
        v *= np.float32(std)
        v += np.float32(mean)
        out[2 * p0:2 * (p0 + cnt)] = v

    starts = range(0, total, slab)
    if len(starts) <= 2:
        for p0 in starts:
            fill(p0)
    else:                                                                      # NumPy releases the interpreter lock inside its loops
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 4)) as ex:
            list(ex.map(fill, starts))
    return torch.from_numpy(out[:n])


def _host_randint(key: int, n: int) -> torch.Tensor:
    z = _bits(key, 0, n)
    return torch.from_numpy(((z >> np.uint64(33)) % np.uint64(RANDINT_RANGE)).astype(np.int32))


def random_tensor(p: ParamSpec, seed: int, device="cpu", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """The tensor ``p`` declares, drawn from (seed, its name): on a CUDA device by the library's kernel, on the host
    by the NumPy restatement of it; the same bits either way (values are rounded to ``dtype`` from float32)."""
    dev = torch.device(device)
    if p.init == "zeros":
        return torch.zeros(p.shape, dtype=dtype, device=dev)
    key = tensor_key(seed, p.name)
    n = 1
    for d in p.shape:
        n *= int(d)
    if p.init == "randint":
        if dev.type == "cuda":
            from .. import kernels as K

            out = torch.empty(p.shape, dtype=torch.int32, device=dev)
            K.fill_randint(out, key, RANDINT_RANGE)
            return out
        return _host_randint(key, n).reshape(p.shape).to(dev)
    if p.init == "normal":
        mean, std = 0.0, float(p.std)
    elif p.init == "ones_normal":
        mean, std = 1.0, 0.1
    else:
        raise ValueError(f"unknown init {p.init!r} of tensor {p.name}")
    if dev.type == "cuda" and dtype in (torch.float32, torch.bfloat16):
        from .. import kernels as K

        out = torch.empty(p.shape, dtype=dtype, device=dev)
        K.fill_normal(out, key, mean, std)
        return out
    return _host_normal(key, n, mean, std).reshape(p.shape).to(device=dev, dtype=dtype)


def random_tensors(params: Sequence[ParamSpec], seed: int, run_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """Every declared tensor that random mode draws (``ParamSpec.draw``), on ``device`` in its device dtype."""
    return {p.name: random_tensor(p, seed, device, p.device_dtype(run_dtype)) for p in params if p.draw}


def write_model_folder(path, config, seed: int, store_dtype: str = "float32") -> Path:
    """Write config.json and model.safetensors for ``config`` (a configuration
    object of a registered architecture, or its dict) with random weights."""
    from ..config import config_from_dict
    from ..models.decoder import declared_params

    if isinstance(config, dict):
        cfg_dict = dict(config)
        config = config_from_dict(cfg_dict)
    else:
        cfg_dict = config.to_dict()
    if store_dtype not in _STORE_DTYPES:
        raise ValueError(f"store_dtype must be one of {sorted(_STORE_DTYPES)}")
    dtype = _STORE_DTYPES[store_dtype]
    cfg_dict["torch_dtype"] = store_dtype
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    params = declared_params(config.to_model_spec())
    tensors = {}
    for p in params:
        if not p.draw:
            continue
        t = random_tensor(p, seed, "cpu", torch.float32)
        if p.role == "table":
            tensors[p.name] = t.to(torch.int32)
        elif p.role == "keep":
            tensors[p.name] = t
        else:
            tensors[p.name] = t.to(dtype)
    (path / "config.json").write_text(json.dumps(cfg_dict, indent=1))
    write_file(path / "model.safetensors", tensors)
    return path
