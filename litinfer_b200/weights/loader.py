"""Weights by tensor name, checked against what the model's parts declare.

Every part lists its tensors as :class:`ParamSpec` (full name, shape, role).
The loader reads the folder's ``*.safetensors`` files in sorted order (as
python/llaisys/models/qwen2.py:133 does), compares names and shapes with the
declaration and raises **one** :class:`WeightError` that lists everything that
is missing, unexpected or of the wrong shape.  LitInfer checks names only, and
on every forward (src/llaisys/models/qwen2.cpp:53-92); here it happens once.

How a tensor is held on the device, by role:

* ``matrix``: operand of a matrix product or the embedding table: the run
  dtype (bfloat16, or float32 on the 32-bit path);
* ``vector``: norm weights and biases, consumed inside 32-bit arithmetic:
  always float32, so a tensor stored in 32-bit stays so and one stored in
  16 bits is widened without loss;
* ``table``: integer tables: int32;
* ``keep``: as stored (float32 stays float32), for state-like constants.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import iter_tensors, read_header


class WeightError(RuntimeError):
    """Raised once per load, with every problem found."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        parts = []
        if self.missing:
            parts.append(f"missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            parts.append(f"unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            parts.append(
                f"wrong shapes ({len(self.wrong_shape)}): "
                + ", ".join(f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape)
            )
        if self.wrong_dtype:
            parts.append(
                f"wrong kinds ({len(self.wrong_dtype)}): "
                + ", ".join(f"{n} is stored as {got}, expected {want}" for n, got, want in self.wrong_dtype)
            )
        super().__init__("model weights do not match the configuration: " + "; ".join(parts))


@dataclass(frozen=True)
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"            # matrix | vector | table | keep
    init: str = "normal"            # normal | ones_normal | zeros | randint
    std: float = 0.02
    optional: bool = False          # the file may lack it (the part then does without)
    aliases: Tuple[str, ...] = ()   # other names it may be stored under, tried in order after ``name``
    draw: bool = True               # whether random-weights mode makes one (an optional tensor may say no)

    def device_dtype(self, run_dtype: torch.dtype, stored: Optional[torch.dtype] = None) -> torch.dtype:
        if self.role == "matrix":
            return run_dtype
        if self.role == "vector":
            return torch.float32
        if self.role == "table":
            return torch.int32
        if self.role == "keep":
            return stored if stored is not None else torch.float32
        raise ValueError(f"unknown role {self.role!r} of tensor {self.name}")


_FLOAT_NAMES = {"F64", "F32", "F16", "BF16"}


def safetensors_files(model_dir) -> List[Path]:
    files = sorted(Path(model_dir).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors file in {model_dir}")
    return files


def check_against(params: Sequence[ParamSpec], stored: Dict[str, dict]) -> Dict[str, str]:
    """Compare the declaration with a header; returns declared name -> stored name."""
    resolve: Dict[str, str] = {}
    missing, wrong_shape, wrong_dtype = [], [], []
    claimed = set()
    for p in params:
        found = next((n for n in (p.name,) + p.aliases if n in stored), None)
        if found is None:
            if not p.optional:
                missing.append(p.name)
            continue
        claimed.add(found)
        info = stored[found]
        if tuple(info["shape"]) != tuple(p.shape):
            wrong_shape.append((found, tuple(info["shape"]), tuple(p.shape)))
        is_float = info["dtype"] in _FLOAT_NAMES
        if p.role == "table" and is_float:
            wrong_dtype.append((found, info["dtype"], "an integer type"))
        elif p.role in ("matrix", "vector") and not is_float:
            wrong_dtype.append((found, info["dtype"], "a floating-point type"))
        resolve[p.name] = found
    unexpected = sorted(n for n in stored if n not in claimed)
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)
    return resolve


def load_tensors(model_dir, params: Sequence[ParamSpec], run_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """All declared tensors on ``device``, keyed by declared name."""
    files = safetensors_files(model_dir)
    stored: Dict[str, dict] = {}
    where: Dict[str, Path] = {}
    for f in files:
        header, _ = read_header(f)
        for n, info in header.items():
            stored[n] = info
            where[n] = f
    resolve = check_against(params, stored)
    by_stored = {resolve[p.name]: p for p in params if p.name in resolve}
    out: Dict[str, torch.Tensor] = {}
    for f in files:
        wanted = {n for n in by_stored if where[n] == f}
        if not wanted:
            continue
        for n, t in iter_tensors(f, wanted):
            p = by_stored[n]
            out[p.name] = t.to(device=device, dtype=p.device_dtype(run_dtype, t.dtype)).contiguous()
    return out
