"""Random-weights mode: tensors from a declaration and a seed, and a model
folder (config.json, model.safetensors) written from a configuration.

LitInfer has no such mode.  Distributions: matrices and biases N(0, std) with
the declared std (0.02 unless a part says otherwise), norm weights
1 + N(0, 0.1), so that a wrong norm weight or bias shows in the logits.  Each
tensor has its own stream keyed on (seed, tensor name): the values of one
tensor do not depend on which other tensors exist or in which order they are
drawn.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Iterable, Sequence

import torch

from .loader import ParamSpec
from .safetensors_io import write_file

_STORE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(p: ParamSpec, seed: int, device="cpu", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed(_tensor_seed(seed, p.name))
    if p.init == "zeros":
        return torch.zeros(p.shape, dtype=dtype, device=dev)
    if p.init == "randint":
        return torch.randint(0, 2**15, p.shape, generator=g, device=dev, dtype=torch.int32)
    # drawn in float32 in slabs, so that a large tensor never holds two float32 copies
    out = torch.empty(p.shape, dtype=dtype, device=dev)
    flat = out.view(-1)
    slab = 1 << 26
    for lo in range(0, flat.numel(), slab):
        n = min(slab, flat.numel() - lo)
        x = torch.randn(n, generator=g, device=dev, dtype=torch.float32)
        if p.init == "normal":
            x.mul_(p.std)
        elif p.init == "ones_normal":
            x.mul_(0.1).add_(1.0)
        else:
            raise ValueError(f"unknown init {p.init!r} of tensor {p.name}")
        flat[lo:lo + n] = x.to(dtype)
    return out


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
