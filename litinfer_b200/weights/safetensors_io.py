"""Reader and writer of the safetensors container, without any library.

Layout (as LitInfer's loader reads it, python/llaisys/models/qwen2.py:112-129):
8 bytes little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets"}}`` (``__metadata__`` skipped),
then the tensors' bytes.  The file is memory-mapped and each tensor is copied
out before the mapping closes, so 32-bit and 16-bit files load alike
(LitInfer's reader fails on F32 files because a view outlives the mapping).
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterator, Mapping, Tuple

import numpy as np
import torch

_TO_TORCH = {
    "F64": (np.float64, torch.float64),
    "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16),
    "BF16": (np.uint16, torch.bfloat16),
    "I64": (np.int64, torch.int64),
    "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16),
    "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8),
    "BOOL": (np.bool_, torch.bool),
}
_FROM_TORCH = {
    torch.float64: "F64",
    torch.float32: "F32",
    torch.float16: "F16",
    torch.bfloat16: "BF16",
    torch.int64: "I64",
    torch.int32: "I32",
    torch.int16: "I16",
    torch.int8: "I8",
    torch.uint8: "U8",
    torch.bool: "BOOL",
}


class SafetensorsError(ValueError):
    pass


def read_header(path) -> Tuple[Dict[str, dict], int]:
    """The JSON header (without ``__metadata__``) and the offset of the data."""
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors file")
        (hlen,) = struct.unpack("<Q", raw)
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
    header.pop("__metadata__", None)
    data_size = size - 8 - hlen
    for name, info in header.items():
        if info.get("dtype") not in _TO_TORCH:
            raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {info.get('dtype')!r}")
        lo, hi = info["data_offsets"]
        numel = int(np.prod(info["shape"], dtype=np.int64)) if info["shape"] else 1
        itemsize = np.dtype(_TO_TORCH[info["dtype"]][0]).itemsize
        if not (0 <= lo <= hi <= data_size) or hi - lo != numel * itemsize:
            raise SafetensorsError(f"{path}: tensor '{name}' has data_offsets {lo}:{hi} that do not match shape {info['shape']}")
    return header, 8 + hlen


def iter_tensors(path, names=None) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yield (name, CPU tensor) for every tensor (or those in ``names``); each is a copy."""
    path = Path(path)
    header, base = read_header(path)
    with open(path, "rb") as f, mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) as mm:
        for name, info in header.items():
            if names is not None and name not in names:
                continue
            np_dtype, torch_dtype = _TO_TORCH[info["dtype"]]
            lo, hi = info["data_offsets"]
            arr = np.frombuffer(mm, dtype=np_dtype, count=(hi - lo) // np.dtype(np_dtype).itemsize, offset=base + lo).copy()
            t = torch.from_numpy(arr)
            if torch_dtype == torch.bfloat16:
                t = t.view(torch.bfloat16)
            yield name, t.reshape(info["shape"])
            del arr


def write_file(path, tensors: Mapping[str, torch.Tensor]) -> None:
    """Write ``tensors`` (CPU or device) as one safetensors file, in the mapping's order."""
    header, off = {}, 0
    for name, t in tensors.items():
        if t.dtype not in _FROM_TORCH:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _FROM_TORCH[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name, t in tensors.items():
            c = t.detach().contiguous().cpu()
            if c.dtype == torch.bfloat16:
                c = c.view(torch.int16)
            f.write(c.numpy().tobytes())
