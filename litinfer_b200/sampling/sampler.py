"""Choosing the next token: greedy, temperature, top-k, top-p.

Which tokens stay candidates follows LitInfer's sampler
(src/llaisys/models/qwen2.cpp:890-920): logits / temperature; the ``top_k``
largest if 0 < k < vocab; softmax over those; the shortest prefix (in
descending order) whose cumulative probability reaches ``top_p`` if
0 < p < 1; softmax again over what is left; draw.  Greedy when ``top_k == 1``
(the default of ``generate``, python/llaisys/models/qwen2.py:305-311) or when
``temperature <= 0`` (qwen2.cpp:893-895): the first maximum wins
(src/ops/argmax/op.cpp:28-33).

The draw differs from LitInfer's on purpose.  LitInfer consumes one shared
``mt19937`` in batch order, so a request's tokens depend on what else is
running.  Here the draw is Gumbel-max, ``argmax_i(z_i + g_i)`` over the
candidates with ``g_i = -log(-log(u_i))``, which samples exactly from their
softmax, and ``u_i`` comes from a counter-based generator keyed on (the
request's seed, the index of the output token, the token id i): the result
depends on nothing but the request itself.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np
import torch

from .. import kernels as K


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 1
    top_p: float = 1.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.top_k == 1 or self.temperature <= 0.0


class Sampler:
    """Device-side sampling of one token per logits row."""

    def __init__(self, device) -> None:
        self.device = torch.device(device)
        # the rows' parameters go to the device through pinned memory, without blocking the host (two buffers in turn:
        # a step may be launched before the one before it has been read)
        self._pinned: List[torch.Tensor] = []
        self._on_device: List[torch.Tensor] = []
        self._copied: List = []
        self._turn = 0

    def _upload(self, packed: np.ndarray) -> torch.Tensor:
        if self.device.type != "cuda":
            return torch.from_numpy(packed.copy())
        R = packed.shape[0]
        if not self._pinned or self._pinned[0].shape[0] < R:
            for ev in self._copied:
                ev.synchronize()
            cap = max(64, 2 * R)
            self._pinned = [torch.empty((cap, 6), dtype=torch.int32).pin_memory() for _ in range(2)]
            self._on_device = [torch.empty((cap, 6), dtype=torch.int32, device=self.device) for _ in range(2)]
            self._copied = [torch.cuda.Event() for _ in range(2)]
            for ev in self._copied:
                ev.record(torch.cuda.current_stream(self.device))
        t = self._turn
        self._turn ^= 1
        self._copied[t].synchronize()                     # the copy that last used this pinned buffer has finished
        self._pinned[t].numpy()[:R] = packed
        dst = self._on_device[t][:R]
        dst.copy_(self._pinned[t][:R], non_blocking=True)
        self._copied[t].record(torch.cuda.current_stream(self.device))
        return dst

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], output_index: Sequence[int]) -> torch.Tensor:
        """``logits`` float32 [R, V]; returns int32 [R] on the device."""
        R = logits.shape[0]
        if len(params) != R or len(output_index) != R:
            raise ValueError("one SamplingParams and one output index per logits row")
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
        if R == 0:
            return out
        if all(p.greedy for p in params):
            K.argmax(logits, out)
            return out
        # rows that are greedy get temperature 0, which the kernel reads as argmax
        packed = np.empty((R, 6), dtype=np.int32)
        as_float = packed.view(np.float32)
        as_float[:, 0] = [0.0 if p.greedy else float(p.temperature) for p in params]
        packed[:, 1] = [min(max(int(p.top_k), -1), 2**31 - 1) for p in params]
        as_float[:, 2] = [float(p.top_p) for p in params]
        seeds = np.array([int(p.seed) & 0xFFFF_FFFF_FFFF_FFFF for p in params], dtype=np.uint64)
        packed[:, 3] = (seeds & np.uint64(0xFFFF_FFFF)).astype(np.uint32).view(np.int32)
        packed[:, 4] = (seeds >> np.uint64(32)).astype(np.uint32).view(np.int32)
        packed[:, 5] = [int(i) for i in output_index]
        K.sample(logits, self._upload(packed), out)
        return out


def _as_i32(u: int) -> int:
    return u - (1 << 32) if u >= (1 << 31) else u
