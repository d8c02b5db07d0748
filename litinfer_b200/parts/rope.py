"""Rotary position encoding, rotate-half pairing (src/ops/rope/op.cpp:13-20, 33-39).

For pair j of the first ``rotary_dim`` elements of a head:
``phi = float(pos) / theta^(2j / rotary_dim)``, ``(a, b) = (x[j], x[j + rotary_dim/2])``,
``x'[j] = a cos(phi) - b sin(phi)``, ``x'[j + rotary_dim/2] = b cos(phi) + a sin(phi)``.
The part owns the table of denominators ``theta^(2j/rotary_dim)`` (float32);
the kernel divides the position by it and takes sine and cosine in float32.
Another frequency rule (scaled, partial) is another table or ``rotary_dim``.
"""

from __future__ import annotations

import torch

from .base import POSITIONS, Position, Rotary


@POSITIONS.register("rope")
class RotaryEmbedding(Position):
    def __init__(self, spec, prefix, dtype, device, head_dim=None):
        super().__init__(spec, prefix, dtype, device)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec.get("rotary_dim") or head_dim)
        pairing = spec.get("pairing", "half")
        if pairing != "half":
            raise ValueError(f"rope pairing '{pairing}' is not supported (rotate-half only)")
        if self.rotary_dim % 2 or (head_dim is not None and self.rotary_dim > head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")
        j = torch.arange(self.rotary_dim // 2, dtype=torch.float32)
        denom = torch.pow(torch.tensor(self.theta, dtype=torch.float32), (2.0 * j) / float(self.rotary_dim))
        self.denominators = denom.to(self.device)

    # Steps of more tokens than this get a table of cosines and sines, made once and shared by the layers (products that
    # rotate in their epilogue read it); shorter steps compute the angles where they rotate.
    TABLE_FROM_TOKENS = 65

    def fused_decode(self):
        return {"denominators": self.denominators, "rotary_dim": self.rotary_dim} if type(self) is RotaryEmbedding else None

    def rotary(self, ctx) -> Rotary:
        return Rotary(self.denominators, self.rotary_dim, self.table(ctx))

    def table(self, ctx):
        """``[tokens, rotary_dim / 2, 2]`` float32 cos and sin of this step's positions, or None for a short step."""
        if ctx.num_tokens < self.TABLE_FROM_TOKENS or self.dtype != torch.bfloat16:
            return None
        key = ("rope_table", self.theta, self.rotary_dim)
        t = ctx.scratch.get(key)
        if t is None:
            from .. import kernels as K

            t = torch.empty((ctx.num_tokens, self.rotary_dim // 2, 2), dtype=torch.float32, device=ctx.positions.device)
            K.rope_table(ctx.positions, self.denominators, t)
            ctx.scratch[key] = t
        return t
