"""RMSNorm: y_j = w_j * x_j / sqrt(mean(x^2) + eps), per token
(src/ops/rms_norm/op.cpp:13-24).  Sum, reciprocal root and products in
float32 on the float32 residual stream; one rounding of y to the run dtype."""

from __future__ import annotations

import os
from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import NORMS, Deferred, Norm

DEFER_UP_TO = int(os.environ.get("LITINFER_B200_DEFER_UP_TO", "32"))


def defers(tokens: int) -> bool:
    """Whether the norm between two products rides on them for a step of this many tokens.  Measured (1.5B shape, a
    context of 2,048): it saves two kernels a layer and 4-9 % of the step up to 32 tokens (24 tokens 2.12 -> 2.03 ms, 32
    tokens 2.12 -> 2.04 ms); at 64 tokens the epilogues of the weight-streaming products carry too much (2.54 -> 2.78
    ms).  (Tried in the tensor-memory GEMM of prefill too: there the residual stream read and written by the epilogue's
    threads, a row each, cost more than the norm kernels it replaced.)"""
    return 0 < tokens <= DEFER_UP_TO


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec(self.prefix + "weight", (self.size,), role="vector", init="ones_normal")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors.pop(self.prefix + "weight")

    def fused_decode(self):
        return {"weight": self.weight, "eps": self.eps, "size": self.size} if type(self) is RMSNorm and self.weight is not None else None

    def forward(self, x32):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.rmsnorm(x32, self.weight, self.eps, out)
        return out

    def add_forward(self, x32, delta):
        out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
        K.add_rmsnorm(x32, delta, self.weight, self.eps, out)
        return out

    def after_linear(self, linear, a, x32, defer=False):
        # bfloat16 and a consumer that applies the reciprocal root itself: the product adds to the stream and leaves
        # weight * x with the sums of squares, all in its epilogue; this norm has no kernel of its own.
        if defer and self.dtype == torch.bfloat16 and not isinstance(a, Deferred) and defers(a.shape[0]):
            h = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
            parts = K.linear_add_scaled_parts(a, linear.weight, x32, h)
            if parts:
                ssq = torch.empty((x32.shape[0], parts), dtype=torch.float32, device=x32.device)
                K.linear_add_scaled(a, linear.weight, linear.bias, x32, self.weight, h, ssq)
                return Deferred(h, ssq, self.size, self.eps)
        return self.add_forward(x32, linear(a))

    def gather_forward(self, x32, rows):
        out = torch.empty((rows.shape[0], x32.shape[1]), dtype=self.dtype, device=x32.device)
        K.gather_rmsnorm(x32, rows, self.weight, self.eps, out)
        return out
