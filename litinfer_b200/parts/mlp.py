"""Dense SwiGLU feed-forward: down(up(h) * silu(gate(h))), no biases
(src/llaisys/models/qwen2.cpp:744-759; src/ops/swiglu/op.cpp:17-23, silu as
g / (1 + exp(-g))).  gate and up are one fused product; the activation is
computed in float32 and rounded once; in bfloat16 it is the epilogue of that product."""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import FEED_FORWARDS, FeedForward
from .linear import FusedLinear, GateUpLinear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    takes_deferred = True            # the gate|up product applies the factor

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        names = spec.get("names", {})
        self.gate_up = GateUpLinear(prefix, names.get("gate", "gate_proj"), names.get("up", "up_proj"), self.hidden,
                                    self.intermediate, dtype)
        self.down = FusedLinear(prefix, [names.get("down", "down_proj")], self.intermediate, [self.hidden], False, dtype)

    def params(self) -> List[ParamSpec]:
        return self.gate_up.params() + self.down.params()

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gate_up.bind(tensors)
        self.down.bind(tensors)

    def fused_decode(self):
        if type(self) is not SwiGLU or not self.gate_up.fused_activation or self.down.bias is not None:
            return None
        return {"w_gate_up": self.gate_up.weight, "w_down": self.down.weight, "hidden": self.hidden, "intermediate": self.intermediate}

    def forward(self, h, ctx):
        return self.down(self.gate_up.activation(h))

    def forward_into(self, h, ctx, tail):
        return tail.apply_linear(self.down, self.gate_up.activation(h))
