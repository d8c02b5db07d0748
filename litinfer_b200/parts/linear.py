"""Linear map out = x W^T (+ b) with W stored [out, in], as LitInfer's linear
op reads it (src/ops/linear/cpu/linear_cpu.cpp:45-60): accumulation in
float32, bias added in float32, one rounding.  Several maps of the same input
can be declared under their own tensor names and fused into one matrix when
the weights are bound (q|k|v, gate|up), so that one product serves them."""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import Deferred


def undefer(x, weight: torch.Tensor):
    """(input tensor, row_scale) for a product over ``x``: a deferred activation keeps its factor for the product if
    the product's kernel takes one, else it is multiplied out first."""
    if not isinstance(x, Deferred):
        return x, None
    if K.linear_scaled_accepts(x.h, weight, x.h):
        return x.h, x.row_scale
    return x.materialize(), None


class FusedLinear:
    """``names``: tensor-name stems (without .weight / .bias); ``outs``: their output sizes.
    ``bias``: True (each map has one), False (none), or None: the biases follow the file, each map on
    its own; a map without one counts as zeros when another has one."""

    def __init__(self, prefix: str, names: Sequence[str], in_features: int, outs: Sequence[int], bias: Optional[bool],
                 dtype: torch.dtype, std: float = 0.02) -> None:
        self.prefix = prefix
        self.names = list(names)
        self.in_features = int(in_features)
        self.outs = [int(o) for o in outs]
        self.out_features = sum(self.outs)
        self.has_bias = bool(bias) or bias is None          # declared; with None the file decides when bound
        self.bias_optional = bias is None
        self.dtype = dtype
        self.std = std
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def params(self) -> List[ParamSpec]:
        out = []
        for n, o in zip(self.names, self.outs):
            out.append(ParamSpec(f"{self.prefix}{n}.weight", (o, self.in_features), role="matrix", std=self.std))
            if self.has_bias:
                out.append(ParamSpec(f"{self.prefix}{n}.bias", (o,), role="vector", std=self.std, optional=self.bias_optional))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        ws = [tensors.pop(f"{self.prefix}{n}.weight") for n in self.names]
        self.weight = ws[0] if len(ws) == 1 else torch.cat(ws, dim=0).contiguous()
        del ws
        if self.has_bias:
            bs = [tensors.pop(f"{self.prefix}{n}.bias", None) if self.bias_optional else tensors.pop(f"{self.prefix}{n}.bias")
                  for n in self.names]
            if all(b is None for b in bs):
                self.bias = None
            else:
                like = next(b for b in bs if b is not None)
                bs = [b if b is not None else torch.zeros(o, dtype=like.dtype, device=like.device) for b, o in zip(bs, self.outs)]
                self.bias = bs[0] if len(bs) == 1 else torch.cat(bs, dim=0).contiguous()

    def __call__(self, x, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``x`` may be a :class:`~litinfer_b200.parts.base.Deferred` activation: its factor per token goes on the product."""
        x, row_scale = undefer(x, self.weight)
        out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or self.dtype, device=x.device)
        K.linear(x, self.weight, self.bias, out, row_scale=row_scale)
        return out


class GateUpLinear(FusedLinear):
    """gate and up maps of a gated feed-forward.  In bfloat16, with sizes that are multiples of
    8, the two matrices are interleaved in groups of 8 rows when bound and the product's
    epilogue applies up * silu(gate), so the [tokens, 2 * intermediate] product never goes to
    memory.  Otherwise (the 32-bit path) the fused product is followed by the swiglu kernel."""

    def __init__(self, prefix, gate_name, up_name, in_features, intermediate, dtype, std=0.02):
        super().__init__(prefix, [gate_name, up_name], in_features, [intermediate, intermediate], False, dtype, std)
        self.intermediate = int(intermediate)
        self.fused_activation = dtype == torch.bfloat16 and intermediate % 8 == 0 and in_features % 8 == 0

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if not self.fused_activation:
            return super().bind(tensors)
        gate = tensors.pop(f"{self.prefix}{self.names[0]}.weight")
        up = tensors.pop(f"{self.prefix}{self.names[1]}.weight")
        self.weight = K.interleave_gate_up(gate, up)

    def activation(self, x: torch.Tensor) -> torch.Tensor:
        """up(x) * silu(gate(x)), [tokens, intermediate]."""
        if self.fused_activation:
            x, row_scale = undefer(x, self.weight)
            act = torch.empty((x.shape[0], self.intermediate), dtype=self.dtype, device=x.device)
            K.linear(x, self.weight, None, act, epilogue="swiglu", row_scale=row_scale)
        else:
            both = self(x)                                 # x may be deferred: the product multiplies its factor out
            act = torch.empty((both.shape[0], self.intermediate), dtype=self.dtype, device=both.device)
            K.swiglu(both, act)
        return act
