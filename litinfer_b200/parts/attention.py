"""Grouped-query attention over a paged cache of keys and values.

Formulas (src/llaisys/models/qwen2.cpp:613-699, src/ops/paged_attention/op.cpp:194-234):
q, k, v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv; position encoding on q and k;
k (after encoding) and v go into the cache at the token's position; query
head ``i`` reads key head ``i // (heads / kv_heads)``; the query at position p
sees keys 0..p, or with a window only those with p - t < window;
scores * scale, softmax in float32, weighted sum of v; output map without
bias unless the spec says so.  Sizes, scale, window and bias flags are
parameters of the spec; the position encoding is a part of its own, named by the spec
(``position``; None: none) and asked only through :meth:`~litinfer_b200.parts.base.Position.rotary`.
``qkv_bias`` may be ``None``: the biases then follow the file, each on its own
(LitInfer's linear takes a missing bias as none, src/llaisys/ops.cc:27-29).
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import MIXERS, POSITIONS, Mixer, PagedKV
from .linear import FusedLinear, undefer


@MIXERS.register("attention")
class PagedAttention(Mixer):
    takes_deferred = True            # the q|k|v product applies the factor

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.ctas_per_work_unit = self.num_heads           # the kernel for long portions runs one CTA per head and entry
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} heads are not a multiple of {self.num_kv_heads} key/value heads")
        names = spec.get("names", {})
        self.q_dim = self.num_heads * self.head_dim
        self.kv_dim = self.num_kv_heads * self.head_dim
        self.qkv = FusedLinear(
            prefix, [names.get("q", "q_proj"), names.get("k", "k_proj"), names.get("v", "v_proj")],
            self.hidden, [self.q_dim, self.kv_dim, self.kv_dim], spec.get("qkv_bias", False), dtype)
        self.out = FusedLinear(prefix, [names.get("o", "o_proj")], self.q_dim, [self.hidden], bool(spec.get("out_bias", False)), dtype)
        position = spec.get("position")
        self.position = POSITIONS.build(position, prefix, dtype, device, head_dim=self.head_dim) if position is not None else None

    def params(self) -> List[ParamSpec]:
        return self.qkv.params() + self.out.params()

    def parts(self):
        return [self.position] if self.position is not None else []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.qkv.bind(tensors)
        self.out.bind(tensors)

    def cache_requirement(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window)

    def fused_decode(self):
        rope = self.position.fused_decode() if self.position is not None else None
        if type(self) is not PagedAttention or rope is None or rope["rotary_dim"] != self.head_dim or self.out.bias is not None:
            return None
        return {"w_qkv": self.qkv.weight, "b_qkv": self.qkv.bias, "w_o": self.out.weight, "hidden": self.hidden, "heads": self.num_heads,
                "kv_heads": self.num_kv_heads, "head_dim": self.head_dim, "scale": self.scale, "window": self.window,
                "rope_denominators": rope["denominators"]}

    def forward(self, h, ctx, cache):
        return self.out(self._attend(h, ctx, cache))

    def forward_into(self, h, ctx, cache, tail):
        return tail.apply_linear(self.out, self._attend(h, ctx, cache))

    def _attend(self, h, ctx, cache):
        """Everything before the output projection: [tokens, heads * head_dim]."""
        view = ctx.group(cache.group)
        h, row_scale = undefer(h, self.qkv.weight)
        qkv = torch.empty((h.shape[0], self.qkv.out_features), dtype=self.dtype, device=h.device)
        # projection, position encoding of q and k, k and v into the cache: one call (and for few tokens one kernel)
        rot = self.position.rotary(ctx) if self.position is not None else None
        K.linear_rope_kv(
            h, self.qkv.weight, self.qkv.bias, qkv, ctx.positions, rot.denominators if rot else None, rot.rotary_dim if rot else 0,
            view.slot_mapping, cache.k, cache.v, self.num_heads, self.num_kv_heads, self.head_dim, cache.writes, row_scale=row_scale,
            cos_sin=rot.table if rot else None)
        o = torch.empty((h.shape[0], self.q_dim), dtype=self.dtype, device=h.device)
        K.paged_attention(
            qkv, o, cache.k, cache.v, view.block_table, ctx.q_start, ctx.ctx_lens, ctx.seq_of_token, ctx.positions,
            self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window,
            ctx.max_q_len, ctx.max_ctx_len, old_lens=ctx.old_lens, singles=ctx.num_single,
            units=ctx.attn_units, unit_slots=ctx.attn_unit_slots)
        return o
