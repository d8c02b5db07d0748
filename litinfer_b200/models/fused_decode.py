"""A decode step as one persistent kernel (``csrc/decode_step.cu``).

LitInfer runs a step layer by layer, operator by operator (src/llaisys/models/qwen2.cpp:967-1047).  So does
:meth:`DecoderModel.forward`, part by part, for every kind of step and every kind of part.  For the one shape of
step that decides the speed of generation, single new tokens of up to 16 sequences in bfloat16, and for layers
that are what the fused kernel is built for (pre-norm blocks of paged attention with a full rotation, a gated
feed-forward with the fused activation, RMSNorms), the same arithmetic runs as a single launch instead.

No part knows about this file.  A part that can take part says so by answering :meth:`Part.fused_decode` with its
tensors and constants; a part that does not (any part registered from outside) makes the model run part by part, as
before.  The plan (a table of the layers' pointers in device memory, scratch buffers) is made once per cache and
batch tile and kept, because captured graphs hold its addresses.
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch

from .. import kernels as K

MAX_GROUPS = 8
MAX_TOKENS = 16

_vp, _fp, _ip = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p


class LayerStruct(ctypes.Structure):
    """``LiDecodeLayer`` of csrc/decode_step.h."""

    _fields_ = [
        ("w_qkv", _vp), ("b_qkv", _fp), ("w_o", _vp), ("w_gate_up", _vp), ("w_down", _vp), ("norm_ffn", _fp), ("norm_next", _fp),
        ("kcache", _vp), ("vcache", _vp), ("rope_denom", _fp),
        ("eps_ffn", ctypes.c_float), ("eps_next", ctypes.c_float), ("scale", ctypes.c_float),
        ("window", ctypes.c_int), ("group", ctypes.c_int), ("num_pages", ctypes.c_int), ("write_cache", ctypes.c_int), ("reserved", ctypes.c_int),
    ]


class StepStruct(ctypes.Structure):
    """``LiDecodeStep`` of csrc/decode_step.h."""

    _fields_ = [
        ("layers", _vp), ("num_layers", ctypes.c_int), ("M", ctypes.c_int),
        ("hidden", ctypes.c_int), ("heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("head_dim", ctypes.c_int),
        ("intermediate", ctypes.c_int), ("vocab", ctypes.c_int), ("page_size", ctypes.c_int), ("max_blocks", ctypes.c_int),
        ("embedding", _vp), ("norm_first", _fp), ("eps_first", ctypes.c_float), ("rows", ctypes.c_int),
        ("token_ids", _ip), ("positions", _ip), ("ctx_lens", _ip), ("old_lens", _ip), ("logit_rows", _ip),
        ("slot_mapping", _ip * MAX_GROUPS), ("block_table", _ip * MAX_GROUPS),
        ("lm_head", _vp), ("logits", _fp),
        ("x32", _fp), ("h_a", _vp), ("h_b", _vp), ("ssq_a", _fp), ("ssq_b", _fp), ("qkv", _vp), ("attn", _vp), ("act", _vp),
        ("attn_part", _fp), ("attn_counters", _vp), ("barrier", _vp),
        ("splits", ctypes.c_int), ("stage_k", ctypes.c_int), ("stages", ctypes.c_int), ("balance", ctypes.c_int), ("x_cols", ctypes.c_int),
    ]


def enabled() -> bool:
    """Off unless ``LITINFER_B200_FUSED_DECODE=1``: as measured (1.5B shape, batch 8, context 2,048) the fused step takes
    3.4 ms where the chain of separate kernels takes 1.3 ms.  Its weight stream alone would sustain a step of 0.65 ms, but
    the consumers' critical path does not: a layer is some twenty dependent round trips to L2 (1.2 us each while the
    stream saturates the memory system, against 0.16 us idle), five grid-wide barriers, and 150 KB of code that no longer
    fits the instruction cache.  Kept for the cases and the measurements, not as the default path."""
    return os.environ.get("LITINFER_B200_FUSED_DECODE", "0") == "1"


def describe(model) -> Optional[List[dict]]:
    """What each schedule entry's block says of itself for the fused step, or None if any of them (or the model
    around them) is not what the kernel is built for."""
    spec = model.spec
    if model.dtype != torch.bfloat16 or model.device.type != "cuda":
        return None
    if spec.position is not None or spec.embedding_scale is not None or spec.logit_cap is not None:
        return None
    final = model.final_norm.fused_decode()
    if final is None or model.lm_head is None or model.lm_head.dtype != torch.bfloat16:
        return None
    out = []
    for e in spec.schedule:
        d = model.blocks[e.block].fused_decode()
        if d is None:
            return None
        out.append(d)
    first = out[0]
    for d in out:
        if any(d[k] != first[k] for k in ("hidden", "heads", "kv_heads", "head_dim", "intermediate")):
            return None
    for i, d in enumerate(out):
        d["norm_next"] = out[i + 1]["norm_first"] if i + 1 < len(out) else final
    lib = K.library()
    if lib.li_decode_step_accepts(1, first["hidden"], first["heads"], first["kv_heads"], first["head_dim"], first["intermediate"],
                                  spec.vocab_size, 16) != 0:
        return None
    return out


class _Plan:
    """The layer table for one set of caches and the scratch for one tile of tokens."""

    def __init__(self, model, layers: List[dict], caches, tile: int, max_blocks: int, page_size: int) -> None:
        dev = model.device
        first = layers[0]
        H, nh, nkv, dh, I = first["hidden"], first["heads"], first["kv_heads"], first["head_dim"], first["intermediate"]
        self.keep = []                                         # tensors whose addresses the table holds
        arr = (LayerStruct * len(layers))()
        for i, (d, cache) in enumerate(zip(layers, caches)):
            if cache.kind != "paged" or cache.k is None or cache.group >= MAX_GROUPS:
                raise K.KernelError("fused decode: a layer without a paged cache")
            L = arr[i]
            L.w_qkv, L.b_qkv = d["w_qkv"].data_ptr(), (d["b_qkv"].data_ptr() if d["b_qkv"] is not None else None)
            L.w_o, L.w_gate_up, L.w_down = d["w_o"].data_ptr(), d["w_gate_up"].data_ptr(), d["w_down"].data_ptr()
            L.norm_ffn, L.norm_next = d["norm_ffn"]["weight"].data_ptr(), d["norm_next"]["weight"].data_ptr()
            L.kcache, L.vcache, L.rope_denom = cache.k.data_ptr(), cache.v.data_ptr(), d["rope_denominators"].data_ptr()
            L.eps_ffn, L.eps_next, L.scale = d["norm_ffn"]["eps"], d["norm_next"]["eps"], d["scale"]
            L.window, L.group, L.num_pages, L.write_cache = int(d["window"] or 0), cache.group, cache.k.shape[0], 1 if cache.writes else 0
        raw = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).clone()
        self.table = raw.to(dev)
        self.tile = tile
        self.splits = max(1, -(-(max_blocks * page_size) // 256))
        bf, f32 = torch.bfloat16, torch.float32
        parts = -(-H // 16)
        self.x32 = torch.empty((tile, H), dtype=f32, device=dev)
        self.h_a, self.h_b = torch.empty((tile, H), dtype=bf, device=dev), torch.empty((tile, H), dtype=bf, device=dev)
        self.ssq_a, self.ssq_b = torch.empty((tile, parts), dtype=f32, device=dev), torch.empty((tile, parts), dtype=f32, device=dev)
        self.qkv = torch.empty((tile, (nh + 2 * nkv) * dh), dtype=bf, device=dev)
        self.attn = torch.empty((tile, nh * dh), dtype=bf, device=dev)
        self.act = torch.empty((tile, I), dtype=bf, device=dev)
        self.attn_part = torch.empty((tile * nh * self.splits * (dh + 2),), dtype=f32, device=dev)
        self.attn_counters = torch.zeros((tile * nkv + 1,), dtype=torch.int32, device=dev)
        self.barrier = self.attn_counters[tile * nkv:]
        stage_k, stages, x_cols, scratch = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
        K._check(K.library().li_decode_step_plan(tile, H, nh, nkv, dh, self.splits, ctypes.byref(stage_k), ctypes.byref(stages),
                                                 ctypes.byref(x_cols), ctypes.byref(scratch)), "decode step plan")
        self.x_cols = x_cols.value if os.environ.get("LITINFER_B200_FUSED_X", "1") != "0" else 0
        self.stage_k = int(os.environ.get("LITINFER_B200_FUSED_STAGE_K", stage_k.value))
        self.stages = int(os.environ.get("LITINFER_B200_FUSED_STAGES", stages.value))
        s = StepStruct()
        s.layers, s.num_layers = self.table.data_ptr(), len(layers)
        s.hidden, s.heads, s.kv_heads, s.head_dim, s.intermediate = H, nh, nkv, dh, I
        s.vocab, s.page_size, s.max_blocks = model.spec.vocab_size, page_size, max_blocks
        s.embedding, s.norm_first, s.eps_first = model.embedding.data_ptr(), first["norm_first"]["weight"].data_ptr(), first["norm_first"]["eps"]
        s.lm_head = model.lm_head.data_ptr()
        s.x32, s.h_a, s.h_b, s.ssq_a, s.ssq_b = (t.data_ptr() for t in (self.x32, self.h_a, self.h_b, self.ssq_a, self.ssq_b))
        s.qkv, s.attn, s.act, s.attn_part = (t.data_ptr() for t in (self.qkv, self.attn, self.act, self.attn_part))
        s.attn_counters, s.barrier = self.attn_counters.data_ptr(), self.barrier.data_ptr()
        s.splits, s.stage_k, s.stages, s.x_cols = self.splits, self.stage_k, self.stages, self.x_cols
        s.balance = 2 if os.environ.get("LITINFER_B200_FUSED_DEBUG") else 0            # bit 1: progress marks in the mapped status area
        self.step = s


class FusedDecode:
    """Runs the steps it accepts; :meth:`run` returns None for the others."""

    def __init__(self, model, enable: Optional[bool] = None) -> None:
        self.model = model
        self.layers = describe(model) if (enabled() if enable is None else enable) else None
        self._plans: Dict[tuple, _Plan] = {}
        self.launches = 0

    def accepts(self, ctx, caches) -> bool:
        if self.layers is None or ctx.max_q_len != 1 or ctx.num_tokens != ctx.num_seqs or not 1 <= ctx.num_tokens <= MAX_TOKENS:
            return False
        return len(ctx.groups) <= MAX_GROUPS and all(c.kind == "paged" for c in caches)

    def run(self, ctx, caches) -> Optional[torch.Tensor]:
        if not self.accepts(ctx, caches):
            return None
        model = self.model
        M = ctx.num_tokens
        tile = 8 if M <= 8 else 16
        mb, page = ctx.groups[0].max_blocks, ctx.groups[0].page_size
        key = (tile, mb, page) + tuple(c.k.data_ptr() for c in caches)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = _Plan(model, self.layers, caches, tile, mb, page)
        R = ctx.num_logit_rows
        logits = torch.empty((R, model.spec.vocab_size), dtype=torch.float32, device=model.device)
        s = plan.step
        s.M, s.rows = M, R
        s.token_ids, s.positions, s.ctx_lens = ctx.token_ids.data_ptr(), ctx.positions.data_ptr(), ctx.ctx_lens.data_ptr()
        s.old_lens = ctx.old_lens.data_ptr() if ctx.old_lens is not None else None
        s.logit_rows, s.logits = (ctx.logit_rows.data_ptr() if R else None), (logits.data_ptr() if R else None)
        for g, view in enumerate(ctx.groups):
            s.slot_mapping[g], s.block_table[g] = view.slot_mapping.data_ptr(), view.block_table.data_ptr()
        K._check(K.library().li_decode_step(ctypes.byref(s), K._stream(logits)), "decode step")
        self.launches += 1
        return logits
