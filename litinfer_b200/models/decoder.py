"""The one model class: a decoder assembled from a ModelSpec.

embedding (-> the model's own position encoding, if the spec names one) ->
blocks in the order of the schedule -> final norm and lm_head on the wanted
rows only (LitInfer computes logits for every row and uses one,
src/llaisys/models/qwen2.cpp:331-350).  The lm_head follows the file, as in
LitInfer (python/llaisys/models/qwen2.py:143-146, 196-199): a stored one is
used, a missing one is the embedding table, whatever config.json says; the
spec's ``tie_word_embeddings`` only decides what random-weights mode makes.  Which architecture a ModelSpec came
from does not matter here; the architecture registry supplies the spec and
the part registries supply the parts.
"""

from __future__ import annotations

from pathlib import Path
from dataclasses import replace
from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..config import ModelSpec, load_config, validate_schedule
from ..parts import BLOCKS, NORMS, POSITIONS
from ..parts.base import FixedState, PagedKV
from ..weights.loader import ParamSpec, load_tensors
from ..weights.random_init import random_tensors

RUN_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def run_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"run dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return RUN_DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"run dtype must be bfloat16 or float32, got {name!r}") from None


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype, device) -> None:
        validate_schedule(spec)
        self.spec = spec
        self.dtype = run_dtype(dtype)
        self.device = torch.device(device)
        self.blocks = [BLOCKS.build(b, b.prefix, self.dtype, self.device) for b in spec.blocks]
        self.final_norm = NORMS.build(spec.final_norm, spec.final_norm_prefix, self.dtype, self.device)
        self.position = (POSITIONS.build(spec.position, spec.position_prefix, self.dtype, self.device)
                         if spec.position is not None else None)
        self.embedding: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self.head_is_tied = False
        self._fused = None                                     # models/fused_decode.py, made at the first step

    # ------------------------------------------------------------------
    def params(self) -> List[ParamSpec]:
        s = self.spec
        out = [ParamSpec(s.embedding_name, (s.vocab_size, s.hidden_size), role="matrix")]
        if self.position is not None:
            out.extend(self.position.all_params())
        for b in self.blocks:
            out.extend(b.all_params())
        out.extend(self.final_norm.all_params())
        # optional either way: the file decides (see bind); random-weights mode makes one unless the spec ties
        out.append(ParamSpec(s.lm_head_name, (s.vocab_size, s.hidden_size), role="matrix", optional=True,
                             draw=not s.tie_word_embeddings))
        if s.aliases:
            out = [replace(p, aliases=p.aliases + tuple(s.aliases[p.name])) if p.name in s.aliases else p for p in out]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors.pop(s.embedding_name)
        if self.position is not None:
            self.position.bind_all(tensors)
        for b in self.blocks:
            b.bind_all(tensors)
        self.final_norm.bind_all(tensors)
        # a stored head is used; without one the head is the embedding table itself
        # (python/llaisys/models/qwen2.py:196-199: ``if not w.out_embed and w.in_embed``)
        head = tensors.pop(s.lm_head_name, None)
        self.head_is_tied = head is None
        self.lm_head = self.embedding if head is None else head
        if tensors:
            raise RuntimeError("tensors left unbound: " + ", ".join(sorted(tensors)))

    def cache_requirements(self):
        """For each schedule entry: PagedKV, FixedState or None (entries that read another's cache: None)."""
        out = []
        for e in self.spec.schedule:
            out.append(self.blocks[e.block].cache_requirement() if e.cache_from is None else None)
        return out

    # ------------------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir, dtype, device, spec: Optional[ModelSpec] = None) -> "DecoderModel":
        spec = spec or load_config(model_dir).to_model_spec()
        model = cls(spec, dtype, device)
        model.bind(load_tensors(model_dir, model.params(), model.dtype, model.device))
        return model

    @classmethod
    def from_random(cls, spec: ModelSpec, seed: int, dtype, device) -> "DecoderModel":
        model = cls(spec, dtype, device)
        model.bind(random_tensors(model.params(), seed, model.dtype, model.device))
        return model

    # ------------------------------------------------------------------
    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the step's tokens; float32 logits ``[len(ctx.logit_rows), vocab]``."""
        s = self.spec
        if self.device.type == "cuda" and self.dtype == torch.bfloat16:
            # steps of single tokens of few sequences: one persistent kernel, if every part is one it is built for
            if self._fused is None:
                from .fused_decode import FusedDecode

                self._fused = FusedDecode(self)
            logits = self._fused.run(ctx, caches)
            if logits is not None:
                return logits
        x32 = torch.empty((ctx.num_tokens, s.hidden_size), dtype=torch.float32, device=self.device)
        K.embedding(self.embedding, ctx.token_ids, x32)
        if s.embedding_scale is not None:
            K.scale_inplace(x32, float(s.embedding_scale))
        if self.position is not None:
            self.position.add_to_stream(x32, ctx)
        carry = None
        last = len(s.schedule) - 1
        for i, e in enumerate(s.schedule):
            # a block is told the first norm of the block that runs next, so that it can apply it in its own tail
            next_entry = self.blocks[s.schedule[i + 1].block].entry() if i < last else None
            x32, carry = self.blocks[e.block].forward(x32, ctx, caches[i], carry, next_entry)
        if carry is not None and carry.delta is not None:
            K.residual_add(x32, carry.delta)
        R = ctx.num_logit_rows
        logits = torch.empty((R, s.vocab_size), dtype=torch.float32, device=self.device)
        if R:
            y = self.final_norm.gather_forward(x32, ctx.logit_rows)
            K.linear(y, self.lm_head, None, logits)
            if s.logit_cap is not None:
                K.logit_cap(logits, float(s.logit_cap))
        return logits


def declared_params(spec: ModelSpec) -> List[ParamSpec]:
    """The tensors a model of this spec holds (built on the meta device: no memory)."""
    return DecoderModel(spec, torch.float32, "meta").params()
