"""The one model class: a decoder assembled from a ModelSpec.

embedding -> blocks in the order of the schedule -> final norm and lm_head on
the wanted rows only (LitInfer computes logits for every row and uses one,
src/llaisys/models/qwen2.cpp:331-350).  Which architecture a ModelSpec came
from does not matter here; the architecture registry supplies the spec and
the part registries supply the parts.
"""

from __future__ import annotations

from pathlib import Path
from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..config import ModelSpec, load_config, validate_schedule
from ..parts import BLOCKS, NORMS
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
        self.embedding: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------
    def params(self) -> List[ParamSpec]:
        s = self.spec
        out = [ParamSpec(s.embedding_name, (s.vocab_size, s.hidden_size), role="matrix")]
        for b in self.blocks:
            out.extend(b.all_params())
        out.extend(self.final_norm.all_params())
        if not s.tie_word_embeddings:
            out.append(ParamSpec(s.lm_head_name, (s.vocab_size, s.hidden_size), role="matrix"))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors.pop(s.embedding_name)
        for b in self.blocks:
            b.bind_all(tensors)
        self.final_norm.bind_all(tensors)
        # tied: the embedding table itself (python/llaisys/models/qwen2.py:196-199)
        self.lm_head = self.embedding if s.tie_word_embeddings else tensors.pop(s.lm_head_name)
        if tensors:
            raise RuntimeError("tensors left unbound: " + ", ".join(sorted(tensors)))

    def cache_requirements(self):
        """For each schedule entry: PagedKV, FixedState or None (entries that read another's cache: None)."""
        out = []
        for e in self.spec.schedule:
            out.append(self.blocks[e.block].mixer.cache_requirement() if e.cache_from is None else None)
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
        x32 = torch.empty((ctx.num_tokens, s.hidden_size), dtype=torch.float32, device=self.device)
        K.embedding(self.embedding, ctx.token_ids, x32)
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
        return logits


def declared_params(spec: ModelSpec) -> List[ParamSpec]:
    """The tensors a model of this spec holds (built on the meta device: no memory)."""
    return DecoderModel(spec, torch.float32, "meta").params()
