"""The continuous-batching engine: scheduler + step function + sampler.

Every call of :meth:`Engine.step` re-forms the batch: schedule, run one step,
sample one token for every request whose portion reached its last token,
append, finish and free.  Method names follow LitInfer's engine interface
(``engine_add_request / engine_step / engine_has_unfinished /
engine_is_finished / engine_get_output``, python/llaisys/models/qwen2.py:458-496);
unlike there, sampling parameters belong to a request, not to a step, and the
output of a running request can be read at any time.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..models.decoder import DecoderModel
from ..sampling.sampler import Sampler, SamplingParams
from .batch import StepItem
from .scheduler import Request, Scheduler, SchedulerConfig
from .step import ModelRunner


@dataclass
class EngineConfig:
    num_pages: int = 256                 # LitInfer's default pool: min(ceil(max_positions / 16), 256) pages (qwen2.cpp:114-120)
    page_size: int = 16                  # src/llaisys/kv_cache/block_kv_cache.hpp:11
    max_num_seqs: int = 64
    max_tokens_per_step: int = 2048
    prefill_chunk: int = 512
    use_graphs: bool = True
    max_context: Optional[int] = None    # longest context a captured decode step must cover


class Engine:
    def __init__(self, model: DecoderModel, config: Optional[EngineConfig] = None) -> None:
        self.model = model
        self.config = config or EngineConfig()
        c = self.config
        spec = model.spec
        self.manager = CacheManager(
            model.cache_requirements(), [e.cache_from for e in spec.schedule],
            c.num_pages, c.page_size, c.max_num_seqs, model.dtype, model.device)
        max_ctx = min(c.max_context or spec.max_position_embeddings, spec.max_position_embeddings, c.num_pages * c.page_size)
        self.runner = ModelRunner(model, self.manager, use_graphs=c.use_graphs, max_context=max_ctx)
        self.scheduler = Scheduler(
            self.manager, SchedulerConfig(c.max_num_seqs, c.max_tokens_per_step, c.prefill_chunk),
            spec.max_position_embeddings, spec.eos_token_ids)
        self.sampler = Sampler(model.device)
        self.tokens_run = 0

    @staticmethod
    def bytes_per_page(model: DecoderModel, page_size: int = 16) -> int:
        """Device bytes one page id stands for, over all cache groups and their entries."""
        probe = CacheManager(model.cache_requirements(), [e.cache_from for e in model.spec.schedule], 1, page_size, 1,
                             model.dtype, "cpu", allocate=False)
        return probe.bytes_per_page()

    # ------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], max_new_tokens: int = 128, params: Optional[SamplingParams] = None) -> int:
        vocab = self.model.spec.vocab_size
        for t in prompt:
            if not 0 <= int(t) < vocab:
                raise IndexError(f"token id {t} outside [0, {vocab})")
        return self.scheduler.add_request(prompt, max_new_tokens, params)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    def is_finished(self, rid: int) -> bool:
        req = self.scheduler.requests.get(rid)
        return True if req is None else req.finished        # unknown ids read as finished (qwen2.cpp:811-813)

    def get_output(self, rid: int) -> List[int]:
        return list(self.scheduler.requests[rid].generated)

    def finish_reason(self, rid: int) -> Optional[str]:
        return self.scheduler.requests[rid].finish_reason

    def num_seqs(self) -> int:
        return len(self.scheduler.requests)

    # ------------------------------------------------------------------
    def step(self) -> List[Request]:
        """One iteration; returns the requests that finished in it."""
        items = self.scheduler.schedule()
        if not items:
            return []
        step_items = [StepItem(it.request.cache, it.tokens, (it.count - 1,) if it.wants_logits else ()) for it in items]
        logits = self.runner.step(step_items)
        self.tokens_run += sum(it.count for it in items)
        wanting = [it for it in items if it.wants_logits]
        sampled: List[Optional[int]] = [None] * len(items)
        if wanting:
            toks = self.sampler.sample(
                logits, [it.request.params for it in wanting], [len(it.request.generated) for it in wanting])
            host = toks.tolist()
            j = 0
            for i, it in enumerate(items):
                if it.wants_logits:
                    sampled[i] = host[j]
                    j += 1
        return self.scheduler.update(items, sampled)

    def run_to_completion(self) -> None:
        while self.has_unfinished():
            self.step()
