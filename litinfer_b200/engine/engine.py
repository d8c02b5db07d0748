"""The continuous-batching engine: scheduler + step function + sampler.

Every call of :meth:`Engine.step` re-forms the batch: schedule, run one step,
sample one token for every request whose portion reached its last token,
append, finish and free.  Method names follow LitInfer's engine interface
(``engine_add_request / engine_step / engine_has_unfinished /
engine_is_finished / engine_get_output``, python/llaisys/models/qwen2.py:458-496);
unlike there, sampling parameters belong to a request, not to a step, and the
output of a running request can be read at any time.

``run_ahead``: while every live request is decoding, the step after the one in
flight is launched before that one's tokens have been read: its input tokens
stay on the device (the sampler's output feeds the next step's embedding), and
the host's bookkeeping for a step overlaps the device's work on the next one.
The tokens of a step then become visible one call of :meth:`Engine.step`
later.  What is launched ahead is only what is certain but for an end-of-sequence
token: no request of the step in flight reaches its length limit with it, nobody
waits to be admitted, pages are there.  If a request ends on an end-of-sequence
token after all, the token computed ahead for it is dropped.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Set

import torch

from ..cache.manager import CacheManager
from ..models.decoder import DecoderModel
from ..sampling.sampler import Sampler, SamplingParams
from .batch import StepItem
from ..cache.pool import OutOfPages
from .scheduler import Request, ScheduledItem, Scheduler, SchedulerConfig
from .step import ModelRunner


@dataclass
class EngineConfig:
    num_pages: int = 256                 # LitInfer's default pool: min(ceil(max_positions / 16), 256) pages (qwen2.cpp:114-120)
    page_size: int = 16                  # src/llaisys/kv_cache/block_kv_cache.hpp:11
    max_num_seqs: int = 64
    max_tokens_per_step: int = 2048
    prefill_chunk: int = 2048
    use_graphs: bool = True
    max_context: Optional[int] = None    # longest context a captured decode step must cover
    run_ahead: bool = True               # launch a decode step before the tokens of the one before it are read


@dataclass
class _Launched:
    """A step on the device whose tokens have not been read yet."""

    items: List[ScheduledItem]
    tokens: Optional[torch.Tensor]                       # int32 [wanting items], on the device
    void: Set[int] = field(default_factory=set)          # requests that ended before this step's token could count
    host: Optional[torch.Tensor] = None                  # pinned copy of ``tokens``, under way on the copy stream
    copied: Optional[torch.cuda.Event] = None


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
        self._ahead: Optional[_Launched] = None
        # With run_ahead the tokens of a step are read while the next step is already queued on the compute stream: the
        # copy to the host goes over a stream of its own, behind an event, so that it does not wait for that next step.
        self._copy_stream = torch.cuda.Stream(model.device) if (c.run_ahead and model.device.type == "cuda") else None
        self._host_tokens = [torch.empty(max(c.max_num_seqs, 1), dtype=torch.int32).pin_memory() for _ in range(2)] if self._copy_stream else []
        self._host_turn = 0

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
        return self._ahead is not None or self.scheduler.has_unfinished()

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
        """One iteration; returns the requests that finished in it (with ``run_ahead``: the requests
        whose end became known in it)."""
        if not self.config.run_ahead:
            items = self.scheduler.schedule()
            if not items:
                return []
            return self._resolve(self._launch(items))
        ahead = self._ahead
        if ahead is None:
            items = self.scheduler.schedule()
            if not items:
                return []
            launched = self._launch(items)
            if self._all_decoding(items):
                self._ahead = launched                     # its tokens are read in the next call, after the step that follows is on its way
                return []
            return self._resolve(launched)
        following = self._launch_after(ahead)
        done = self._resolve(ahead)
        if following is not None:
            following.void = {r.id for r in done}
        self._ahead = following
        return done

    def abort(self, rid: int) -> List[Request]:
        """End request ``rid`` now and give back what it holds.  A step launched ahead is read first, so that the
        tokens it computed for the other requests count; returns the requests whose end became known by that."""
        done = self.drain()
        self.scheduler.abort(rid)
        return done

    def drain(self) -> List[Request]:
        """Read the tokens of a step that was launched ahead, if there is one."""
        ahead, self._ahead = self._ahead, None
        return self._resolve(ahead) if ahead is not None else []

    # ------------------------------------------------------------------
    def _launch(self, items: List[ScheduledItem], token_source: Optional[torch.Tensor] = None) -> _Launched:
        """Run the step and sample; nothing is read back.  ``token_source``: the items are single decode tokens whose
        ids are the device tensor's entries (the tokens of the step before, not appended to the requests yet)."""
        ahead_by = 0 if token_source is None else 1
        if token_source is None:
            step_items = [StepItem(it.request.cache, it.tokens, (it.count - 1,) if it.wants_logits else ()) for it in items]
        else:
            step_items = [StepItem(it.request.cache, (0,), (0,)) for it in items]
        logits = self.runner.step(step_items, token_source=token_source)
        self.tokens_run += sum(it.count for it in items)
        wanting = [it for it in items if it.wants_logits]
        toks = None
        if wanting:
            toks = self.sampler.sample(
                logits, [it.request.params for it in wanting], [len(it.request.generated) + ahead_by for it in wanting])
        launched = _Launched(items, toks)
        if toks is not None and self._copy_stream is not None and toks.numel() <= self._host_tokens[0].numel():
            sampled_ev = torch.cuda.Event()
            sampled_ev.record(torch.cuda.current_stream(self.model.device))
            launched.host = self._host_tokens[self._host_turn][:toks.numel()]      # two buffers: at most two steps are unread
            self._host_turn ^= 1
            launched.copied = torch.cuda.Event()
            with torch.cuda.stream(self._copy_stream):
                self._copy_stream.wait_event(sampled_ev)
                launched.host.copy_(toks, non_blocking=True)
                launched.copied.record(self._copy_stream)
        return launched

    def _resolve(self, launched: _Launched) -> List[Request]:
        """Read the step's tokens and let the scheduler append them, finish and free."""
        items = launched.items
        sampled: List[Optional[int]] = [None] * len(items)
        if launched.tokens is not None:
            if launched.copied is not None:
                launched.copied.synchronize()
                host = launched.host.tolist()
            else:
                host = launched.tokens.tolist()
            j = 0
            for i, it in enumerate(items):
                if it.wants_logits:
                    sampled[i] = host[j]
                    j += 1
        # requests that ended before this step's token could count: on an end-of-sequence token of the step before
        # (void), or aborted through the scheduler while the step was in flight (no longer running)
        if launched.void or any(it.request.status != "running" for it in items):
            keep = [i for i, it in enumerate(items) if it.request.id not in launched.void and it.request.status == "running"]
            items = [items[i] for i in keep]
            sampled = [sampled[i] for i in keep]
        return self.scheduler.update(items, sampled)

    def _all_decoding(self, items: List[ScheduledItem]) -> bool:
        return (not self.scheduler.waiting and len(items) == len(self.scheduler.running)
                and all(it.count == 1 and it.wants_logits for it in items))

    def _launch_after(self, ahead: _Launched) -> Optional[_Launched]:
        """The step that follows ``ahead`` if it is certain but for end-of-sequence tokens: the same requests, each one
        token further, fed from ``ahead``'s tokens on the device.  None if anything else could happen."""
        sch = self.scheduler
        if ahead.tokens is None or ahead.void or not self._all_decoding(ahead.items):
            return None
        for it in ahead.items:
            req = it.request
            if req.status != "running":
                return None
            # with the token in flight the request would reach a limit: the scheduler has to see that first
            if len(req.generated) + 1 >= req.max_new_tokens or req.num_tokens + 1 > sch.max_positions:
                return None
        try:
            for it in ahead.items:
                self.manager.extend(it.request.cache, it.request.num_cached + 1)
        except OutOfPages:
            return None                                    # pages taken so far stay with their requests, which need them next step anyway
        items = [ScheduledItem(it.request, it.request.num_cached, 1, True) for it in ahead.items]
        return self._launch(items, token_source=ahead.tokens)

    def run_to_completion(self) -> None:
        while self.has_unfinished():
            self.step()
        self.drain()
