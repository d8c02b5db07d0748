"""The scheduler's decisions written out in plain Python, for the tests: what the scheduler of the host runtime
(``csrc/host/scheduler.cpp``) has to decide, step by step, under the same requests and the same drawn tokens."""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from litinfer_b200.cache import CacheManager, OutOfPages, RequestCache
from litinfer_b200.sampling import SamplingParams

DEFAULT_MAX_NEW_TOKENS = 512        # src/llaisys/models/qwen2.cpp:795


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64
    max_tokens_per_step: int = 2048
    prefill_chunk: int = 2048            # a portion of a prompt per step: the step's whole budget (the tensor-memory kernels are at their best from about 2,000 rows)

    def __post_init__(self):
        for k in ("max_num_seqs", "max_tokens_per_step", "prefill_chunk"):
            if getattr(self, k) <= 0:
                raise ValueError(f"{k} must be positive")


@dataclass
class Request:
    id: int
    prompt: List[int]
    max_new_tokens: int
    params: SamplingParams
    generated: List[int] = field(default_factory=list)
    status: str = "waiting"                 # waiting | running | finished
    finish_reason: Optional[str] = None     # eos | length | max_positions | aborted
    cache: Optional[RequestCache] = None
    preemptions: int = 0
    admitted_at: int = -1

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.generated)

    def token_slice(self, start: int, count: int) -> List[int]:
        """tokens[start:start + count] without building the whole list."""
        n = len(self.prompt)
        stop = start + count
        if stop <= n:
            return self.prompt[start:stop]
        if start >= n:
            return self.generated[start - n:stop - n]
        return self.prompt[start:] + self.generated[:stop - n]

    @property
    def num_cached(self) -> int:
        return self.cache.length if self.cache is not None else 0

    @property
    def finished(self) -> bool:
        return self.status == "finished"


@dataclass
class ScheduledItem:
    request: Request
    start: int                  # position of the first token of this portion
    count: int
    wants_logits: bool          # the portion reaches the request's last token

    @property
    def tokens(self) -> List[int]:
        return self.request.token_slice(self.start, self.count)


class RequestRefused(ValueError):
    pass


class Scheduler:
    def __init__(self, manager: CacheManager, config: SchedulerConfig, max_positions: int, eos_token_ids: Sequence[int] = ()) -> None:
        self.manager = manager
        self.config = config
        self.max_positions = int(max_positions)
        self.eos = set(int(e) for e in eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.requests: Dict[int, Request] = {}
        self._next_id = 0
        self._clock = 0
        self.num_preemptions = 0

    # ------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], max_new_tokens: int = 128, params: Optional[SamplingParams] = None) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise RequestRefused("a request needs at least one prompt token")
        if max_new_tokens is None or max_new_tokens <= 0:
            max_new_tokens = DEFAULT_MAX_NEW_TOKENS
        # the last generated token is never fed back, hence the -1 (python/llaisys/models/qwen2.py:342-346)
        most = len(prompt) + max_new_tokens - 1
        if most > self.max_positions:
            raise RequestRefused(
                f"prompt of {len(prompt)} tokens plus {max_new_tokens} new ones exceeds the model's {self.max_positions} positions")
        pages = -(-most // self.manager.page_size)
        if pages > self.manager.num_pages:
            raise RequestRefused(
                f"the request may hold {most} tokens ({pages} pages), the cache has {self.manager.num_pages} pages")
        rid = self._next_id
        self._next_id += 1
        req = Request(rid, prompt, int(max_new_tokens), params or SamplingParams())
        self.requests[rid] = req
        self.waiting.append(req)
        return rid

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, rid: int) -> None:
        req = self.requests[rid]
        if req.finished:
            return
        if req.status == "running":
            self.running.remove(req)
            self._give_back(req)
        else:
            self.waiting.remove(req)
        req.status, req.finish_reason = "finished", "aborted"

    def forget(self, rid: int) -> None:
        """Drop a finished request's record (LitInfer keeps them forever, qwen2.cpp:797-798)."""
        if not self.requests[rid].finished:
            raise ValueError(f"request {rid} is not finished")
        del self.requests[rid]

    # ------------------------------------------------------------------
    def _give_back(self, req: Request) -> None:
        if req.cache is not None:
            self.manager.release(req.cache)
            req.cache = None

    def _preempt(self, req: Request) -> None:
        self.running.remove(req)
        self._give_back(req)
        req.status = "waiting"
        req.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)

    def _fit(self, req: Request, want: int) -> int:
        """How many of the next ``want`` tokens fit into the free pages of every group."""
        rc = req.cache
        page = self.manager.page_size
        most = want
        for gid, g in enumerate(self.manager.groups):
            have = rc.num_blocks(gid) * page - rc.length
            most = min(most, have + g.pool.num_free * page)
        return max(0, most)

    def schedule(self) -> List[ScheduledItem]:
        """Pick the next step's items and allocate their pages."""
        cfg = self.config
        preempted_before = self.num_preemptions
        while True:
            budget = cfg.max_tokens_per_step
            items: List[ScheduledItem] = []
            picked = set()
            # 1. decoding requests, oldest first; preempt the youngest when a page is missing
            for req in list(self.running):
                if req.status != "running" or budget <= 0:
                    continue
                if req.num_tokens - req.num_cached != 1:
                    continue
                while True:
                    try:
                        self.manager.extend(req.cache, req.num_cached + 1)
                        break
                    except OutOfPages:
                        victim = self.running[-1]
                        self._preempt(victim)
                        if victim is req:
                            break
                if req.status != "running":
                    continue
                items.append(ScheduledItem(req, req.num_cached, 1, True))
                picked.add(req.id)
                budget -= 1
            # 2. prompt portions of running requests
            for req in self.running:
                if budget <= 0:
                    break
                if req.id in picked:
                    continue
                left = req.num_tokens - req.num_cached
                n = self._fit(req, min(left, cfg.prefill_chunk, budget))
                if n <= 0:
                    continue
                self.manager.extend(req.cache, req.num_cached + n)
                items.append(ScheduledItem(req, req.num_cached, n, n == left))
                picked.add(req.id)
                budget -= n
            # 3. admit waiting requests, in order
            while self.waiting and budget > 0 and len(self.running) < cfg.max_num_seqs and self.manager.num_free_slots() > 0:
                if self.num_preemptions != preempted_before:
                    break                   # a request was just preempted for lack of pages: admit nobody this step
                req = self.waiting[0]
                req.cache = self.manager.admit(req.id)
                n = self._fit(req, min(req.num_tokens, cfg.prefill_chunk, budget))
                if n <= 0:
                    self._give_back(req)
                    break
                self.waiting.popleft()
                req.status = "running"
                req.admitted_at = self._clock
                self._clock += 1
                self.running.append(req)
                self.manager.extend(req.cache, n)
                items.append(ScheduledItem(req, 0, n, n == req.num_tokens))
                picked.add(req.id)
                budget -= n
            if items or not self.running:
                return items
            # nothing can run although requests are live: free the youngest one's pages
            self._preempt(self.running[-1])

    # ------------------------------------------------------------------
    def update(self, items: Sequence[ScheduledItem], sampled: Sequence[Optional[int]]) -> List[Request]:
        """After the step: ``sampled[i]`` is the token drawn for ``items[i]`` (None if it
        wanted no logits).  Returns the requests that finished."""
        done = []
        for it, tok in zip(items, sampled):
            req = it.request
            if not it.wants_logits:
                continue
            if tok is None:
                raise ValueError(f"request {req.id} wanted a token and got none")
            tok = int(tok)
            if tok in self.eos:
                req.finish_reason = "eos"                       # the token is dropped (qwen2.cpp:1060-1062)
            else:
                req.generated.append(tok)
                if len(req.generated) >= req.max_new_tokens:
                    req.finish_reason = "length"
                elif req.num_tokens > self.max_positions:
                    req.finish_reason = "max_positions"
            if req.finish_reason is not None:
                self.running.remove(req)
                self._give_back(req)
                req.status = "finished"
                done.append(req)
        return done
