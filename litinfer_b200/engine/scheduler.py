"""The scheduler: which requests run in the next step, with how many tokens.

LitInfer's engine has no admission control, no token budget and no portions:
every unfinished request runs each step, a new one with its entire prompt
(src/llaisys/models/qwen2.cpp:934-941), and when pages run out it throws in
mid-step with some requests already advanced (qwen2.cpp:839-844).  Decided
here instead:

* Requests wait in FIFO order and are admitted while a state slot is free,
  fewer than ``max_num_seqs`` run, budget is left and at least one of their
  tokens fits into free pages.
* Each step spends at most ``max_tokens_per_step`` tokens: first one token for
  every running request that is decoding, then portions of prompts (at most
  ``prefill_chunk`` tokens each, and no more than the free pages hold) for
  running requests in admission order, then for newly admitted ones.
* **When pages run out** for a decoding request, the most recently admitted
  running request is preempted: its pages and slot are given back and it
  returns to the head of the waiting queue with the tokens it has produced so
  far, to be recomputed later.  A prompt portion never preempts anybody; it
  shrinks or waits.  If nothing at all can run, the most recently admitted
  request is preempted so that the oldest can.
* A request that could never fit (more tokens than the pool or the position
  limit holds) is refused when it is added.
* Finishing follows LitInfer (qwen2.cpp:1060-1066): an end-of-sequence token
  ends the request and is not part of its output; otherwise it ends after
  exactly ``max_new_tokens`` tokens (``<= 0`` means 512, qwen2.cpp:795).
  Pages are given back at once.

The decisions are taken in the host runtime (``csrc/host/scheduler.cpp``, C++)
over the cache manager's bookkeeping; this module holds the requests' tokens
and outputs and mirrors what the runtime did.  Host-only logic: no device.
"""

from __future__ import annotations

import ctypes
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

import numpy as np

from ..cache import native
from ..cache.manager import CacheManager, RequestCache
from ..sampling.sampler import SamplingParams

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
    """The Python face of the scheduler in the host runtime (``csrc/host/scheduler.cpp``): the decisions are taken
    there, over the cache manager's bookkeeping; the requests' tokens, sampling parameters and outputs live here."""

    _REASONS = {1: "eos", 2: "length", 3: "max_positions"}

    def __init__(self, manager: CacheManager, config: SchedulerConfig, max_positions: int, eos_token_ids: Sequence[int] = ()) -> None:
        self.manager = manager
        self.config = config
        self.max_positions = int(max_positions)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.requests: Dict[int, Request] = {}
        self._next_id = 0
        self._clock = 0
        self._lib = native.library()
        self._h = self._lib.li_sched_create(manager._h, config.max_num_seqs, config.max_tokens_per_step, config.prefill_chunk,
                                            self.max_positions)
        if not self._h:
            raise RuntimeError("the host runtime could not create the scheduler")
        cap = 4 * config.max_num_seqs + 64
        self._items = np.zeros(4 * cap, dtype=np.int32)
        self._events = np.zeros(3 * 8 * cap, dtype=np.int32)
        self.eos = eos_token_ids

    def __del__(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.li_sched_destroy(h)

    @property
    def eos(self):
        return self._eos

    @eos.setter
    def eos(self, ids) -> None:
        self._eos = set(int(e) for e in ids)
        arr = np.asarray(sorted(self._eos) or [0], dtype=np.int32)
        native.check(self._lib.li_sched_set_eos(self._h, arr.ctypes.data, len(self._eos)))

    @property
    def num_preemptions(self) -> int:
        w, r, p = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
        self._lib.li_sched_counts(self._h, ctypes.byref(w), ctypes.byref(r), ctypes.byref(p))
        return p.value

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
        native.check(self._lib.li_sched_add(self._h, rid, len(prompt), int(max_new_tokens)))
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
        was_running = ctypes.c_int(0)
        native.check(self._lib.li_sched_abort(self._h, rid, ctypes.byref(was_running)))
        if req.status == "running":
            self.running.remove(req)
            self._dropped(req)
        else:
            self.waiting.remove(req)
        req.status, req.finish_reason = "finished", "aborted"

    def forget(self, rid: int) -> None:
        """Drop a finished request's record (LitInfer keeps them forever, qwen2.cpp:797-798)."""
        if not self.requests[rid].finished:
            raise ValueError(f"request {rid} is not finished")
        native.check(self._lib.li_sched_forget(self._h, rid))
        del self.requests[rid]

    # ------------------------------------------------------------------
    def _dropped(self, req: Request) -> None:
        """The host runtime gave the request's pages and slot back: forget its cache here too."""
        if req.cache is not None:
            self.manager.dropped(req.cache)
            req.cache = None

    def _apply(self, n_events: int) -> None:
        """What the host runtime did to the requests while it scheduled, in order."""
        ev = self._events
        for i in range(n_events):
            kind, rid, arg = int(ev[3 * i]), int(ev[3 * i + 1]), int(ev[3 * i + 2])
            req = self.requests[rid]
            if kind == 1:                                   # admitted, with its state slot
                self._dropped(req)
                req.cache = self.manager.adopt(rid, arg)
                self.waiting.remove(req)
                req.status = "running"
                req.admitted_at = self._clock
                self._clock += 1
                self.running.append(req)
            elif kind == 2:                                 # preempted: back to the head of the queue, to be recomputed
                self.running.remove(req)
                self._dropped(req)
                req.status = "waiting"
                req.preemptions += 1
                self.waiting.appendleft(req)
            else:
                raise RuntimeError(f"unknown scheduler event {kind}")

    def schedule(self) -> List[ScheduledItem]:
        """Pick the next step's items and allocate their pages."""
        n_items, n_events = ctypes.c_int(0), ctypes.c_int(0)
        rc = self._lib.li_sched_schedule(self._h, self._items.ctypes.data, self._items.size // 4, ctypes.byref(n_items),
                                         self._events.ctypes.data, self._events.size // 3, ctypes.byref(n_events))
        self._apply(min(n_events.value, self._events.size // 3))
        native.check(rc)
        it = self._items
        return [ScheduledItem(self.requests[int(it[4 * i])], int(it[4 * i + 1]), int(it[4 * i + 2]), bool(it[4 * i + 3]))
                for i in range(n_items.value)]

    # ------------------------------------------------------------------
    def update(self, items: Sequence[ScheduledItem], sampled: Sequence[Optional[int]]) -> List[Request]:
        """After the step: ``sampled[i]`` is the token drawn for ``items[i]`` (None if it
        wanted no logits).  Returns the requests that finished."""
        wanting, toks = [], []
        for it, tok in zip(items, sampled):
            if not it.wants_logits:
                continue
            if tok is None:
                raise ValueError(f"request {it.request.id} wanted a token and got none")
            wanting.append(it.request)
            toks.append(int(tok))
        if not wanting:
            return []
        n = len(wanting)
        ids, tk = np.asarray([r.id for r in wanting], dtype=np.int32), np.asarray(toks, dtype=np.int32)
        outcome, reason = np.zeros(n, dtype=np.int32), np.zeros(n, dtype=np.int32)
        native.check(self._lib.li_sched_update(self._h, n, ids.ctypes.data, tk.ctypes.data, outcome.ctypes.data, reason.ctypes.data))
        done = []
        for req, tok, kept, why in zip(wanting, toks, outcome.tolist(), reason.tolist()):
            if kept:
                req.generated.append(tok)                   # an end-of-sequence token is dropped (qwen2.cpp:1060-1062)
            if why:
                req.finish_reason = self._REASONS[why]
                self.running.remove(req)
                self._dropped(req)
                req.status = "finished"
                done.append(req)
        return done
