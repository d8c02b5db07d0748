"""The step function: run a batch of (request, its next tokens) from the cache
and return the logits at the wanted places.

It runs only the tokens it is given, as one ragged batch: portions of prompts
beside single decoded tokens, cut anywhere.  It never allocates pages (the
caller did, with ``CacheManager.extend``) and mutates nothing but the cache
contents of the new tokens and each request's cached length.  LitInfer's
counterpart, ``engine_step`` (src/llaisys/models/qwen2.cpp:922-1080), also
schedules, samples and frees; here those live in the scheduler above.

Steps that consist of single tokens only can be replayed from a captured CUDA
graph per batch-size bucket: the launch sequence of a decode step is fixed, so
one graph launch replaces a few hundred kernel launches.  Steps with portions
of prompts are captured too, per shape (tokens, sequences and logit rows, each
rounded up and padded), once a shape has come back: launched plainly, a step
of a few hundred tokens is bound by the host's launches, not by the device.
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import native
from ..cache.manager import CacheManager
from ..models.decoder import DecoderModel
from ..parts.base import FixedState, Mixer
from .batch import StepContext, StepItem, context_from, pack_step, split_into_tokens


class _DecodeGraph:
    def __init__(self, graph, meta_buf, logits, layout):
        self.graph = graph
        self.meta_buf = meta_buf
        self.logits = logits
        self.layout = layout
        self.ctx = None                  # the captured step's context: tensors that the replays write (the step's block tables)


class ModelRunner:
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
    # A captured step covers contexts up to this (its block tables are that wide); longer ones are launched plainly.  The
    # attention launches do not grow with it: decode attention cuts every sequence's own context into a number of units
    # that the batch decides, and portions walk a work list.
    GRAPH_CONTEXT_CAP = 32768
    # A step of few tokens that holds portions of prompts runs through the captured decode step too, every token an item
    # of its own (batch.split_into_tokens): launched plainly, a step costs the host about 250 launches (3 ms), more than
    # the device needs for it.  Every token then reads its context by itself, so the contexts together are bounded.
    SPLIT_TOKENS = 64
    SPLIT_CONTEXT_SUM = 32768
    # Larger steps with portions of prompts: a captured graph per shape.  Tokens are rounded up in steps of 64, 128 and
    # 256 (at most an eighth of padding from 512 tokens on), sequences to the decode buckets (the padding sequences are
    # empty but the last, which takes the padding tokens), logit rows to the sequences or, if more are wanted, to the
    # tokens.
    STEP_GRAPH_TOKENS = 2048
    # Every kernel of a step may begin while the one before it still runs (programmatic dependent launch,
    # kernels.allow_overlap): a step of few tokens is a chain of short kernels (1.44 -> 1.31 ms at batch 8).  Which kinds
    # of kernel a step of more than OVERLAP_TOKENS tokens launches plainly instead is a setting (none now).  It was the
    # tcgen05 GEMMs and the attention for long portions while steps of thousands of tokens of a 7B-shaped model stopped
    # making progress about two runs in five; the cause was a CTA that held its tensor memory while it waited for the
    # kernel before (csrc/gemm_tcgen05.cu), and those kernels now take it after the wait (0 of 22 runs since, every launch
    # a dependent one).  The padded sizes of captured steps are multiples of 64, so a graph is always replayed for steps
    # of the class it was captured for.
    OVERLAP_TOKENS = 256
    BIG_STEP_NO_OVERLAP = ()
    STEP_GRAPH_LIMIT = 48               # captured shapes kept; further shapes are launched plainly
    STEP_GRAPH_LOGITS = 1 << 26         # logits (floats) a captured shape may hold

    def __init__(self, model: DecoderModel, manager: CacheManager, use_graphs: bool = False,
                 max_context: Optional[int] = None, step_graph_after: int = 1) -> None:
        self.model = model
        self.manager = manager
        self.device = model.device
        # a mixer with state of its own takes a request's tokens in order and advances its state every time the step
        # runs: its portions are never split, and nothing of such a model is captured (capturing runs the step for
        # warm-up, and a captured step would freeze which slots it updates) ...
        self._may_split = not any(isinstance(r, FixedState) for r in model.cache_requirements())

        def mixers_with_state(part):
            if isinstance(part, Mixer) and isinstance(part.cache_requirement(), FixedState):
                yield part
            for child in part.parts():
                yield from mixers_with_state(child)

        # ... except decode steps, if every such mixer says that it takes them from the device's copy of the step
        # (parts.base.Mixer.decodes_from_device); the warm-up runs of a capture then go to the spare slot
        stateful = [m for b in model.blocks for m in mixers_with_state(b)]
        self._state_in_graphs = bool(stateful) and all(getattr(m, "decodes_from_device", False) for m in stateful)
        # the block tables stay on the device (manager.groups[g].tables); a step uploads what changed
        self.resident = bool(manager.groups) and all(g.tables is not None for g in manager.groups) and os.environ.get("LITINFER_B200_RESIDENT_TABLES", "1") != "0"
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda" and (self._may_split or self._state_in_graphs)
        from .. import kernels as K

        if K.profile.enabled:
            self.use_graphs = False                        # LLAISYS_PROFILE times kernel launches: a replayed graph has none to time
        # a captured step has to cover the longest context it may meet (the width of its block tables), so that
        # length is capped; steps with a longer context run without a graph
        self.max_context = min(int(max_context or model.spec.max_position_embeddings), self.GRAPH_CONTEXT_CAP)
        # entries of the attention work list that keep every multiprocessor busy at once (engine.batch.attention_units)
        self.work_budget = 0
        if self.device.type == "cuda":
            def widths(part):
                yield getattr(part, "ctas_per_work_unit", 0)
                for child in part.parts():
                    yield from widths(child)

            widest = max((w for b in model.blocks for w in widths(b)), default=0)
            if widest:
                self.work_budget = torch.cuda.get_device_properties(self.device).multi_processor_count // widest
        if os.environ.get("LITINFER_B200_WORK_BUDGET"):
            self.work_budget = int(os.environ["LITINFER_B200_WORK_BUDGET"])       # for measurements: 0 shares nothing out
        self._graphs: Dict[int, _DecodeGraph] = {}
        # shapes of steps with portions of prompts: how often each came, and the captured ones; a shape is captured
        # when it comes for the (step_graph_after + 1)-th time, since a capture costs three plain runs
        self.step_graph_after = int(step_graph_after)
        self._shape_seen: Dict[tuple, int] = {}
        self._step_graphs: Dict[tuple, _DecodeGraph] = {}
        self._step_pool = None
        self._pinned: Optional[torch.Tensor] = None
        self._copy_done = None
        self.steps_run = 0
        self.graph_replays = 0

    # ------------------------------------------------------------------
    def _upload(self, buf: np.ndarray, into: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One host-to-device copy of the packed metadata, through pinned memory."""
        n = buf.shape[0]
        if self.device.type != "cuda":
            t = torch.from_numpy(buf.copy())
            if into is not None:
                into[:n].copy_(t)
                return into
            return t
        if self._pinned is None or self._pinned.numel() < n:
            if self._copy_done is not None:
                self._copy_done.synchronize()
            self._pinned = torch.empty(max(2 * n, 1 << 16), dtype=torch.int32).pin_memory()
            self._pinned_np = self._pinned.numpy()
            self._copy_done = torch.cuda.Event()
        else:
            self._copy_done.synchronize()         # the last copy out of the pinned buffer has finished
        self._pinned_np[:n] = buf
        if into is None:
            into = torch.empty(n, dtype=torch.int32, device=self.device)
        into[:n].copy_(self._pinned[:n], non_blocking=True)
        self._copy_done.record(torch.cuda.current_stream(self.device))
        return into

    # ------------------------------------------------------------------
    def step(self, items: Sequence[StepItem], token_source: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Float32 logits ``[wanted, vocab]`` in the order of the items and of their ``want``.

        ``token_source`` (int32 on the device, one entry per item; every item a single token): the token ids come
        from there instead of from the items, whose own ids are placeholders: they are copied over the uploaded
        ones on the device, so that a step can be fed by the sampler's output of the step before without a round
        trip through the host."""
        items = list(items)
        decode_only = all(len(it.tokens) == 1 for it in items)
        from .. import kernels as K

        if self.device.type == "cuda":
            # a captured graph keeps what held when it was captured; every shape is of one size class
            big = sum(len(it.tokens) for it in items) > self.OVERLAP_TOKENS
            K.allow_overlap(but=self.BIG_STEP_NO_OVERLAP if big else ())

        if K.profile.enabled:
            K.profile.phase = "decode" if decode_only else "prefill"
        if K.TRACE:
            import sys

            print(f"[LLAISYS] step sequences={len(items)} tokens={sum(len(it.tokens) for it in items)} "
                  f"wanted={sum(len(it.want) for it in items)} graphs={self.use_graphs}", file=sys.stderr, flush=True)
        if token_source is not None and (not decode_only or token_source.numel() != len(items)):
            raise ValueError("token_source needs one token per item and items of one token each")
        fits = decode_only and max(it.cache.length for it in items) + 1 <= self.max_context
        if self.use_graphs and fits and len(items) <= self.GRAPH_BUCKETS[-1]:
            logits = self._step_graph(items, token_source)
        elif self.use_graphs and not decode_only and self._splits(items):
            rows, base = [], 0
            for it in items:
                rows.extend(base + int(w) for w in it.want)
                base += len(it.tokens)
            logits = self._step_graph(split_into_tokens(items), None, rows)
        elif self.use_graphs and not decode_only and (shape := self._step_shape(items)) is not None:
            logits = self._step_shape_graph(items, shape)
        else:
            buf, layout = pack_step(items, self.manager, self.model.spec.vocab_size, work_budget=self.work_budget, resident=self.resident)
            ctx = context_from(self._upload(buf), layout, self.manager.page_size, self.manager)
            if token_source is not None:
                ctx.token_ids[:len(items)].copy_(token_source)
            ctx.sync_tables()
            logits = self.model.forward(ctx, self.manager.entries)
        self.manager.commit_many([it.cache for it in items], [it.cache.length + len(it.tokens) for it in items])
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------------
    def _update_room(self, items: Sequence[StepItem], T: int, S: int, one_request: bool = False) -> Optional[int]:
        """How many changes of the resident block tables a captured step of T tokens in S sequences has room for (a
        function of its shape): every sequence's new pages and as many given back.  If these items need more (requests
        that were extended without ever running), the surplus is sent now, by a small step of its own."""
        if not self.resident:
            return None
        room = 2 * (T // self.manager.page_size + S) + 2
        ids = np.asarray([it.cache.request_id for it in items], dtype=np.int32)
        lens = np.asarray([len(it.tokens) for it in items], dtype=np.int32)
        first = np.asarray([it.cache.length for it in items], dtype=np.int32)
        bound = ctypes.c_int(0)
        native.check(self.manager._lib.li_cm_table_updates_bound(self.manager._h, len(items), ids.ctypes.data, lens.ctypes.data,
                                                                 first.ctypes.data, ctypes.byref(bound)))
        if bound.value > room:
            buf, layout = pack_step(items, self.manager, self.model.spec.vocab_size, resident=True, tokens_of_one_request=one_request)
            context_from(self._upload(buf), layout, self.manager.page_size, self.manager).sync_tables()
        return room

    def _bucket(self, n: int) -> int:
        for b in self.GRAPH_BUCKETS:
            if n <= b:
                return b
        raise ValueError(n)

    def _splits(self, items: Sequence[StepItem]) -> bool:
        """Whether a step with portions of prompts is run as single tokens through the captured decode step."""
        if not self._may_split or sum(len(it.tokens) for it in items) > self.SPLIT_TOKENS:
            return False
        if max(it.cache.length + len(it.tokens) for it in items) > self.max_context:
            return False
        # token j of a portion reads length + j + 1 keys
        reads = sum(len(it.tokens) * it.cache.length + len(it.tokens) * (len(it.tokens) + 1) // 2 for it in items)
        return reads <= self.SPLIT_CONTEXT_SUM

    def _step_shape(self, items: Sequence[StepItem]) -> Optional[tuple]:
        """The padded shape (tokens, sequences, logit rows, whether single tokens stand beside the portions) under which
        a step with portions of prompts is replayed from a captured graph, or None if it is launched plainly: too large,
        a context beyond the captured attention's, a shape that has not come back yet, or a mixer with state of its
        own."""
        if not self._may_split:
            return None
        T = sum(len(it.tokens) for it in items)
        S = len(items)
        if T > self.STEP_GRAPH_TOKENS or S >= self.GRAPH_BUCKETS[-1]:
            return None
        if max(it.cache.length + len(it.tokens) for it in items) > self.max_context:
            return None
        step = 64 if T <= 512 else 128 if T <= 1024 else 256
        Tp = -(-T // step) * step
        Sp = self._bucket(S if Tp == T else S + 1)          # padding tokens need a sequence to be in
        R = sum(len(it.want) for it in items)
        if R > Sp and Tp * self.model.spec.vocab_size > self.STEP_GRAPH_LOGITS:
            return None                                     # logits of every token of a large step: not kept per shape
        # sequences of one token beside the portions go to the decode kernel: a captured shape has that launch or not
        singles = any(len(it.tokens) == 1 for it in items)
        shape = (Tp, Sp, Sp if R <= Sp else Tp, singles)
        if shape in self._step_graphs:
            return shape
        seen = self._shape_seen.get(shape, 0)
        self._shape_seen[shape] = seen + 1
        if seen < self.step_graph_after or len(self._step_graphs) >= self.STEP_GRAPH_LIMIT:
            return None
        return shape

    def _step_shape_graph(self, items: List[StepItem], shape: tuple) -> torch.Tensor:
        """A step with portions of prompts through the captured graph of its padded shape."""
        Tp, Sp, Rp, singles = shape
        max_blocks = -(-self.max_context // self.manager.page_size)
        cap = self._update_room(items, Tp, Sp)
        buf, layout = pack_step(items, self.manager, self.model.spec.vocab_size, pad_seqs=Sp, max_blocks=max_blocks,
                                pad_tokens=Tp, pad_rows=Rp, work_budget=self.work_budget, resident=self.resident, update_cap=cap)
        g = self._step_graphs.get(shape)
        if g is None:
            # the attention launch is sized for the longest portion and the longest context the shape may hold
            g = self._capture(None, max_blocks, buf, layout, max_q_len=Tp, singles=-1 if singles else 0)
            self._step_graphs[shape] = g
        if layout["fields"] != g.layout["fields"]:
            raise RuntimeError("step graph: metadata layout changed between capture and replay")
        self._upload(buf, g.meta_buf)
        g.graph.replay()
        self.graph_replays += 1
        return g.logits[:layout["R_real"]]

    def _step_graph(self, items: List[StepItem], token_source: Optional[torch.Tensor] = None,
                    rows: Optional[List[int]] = None) -> torch.Tensor:
        """A step of single tokens through a captured graph.  Every item gets its token's logits in the captured
        layout; rows that nobody wants are dropped after.  ``rows``: the items are the tokens of a step with portions
        of prompts (split_into_tokens) and these are the wanted places among them, in the order of the answer."""
        B = self._bucket(len(items))
        max_blocks = -(-self.max_context // self.manager.page_size)
        split = rows is not None
        wanted = [bool(len(it.want)) for it in items]
        g = self._graphs.get(B)
        full = [StepItem(it.cache, it.tokens, (0,)) for it in items]
        cap = self._update_room(full, B, B, one_request=split)
        buf, layout = pack_step(full, self.manager, self.model.spec.vocab_size, pad_seqs=B, max_blocks=max_blocks,
                                tokens_of_one_request=split, resident=self.resident, update_cap=cap)
        if g is None:
            g = self._capture(B, max_blocks, buf, layout)
        if layout["fields"] != g.layout["fields"]:
            raise RuntimeError("decode graph: metadata layout changed between capture and replay")
        self._upload(buf, g.meta_buf)
        if token_source is not None:
            o_tok = g.layout["fields"]["token_ids"][0]
            g.meta_buf[o_tok:o_tok + len(items)].copy_(token_source)
        g.graph.replay()
        self.graph_replays += 1
        if rows is None:
            rows = [i for i, w in enumerate(wanted) if w]
        if not rows:
            return g.logits[:0]
        if rows == list(range(rows[0], rows[0] + len(rows))):
            return g.logits[rows[0]:rows[0] + len(rows)]        # a run of rows (the usual case: every item's, or the last token's): a view
        from .. import kernels as K

        out = torch.empty((len(rows), g.logits.shape[1]), dtype=torch.float32, device=self.device)
        K.gather_rows(g.logits, torch.tensor(rows, dtype=torch.int32, device=self.device), out)
        return out

    def _capture(self, B: Optional[int], max_blocks: int, buf: np.ndarray, layout, max_q_len: int = 1, singles: int = 0) -> _DecodeGraph:
        """Capture the model's forward pass over the packed step.  ``B``: the decode bucket it is kept under (None: the
        caller keeps it).  Graphs of padded steps share one memory pool: they run one after the other on one stream, and
        a step's logits are read before the next step starts."""
        meta = torch.zeros(buf.shape[0], dtype=torch.int32, device=self.device)
        self._upload(buf, meta)
        lay = dict(layout)
        # a captured attention launch must cover any context up to the maximum
        lay["max_ctx_len"] = self.max_context
        lay["max_q_len"] = max_q_len
        lay["singles"] = singles
        if "attn_units" in lay["fields"]:                  # the captured launch covers every entry the list has room for
            room = (lay["fields"]["attn_units"][1] - 4) // 4
            lay["unit_slots"] = (room, room)
        ctx = context_from(meta, lay, self.manager.page_size, self.manager)
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            if not self._may_split:
                # state of fixed size: the warm-up runs must advance nobody's, so every sequence names the spare slot
                # meanwhile (its row of the resident block tables names the sink page: keys and values of the step's
                # tokens go there too, and are written to their places by the first replay)
                o, n = lay["fields"]["state_slots"]
                meta[o:o + n].fill_(self.manager.max_requests)
            for _ in range(2):                    # warm-up outside capture (first-call set-up, allocator)
                ctx.scratch.clear()
                ctx.sync_tables()
                self.model.forward(ctx, self.manager.entries)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)
        if not self._may_split:
            self._upload(buf, meta)
        graph = torch.cuda.CUDAGraph()
        if B is None and self._step_pool is None:
            self._step_pool = torch.cuda.graph_pool_handle()
        # what the parts make once per step (a table of rotation angles) is made inside the capture, from the step's
        # metadata, not taken over from the warm-up runs
        ctx.scratch.clear()
        with torch.cuda.graph(graph, pool=None if B is not None else self._step_pool):
            ctx.sync_tables()                          # the step's block tables from the resident ones: part of every replay
            logits = self.model.forward(ctx, self.manager.entries)
        g = _DecodeGraph(graph, meta, logits, lay)
        g.ctx = ctx                                    # the step's block tables, which every replay fills again, live as long as the graph
        if B is not None:
            self._graphs[B] = g
        return g
