"""The metadata of one step: which tokens run, where they sit, what they read.

A step is a list of :class:`StepItem`: a live request, its next tokens (a
portion of a prompt, or one decoded token) and the places among them whose
logits are wanted.  All items form one ragged batch.  The metadata is built on
the host once per step, packed into one int32 buffer and uploaded with one
copy; LitInfer rebuilds and uploads its block table per layer
(src/llaisys/models/qwen2.cpp:993-1007).

Layout of the packed buffer (all int32): token_ids[T] | positions[T] |
seq_of_token[T] | q_start[S+1] | ctx_lens[S] | old_lens[S] | state_slots[S] |
logit_rows[R] | per group: slot_mapping[T] | block_table[S * max_blocks].  With ``pad_seqs``
the batch is padded to that many one-token items that write to the sink page
and whose results nobody reads (a captured decode step has a fixed size).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache


@dataclass
class StepItem:
    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class GroupView:
    block_table: torch.Tensor        # [S, max_blocks] int32, page ids (sink page where none)
    slot_mapping: torch.Tensor       # [T] int32, page * page_size + offset of each token
    max_blocks: int
    page_size: int


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    num_logit_rows: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    q_start: torch.Tensor
    ctx_lens: torch.Tensor
    state_slots: torch.Tensor
    logit_rows: torch.Tensor
    groups: List[GroupView]
    max_q_len: int
    max_ctx_len: int
    # host copies, for parts that loop over requests on the host
    host_q_start: List[int] = field(default_factory=list)
    host_ctx_lens: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)
    # [S] int32: how many keys of each sequence were in the cache before this step (a sequence's own tokens of this step
    # come after them; where a step's sequences are the tokens of one request, so do that request's earlier tokens)
    old_lens: Optional[torch.Tensor] = None
    # how many sequences of a step with longer portions have one token (they can go to a decode kernel); negative: not
    # known (a captured step that may hold any)
    num_single: int = 0
    # what parts make once per step and share between the layers (keyed by the part), e.g. a table of rotation angles
    scratch: dict = field(default_factory=dict)

    def group(self, gid: int) -> GroupView:
        return self.groups[gid]


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


class _TokenOf:
    """One token of an item, seen as a sequence of its own: the request's cache as far as this token."""

    __slots__ = ("request_id", "length", "old_length", "slot", "tables")

    def __init__(self, rc, offset: int) -> None:
        self.request_id = rc.request_id
        self.length = rc.length + offset
        self.old_length = rc.length
        self.slot = rc.slot
        self.tables = rc.tables


def split_into_tokens(items: Sequence[StepItem]) -> List[StepItem]:
    """Every token of every item as an item of one token that wants its logits.  A portion of a prompt is the same work
    as that many decoded tokens whose contexts end one after the other: each token's keys and values are in the cache
    before any attention of the step runs.  Only for mixers without state of their own per request."""
    seen = set()
    out = []
    for it in items:
        if it.cache.request_id in seen:
            raise ValueError(f"request {it.cache.request_id} appears twice in one step")
        seen.add(it.cache.request_id)
        if len(it.tokens) == 0:
            raise ValueError("an item without tokens")
        for w in it.want:
            if not 0 <= w < len(it.tokens):
                raise IndexError(f"request {it.cache.request_id}: wanted place {w} is outside its {len(it.tokens)} tokens")
        out.extend(StepItem(_TokenOf(it.cache, j), (t,), (0,)) for j, t in enumerate(it.tokens))
    return out


def pack_step(items: Sequence[StepItem], manager: CacheManager, vocab_size: int, pad_seqs: int = 0,
              max_blocks: Optional[int] = None, tokens_of_one_request: bool = False, pad_tokens: int = 0,
              pad_rows: int = 0):
    """Host side: validate the items and fill the packed int32 array.

    Returns (array, layout) where layout maps field name -> (offset, length) and
    carries the scalar sizes.  Pages for all tokens must already be allocated.
    ``tokens_of_one_request``: the items come from :func:`split_into_tokens`, several may belong to one request.
    ``pad_tokens`` (with ``pad_seqs`` and ``pad_rows``): the step is padded to exactly that many tokens, sequences
    and logit rows, for a captured step of a fixed shape: the padding sequences are empty but the last, which takes
    the padding tokens; it starts at position 0, writes to the sink page and sees nothing else; the real rows come
    first among the logit rows, and ``layout["R_real"]`` says how many they are.
    """
    S_real = len(items)
    if S_real == 0:
        raise ValueError("a step needs at least one item")
    S = max(S_real, pad_seqs)
    q_lens = [len(it.tokens) for it in items]
    if min(q_lens) <= 0:
        raise ValueError("an item without tokens")
    if pad_tokens:
        rest = pad_tokens - sum(q_lens)
        if rest < 0 or (rest > 0 and S == S_real):
            raise ValueError(f"{sum(q_lens)} tokens in {S_real} sequences cannot be padded to {pad_tokens} tokens in {S}")
        q_lens += [0] * (S - S_real)
        q_lens[-1] += rest
    else:
        q_lens += [1] * (S - S_real)
    T = sum(q_lens)
    page = manager.page_size
    q_start = np.zeros(S + 1, dtype=np.int32)
    np.cumsum(q_lens, out=q_start[1:])
    ctx = np.empty(S, dtype=np.int32)
    old = np.zeros(S, dtype=np.int32)
    slots = np.empty(S, dtype=np.int32)
    token_ids = np.zeros(T, dtype=np.int32)
    positions = np.zeros(T, dtype=np.int32)
    seq_of = np.empty(T, dtype=np.int32)
    rows: List[int] = []
    seen = set()
    for s, it in enumerate(items):
        rc = it.cache
        if rc.request_id in seen and not tokens_of_one_request:
            raise ValueError(f"request {rc.request_id} appears twice in one step")
        seen.add(rc.request_id)
        n, lo = q_lens[s], int(q_start[s])
        toks = np.asarray(it.tokens, dtype=np.int64)
        if toks.min() < 0 or toks.max() >= vocab_size:
            raise IndexError(f"request {rc.request_id}: token id outside [0, {vocab_size})")
        token_ids[lo:lo + n] = toks
        positions[lo:lo + n] = np.arange(rc.length, rc.length + n)
        seq_of[lo:lo + n] = s
        ctx[s] = rc.length + n
        old[s] = getattr(rc, "old_length", rc.length)
        slots[s] = rc.slot
        for w in it.want:
            if not 0 <= w < n:
                raise IndexError(f"request {rc.request_id}: wanted place {w} is outside its {n} tokens")
            rows.append(lo + int(w))
    R_real = len(rows)
    for s in range(S_real, S):
        lo, n = int(q_start[s]), q_lens[s]
        seq_of[lo:lo + n] = s
        positions[lo:lo + n] = np.arange(n)
        ctx[s] = n
        slots[s] = manager.trash_slot
        if not pad_tokens:
            rows.append(lo)                  # padded items want a row too: the layout depends on S alone
    if pad_tokens:
        if len(rows) > pad_rows:
            raise ValueError(f"{len(rows)} wanted rows do not fit the {pad_rows} of the padded step")
        rows.extend([T - 1] * (pad_rows - len(rows)))
    R = len(rows)
    need_blocks = max(-(-int(c) // page) for c in ctx)
    G = len(manager.groups)
    mb = max(need_blocks, max_blocks or 0, 1)
    fields = {}
    off = 0

    def place(name, n):
        nonlocal off
        fields[name] = (off, n)
        off += _round_up(max(n, 1), 4)       # 16-byte aligned starts

    for name, n in (("token_ids", T), ("positions", T), ("seq_of_token", T), ("q_start", S + 1),
                    ("ctx_lens", S), ("old_lens", S), ("state_slots", S), ("logit_rows", R)):
        place(name, n)
    for gid in range(G):
        place(f"slot_mapping{gid}", T)
        place(f"block_table{gid}", S * mb)
    buf = np.zeros(off, dtype=np.int32)

    def put(name, arr):
        o, n = fields[name]
        buf[o:o + n] = arr

    put("token_ids", token_ids)
    put("positions", positions)
    put("seq_of_token", seq_of)
    put("q_start", q_start)
    put("ctx_lens", ctx)
    put("old_lens", old)
    put("state_slots", slots)
    put("logit_rows", np.asarray(rows, dtype=np.int32))
    trash = manager.trash_page
    for gid in range(G):
        bt = np.full((S, mb), trash, dtype=np.int32)
        sm = trash * page + positions % page             # padding tokens: the sink page, the slot of their position
        for s, it in enumerate(items):
            rc = it.cache
            table = rc.tables[gid]
            nb = -(-int(ctx[s]) // page)
            if len(table) < nb:
                raise RuntimeError(f"request {rc.request_id}: pages for {int(ctx[s])} tokens are not allocated (group {gid})")
            row = np.asarray(table[:nb], dtype=np.int32)
            row = np.where(row < 0, trash, row)
            bt[s, :nb] = row
            lo, n = int(q_start[s]), q_lens[s]
            pos = positions[lo:lo + n]
            pages = row[pos // page]
            if (pages == trash).any():
                raise RuntimeError(f"request {rc.request_id}: a new token falls on a page that was given back (group {gid})")
            sm[lo:lo + n] = pages * page + pos % page
        put(f"block_table{gid}", bt.reshape(-1))
        put(f"slot_mapping{gid}", sm)
    singles = sum(1 for q in q_lens[:S_real] if q == 1) if max(q_lens) > 1 else 0
    layout = dict(fields=fields, T=T, S=S, R=R, R_real=R_real, G=G, max_blocks=mb, singles=singles, max_q_len=max(q_lens), max_ctx_len=int(ctx.max()),
                  q_start=q_start.tolist(), ctx_lens=ctx.tolist(), state_slots=slots.tolist())
    return buf, layout


def context_from(device_buf: torch.Tensor, layout, page_size: int) -> StepContext:
    """Views into the uploaded buffer."""
    f = layout["fields"]

    def view(name):
        o, n = f[name]
        return device_buf[o:o + n]

    S, mb = layout["S"], layout["max_blocks"]
    groups = [GroupView(view(f"block_table{g}").view(S, mb), view(f"slot_mapping{g}"), mb, page_size) for g in range(layout["G"])]
    return StepContext(
        num_tokens=layout["T"], num_seqs=S, num_logit_rows=layout["R"],
        token_ids=view("token_ids"), positions=view("positions"), seq_of_token=view("seq_of_token"),
        q_start=view("q_start"), ctx_lens=view("ctx_lens"), state_slots=view("state_slots"), old_lens=view("old_lens"),
        logit_rows=view("logit_rows"), groups=groups,
        max_q_len=layout["max_q_len"], max_ctx_len=layout["max_ctx_len"], num_single=layout.get("singles", 0),
        host_q_start=layout["q_start"], host_ctx_lens=layout["ctx_lens"], host_state_slots=layout["state_slots"])
