"""The metadata of one step: which tokens run, where they sit, what they read.

A step is a list of :class:`StepItem`: a live request, its next tokens (a
portion of a prompt, or one decoded token) and the places among them whose
logits are wanted.  All items form one ragged batch.  The metadata is built on
the host once per step, packed into one int32 buffer and uploaded with one
copy; LitInfer rebuilds and uploads its block table per layer
(src/llaisys/models/qwen2.cpp:993-1007).

Layout of the packed buffer (all int32): token_ids[T] | positions[T] |
seq_of_token[T] | q_start[S+1] | ctx_lens[S] | old_lens[S] | state_slots[S] |
logit_rows[R] | per group: slot_mapping[T] | block_table[S * max_blocks] | attn_units (steps with portions of prompts:
the work list of the attention kernel for long portions, :func:`attention_units`).  With ``pad_seqs``
the batch is padded to that many one-token items that write to the sink page
and whose results nobody reads (a captured decode step has a fixed size); with
``pad_tokens`` to a fixed count of tokens, sequences and rows (a captured step
with portions of prompts).  The buffer is filled by the host runtime
(``li_cm_pack_step`` in ``csrc/host/runtime.cpp``), which holds the block tables.
"""

from __future__ import annotations

import ctypes
import functools
import itertools
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import native
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
    # steps with portions of prompts: the attention work list (attention_units) and how many of its entries to launch
    # when single tokens go to a kernel of their own / when they do not
    attn_units: Optional[torch.Tensor] = None
    attn_unit_slots: tuple = (0, 0)
    # resident block tables: per group (the resident tensor, the step's changes, the step's table to fill, the sink page)
    pending_tables: list = field(default_factory=list)
    # what parts make once per step and share between the layers (keyed by the part), e.g. a table of rotation angles
    scratch: dict = field(default_factory=dict)

    def sync_tables(self) -> None:
        """Apply the step's changes to the resident block tables and fill the step's tables from them (one small kernel
        per cache group).  Applying twice gives the same."""
        from .. import kernels as K

        for tables, updates, out, trash in self.pending_tables:
            K.table_gather(tables, updates, self.state_slots, out, trash)

    def group(self, gid: int) -> GroupView:
        return self.groups[gid]


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


class _TokenOf:
    """One token of an item, seen as a sequence of its own: the request's cache as far as this token."""

    __slots__ = ("request_id", "length", "old_length", "slot")

    def __init__(self, rc, offset: int) -> None:
        self.request_id = rc.request_id
        self.length = rc.length + offset
        self.old_length = rc.length
        self.slot = rc.slot


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


_FIELDS = ("token_ids", "positions", "seq_of_token", "q_start", "ctx_lens", "old_lens", "state_slots", "logit_rows")


TOKEN_TILE = 128          # tokens of a portion that one CTA of the attention kernel for long portions takes
KEY_TILE = 128            # keys it walks at a time
MIN_PART_TILES = 2        # fewest key tiles a CTA takes when a tile of tokens is shared out
MAX_PARTS = 8             # most CTAs that share a tile of tokens


def attention_units(q_lens: Sequence[int], ctx_lens: Sequence[int], work_budget: int = 0) -> np.ndarray:
    """The work list of the attention kernel for long portions (csrc/attention_tcgen05.cu): one entry per tile of 128
    tokens of every sequence of the step, the tile that walks the most keys first (the kernel's time is that of its
    longest CTA, so the long ones must not start late).  ``work_budget``: how many entries keep every multiprocessor
    busy at once (multiprocessors // CTAs per entry).  A step with at most half that many tiles of tokens (a portion
    of a prompt behind a long context) has each tile's keys shared out among up to MAX_PARTS entries of at least
    MIN_PART_TILES key tiles, next to each other in the list; the kernel adds their partial results up.

    int32: [entries of portions (two tokens and more), all entries, 0, 0, then per entry: sequence, tile,
    part | parts << 8, 0].  The sequences of one token come last: they are launched only where no decode kernel takes
    them."""
    tiles, singles = [], []
    for s, (n, c) in enumerate(zip(q_lens, ctx_lens)):
        if n == 1:
            singles.append(s)
        for t in range(-(-n // TOKEN_TILE) if n > 1 else 0):
            last = c - n + min(n, (t + 1) * TOKEN_TILE) - 1          # position of the tile's last token = the last key it sees
            tiles.append((last // KEY_TILE + 1, s, t))
    nsplit = 1
    if tiles and 2 * len(tiles) <= work_budget:
        nsplit = min(MAX_PARTS, work_budget // len(tiles))
    entries = []
    weighed = [(k, s, t, max(1, min(nsplit, -(-k // MIN_PART_TILES)))) for k, s, t in tiles]
    weighed.sort(key=lambda e: -(e[0] / e[3]))
    for _, s, t, parts in weighed:
        entries.extend((s, t, part | (parts << 8), 0) for part in range(parts))
    portions = len(entries)
    entries.extend((s, 0, 1 << 8, 0) for s in singles)
    out = np.zeros(4 + 4 * len(entries), dtype=np.int32)
    out[0], out[1] = portions, len(entries)
    if entries:
        out[4:] = np.asarray(entries, dtype=np.int32).reshape(-1)
    return out


@functools.lru_cache(maxsize=512)
def _fields(T: int, S: int, R: int, G: int, mb: int, U: int = 0, cap: int = -1):
    """Where each field starts in the packed buffer (16-byte aligned starts), the buffer's length (the host runtime's
    fields, then ``U`` words of attention work list), and the starts as the array the host runtime takes.  ``cap`` >= 0:
    instead of a group's block tables the buffer carries up to that many changes of the resident ones."""
    fields = {}
    off = 0
    for name, n in zip(_FIELDS, (T, T, T, S + 1, S, S, S, R)):
        fields[name] = (off, n)
        off += _round_up(max(n, 1), 4)
    for gid in range(G):
        fields[f"slot_mapping{gid}"] = (off, T)
        off += _round_up(max(T, 1), 4)
        if cap >= 0:
            fields[f"table_updates{gid}"] = (off, 1 + 3 * cap)
            off += _round_up(1 + 3 * cap, 4)
        else:
            fields[f"block_table{gid}"] = (off, S * mb)
            off += _round_up(max(S * mb, 1), 4)
    starts = np.asarray([o for o, _ in fields.values()], dtype=np.int32)
    if U:
        fields["attn_units"] = (off, U)
        off += _round_up(U, 4)
    return fields, off, starts


def _ints(values) -> np.ndarray:
    return np.asarray(values, dtype=np.int32) if len(values) else np.zeros(1, dtype=np.int32)


def pack_step(items: Sequence[StepItem], manager: CacheManager, vocab_size: int, pad_seqs: int = 0,
              max_blocks: Optional[int] = None, tokens_of_one_request: bool = False, pad_tokens: int = 0,
              pad_rows: int = 0, work_budget: int = 0, resident: bool = False, update_cap: Optional[int] = None):
    """Host side: validate the items and fill the packed int32 array (the host runtime does both, in C++).

    Returns (array, layout) where layout maps field name -> (offset, length) and
    carries the scalar sizes.  Pages for all tokens must already be allocated.
    ``tokens_of_one_request``: the items come from :func:`split_into_tokens`, several may belong to one request.
    ``pad_tokens`` (with ``pad_seqs`` and ``pad_rows``): the step is padded to exactly that many tokens, sequences
    and logit rows, for a captured step of a fixed shape: the padding sequences are empty but the last, which takes
    the padding tokens; it starts at position 0, writes to the sink page and sees nothing else; the real rows come
    first among the logit rows, and ``layout["R_real"]`` says how many they are.  Without ``pad_tokens`` the padding
    sequences hold one token each and want its row.
    ``work_budget``: see :func:`attention_units`; a step with portions of prompts carries that list (a padded one with
    room for the most entries its shape can have).
    ``resident``: the device keeps the requests' block tables (``manager.groups[g].tables``, a row per state slot); the
    buffer then carries, instead of a table per sequence, what those lack for this step's requests (a count and
    triples of slot, logical page, page id; room for ``update_cap`` of them, by default as many as it can be), and what
    is packed counts as sent: the caller uploads it and applies it (``StepContext.sync_tables``) before packing again.
    """
    S_real = len(items)
    if S_real == 0:
        raise ValueError("a step needs at least one item")
    caches = [it.cache for it in items]
    q_lens = [len(it.tokens) for it in items]
    if min(q_lens) <= 0:
        raise ValueError("an item without tokens")
    starts = [c.length for c in caches]
    olds = [c.old_length for c in caches] if tokens_of_one_request else starts
    counts = [len(it.want) for it in items]
    S = max(S_real, pad_seqs)
    T_real, R_real = sum(q_lens), sum(counts)
    page = manager.page_size
    need_blocks = max(-(-(st + n) // page) for st, n in zip(starts, q_lens))
    if pad_tokens:
        rest = pad_tokens - T_real
        if rest < 0 or (rest > 0 and S == S_real):
            raise ValueError(f"{T_real} tokens in {S_real} sequences cannot be padded to {pad_tokens} tokens in {S}")
        if R_real > pad_rows:
            raise ValueError(f"{R_real} wanted rows do not fit the {pad_rows} of the padded step")
        T, R = int(pad_tokens), int(pad_rows)
        need_blocks = max(need_blocks, -(-rest // page))
    else:
        T, R = T_real + S - S_real, R_real + S - S_real
    G = len(manager.groups)
    mb = max(need_blocks, max_blocks or 0, 1)
    units = None
    lens_all, ctx_all = list(q_lens), [st + n for st, n in zip(starts, q_lens)]
    if pad_tokens and rest > 0:                            # the padding tokens are the last sequence's, from position 0
        lens_all += [0] * (S - S_real - 1) + [rest]
        ctx_all += [0] * (S - S_real - 1) + [rest]
    if max(lens_all) > 1:
        units = attention_units(lens_all, ctx_all, work_budget)
        # a padded step is replayed from a captured launch, whose list has room for any step of its shape
        U = 4 + 4 * (pad_tokens // TOKEN_TILE + S + work_budget) if pad_tokens else len(units)
    ids = _ints([c.request_id for c in caches])
    lens, first = _ints(q_lens), _ints(starts)
    cap = -1
    if resident:
        if mb > manager.table_blocks:
            raise ValueError(f"a context of {mb} pages is beyond the resident block tables ({manager.table_blocks} pages a request)")
        cap = update_cap
        if cap is None:
            bound = ctypes.c_int(0)
            native.check(manager._lib.li_cm_table_updates_bound(manager._h, S_real, ids.ctypes.data, lens.ctypes.data, first.ctypes.data,
                                                                ctypes.byref(bound)))
            cap = bound.value
    fields, total, offsets = _fields(T, S, R, G, mb, U if units is not None else 0, cap)
    buf = np.zeros(total, dtype=np.int32)
    if units is not None:
        o = fields["attn_units"][0]
        buf[o:o + len(units)] = units
    if T_real == S_real:
        tokens = _ints([it.tokens[0] for it in items])
    else:
        tokens = _ints(list(itertools.chain.from_iterable(it.tokens for it in items)))
    wants = _ints(list(itertools.chain.from_iterable(it.want for it in items))) if R_real else _ints(())
    old, cnt = _ints(olds), _ints(counts)
    info = np.zeros(4, dtype=np.int32)
    native.check(manager._lib.li_cm_pack_step(
        manager._h, S_real, ids.ctypes.data, lens.ctypes.data, first.ctypes.data, old.ctypes.data, tokens.ctypes.data,
        cnt.ctypes.data, wants.ctypes.data, int(vocab_size), S, T, R, int(pad_tokens), mb, 1 if tokens_of_one_request else 0,
        manager.trash_page, manager.trash_slot, offsets.ctypes.data, buf.ctypes.data, total, info.ctypes.data, cap))

    def host(name):
        o, n = fields[name]
        return buf[o:o + n].tolist()

    layout = dict(fields=fields, T=T, S=S, R=R, R_real=int(info[0]), G=G, max_blocks=mb, singles=int(info[3]),
                  max_q_len=int(info[1]), max_ctx_len=int(info[2]),
                  unit_slots=(int(units[0]), int(units[1])) if units is not None else (0, 0),
                  q_start=host("q_start"), ctx_lens=host("ctx_lens"), state_slots=host("state_slots"))
    return buf, layout


def context_from(device_buf: torch.Tensor, layout, page_size: int, resident: Optional[CacheManager] = None) -> StepContext:
    """Views into the uploaded buffer.  ``resident``: the manager whose resident block tables the step was packed for;
    the step's own tables are then made on the device by :meth:`StepContext.sync_tables`, which the caller runs before
    the model (inside the capture, for a captured step)."""
    f = layout["fields"]

    def view(name):
        o, n = f[name]
        return device_buf[o:o + n]

    S, mb = layout["S"], layout["max_blocks"]
    pending = []
    if "table_updates0" in f or (layout["G"] and "block_table0" not in f):
        if resident is None:
            raise ValueError("this step was packed for resident block tables: context_from needs the manager")
        groups = []
        for g in range(layout["G"]):
            table = torch.empty((S, mb), dtype=torch.int32, device=device_buf.device)
            pending.append((resident.groups[g].tables, view(f"table_updates{g}"), table, resident.trash_page))
            groups.append(GroupView(table, view(f"slot_mapping{g}"), mb, page_size))
    else:
        groups = [GroupView(view(f"block_table{g}").view(S, mb), view(f"slot_mapping{g}"), mb, page_size) for g in range(layout["G"])]
    return StepContext(
        pending_tables=pending,
        num_tokens=layout["T"], num_seqs=S, num_logit_rows=layout["R"],
        token_ids=view("token_ids"), positions=view("positions"), seq_of_token=view("seq_of_token"),
        q_start=view("q_start"), ctx_lens=view("ctx_lens"), state_slots=view("state_slots"), old_lens=view("old_lens"),
        logit_rows=view("logit_rows"), groups=groups,
        max_q_len=layout["max_q_len"], max_ctx_len=layout["max_ctx_len"], num_single=layout.get("singles", 0),
        attn_units=view("attn_units") if "attn_units" in f else None, attn_unit_slots=tuple(layout.get("unit_slots", (0, 0))),
        host_q_start=layout["q_start"], host_ctx_lens=layout["ctx_lens"], host_state_slots=layout["state_slots"])
