"""A plain packer of a step's metadata, for the tests: what ``litinfer_b200.engine.batch.pack_step`` (whose work is
done by the host runtime in C++) has to produce, written out with numpy.  Same arguments, same buffer, same layout."""

from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


def attention_units(q_lens, ctx_lens, work_budget=0):
    """The attention work list, restated: every 128 tokens of a sequence of two tokens or more are a tile; a tile whose
    last token stands at position p walks p // 128 + 1 key tiles.  If the tiles are at most half of ``work_budget``, every
    tile is cut into min(8, work_budget // tiles, ceil(key tiles / 2)) parts.  Entries: tiles by key tiles per part,
    most first (ties in the order found), a tile's parts in a row; then the sequences of one token."""
    found = []
    for seq in range(len(q_lens)):
        n, c = q_lens[seq], ctx_lens[seq]
        if n < 2:
            continue
        tile = 0
        while tile * 128 < n:
            last_token = min(n, tile * 128 + 128) - 1
            position = c - n + last_token
            found.append([position // 128 + 1, seq, tile])
            tile += 1
    cut = 1
    if found and len(found) * 2 <= work_budget:
        cut = min(8, work_budget // len(found))
    for f in found:
        f.append(max(1, min(cut, (f[0] + 1) // 2)))
    order = sorted(range(len(found)), key=lambda i: (-found[i][0] / found[i][3], i))
    words = []
    for i in order:
        key_tiles, seq, tile, parts = found[i]
        for part in range(parts):
            words += [seq, tile, part + 256 * parts, 0]
    portions = len(words) // 4
    for seq in range(len(q_lens)):
        if q_lens[seq] == 1:
            words += [seq, 0, 256, 0]
    return np.asarray([portions, len(words) // 4, 0, 0] + words, dtype=np.int32)


def pack_step(items: Sequence, manager, vocab_size: int, pad_seqs: int = 0,
              max_blocks: Optional[int] = None, tokens_of_one_request: bool = False, pad_tokens: int = 0,
              pad_rows: int = 0, work_budget: int = 0):
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
    units = attention_units(q_lens, ctx.tolist(), work_budget) if max(q_lens) > 1 else None
    if units is not None:
        # a step padded to a shape keeps room for the most entries the shape can have
        room = 4 + 4 * (pad_tokens // 128 + S + work_budget) if pad_tokens else len(units)
        fields["attn_units"] = (off, room)
        off += _round_up(room, 4)
    buf = np.zeros(off, dtype=np.int32)
    if units is not None:
        o = fields["attn_units"][0]
        buf[o:o + len(units)] = units

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
            table = manager.table(manager.live[rc.request_id], gid)       # rc may stand for one token of the request
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
                  unit_slots=(int(units[0]), int(units[1])) if units is not None else (0, 0),
                  q_start=q_start.tolist(), ctx_lens=ctx.tolist(), state_slots=slots.tolist())
    return buf, layout


class PlainResidentTables:
    """What a step has to send so that a device copy of the requests' block tables (a row per state slot) is up to date,
    restated: for every live request (``forget`` when it is released: an id admitted anew starts afresh) remember how many leading
    logical pages were sent, and how many of those were sent again as given back.  Per item and group, in the order of
    the items: first the pages that have been given back since (they go back as a growing prefix), then the pages not
    sent yet, each as (slot, logical page, page id or the sink page)."""

    def __init__(self, manager):
        self.manager = manager
        self.state = {}                      # request id -> per group [sent, given_back]

    def forget(self, request_id):
        self.state.pop(request_id, None)

    def updates(self, items):
        m = self.manager
        out = [[] for _ in m.groups]
        for it in items:
            rc = it.cache
            live = m.live[rc.request_id]
            st = self.state.setdefault(rc.request_id, [[0, 0] for _ in m.groups])
            nb = -(-(rc.length + len(it.tokens)) // m.page_size)
            for g in range(len(m.groups)):
                table = m.table(live, g)
                sent, back = st[g]
                while back < nb and table[back] < 0:
                    if back < sent:
                        out[g].append((live.slot, back, m.trash_page))
                    back += 1
                while sent < nb:
                    out[g].append((live.slot, sent, m.trash_page if table[sent] < 0 else table[sent]))
                    sent += 1
                st[g] = [sent, back]
        return out
