"""The cache manager's bookkeeping (no page lost, held twice or freed twice,
under random orders of requests; windows give pages back) and the scheduler's
decisions (budget, portions, admission, what happens when pages run out,
finishing).  Host-only logic: no GPU, no model."""

from __future__ import annotations

import random

import pytest
import torch

from litinfer_b200.cache import CacheManager, OutOfPages, PoolError
from pool_face import PagePool
from litinfer_b200.engine import RequestRefused, Scheduler, SchedulerConfig
from litinfer_b200.parts import FixedState, PagedKV
from litinfer_b200.sampling import SamplingParams


def manager(num_pages=8, max_requests=4, window=None, two_groups=False, allocate=False):
    reqs = [PagedKV(2, 16, None), PagedKV(2, 16, window)] if two_groups else [PagedKV(2, 16, window)] * 2
    return CacheManager(reqs, [None, None], num_pages, 16, max_requests, torch.float32, "cpu", allocate=allocate)


# --------------------------------------------------------------------------
# pool
# --------------------------------------------------------------------------

def test_pool_is_lifo_and_checks_ownership():
    p = PagePool(4)
    assert [p.alloc(1), p.alloc(1), p.alloc(2)] == [0, 1, 2]          # page 0 first (block_kv_cache.hpp:34-37)
    p.free(1, 1)
    assert p.alloc(3) == 1                                            # the page just given back is used again at once
    with pytest.raises(PoolError, match="held by 3"):
        p.free(1, 1)
    p.free(1, 3)
    with pytest.raises(PoolError, match="freed twice"):
        p.free(1, 3)
    with pytest.raises(PoolError, match="outside"):
        p.free(9, 1)
    p.alloc(1), p.alloc(1)
    with pytest.raises(OutOfPages):
        p.alloc(1)
    p.check()


def test_groups_and_layouts():
    m = CacheManager([PagedKV(2, 16, None), PagedKV(2, 16, 24), PagedKV(2, 16, None), None, FixedState((5,), torch.float32)],
                     [None, None, None, 0, None], 6, 16, 3, torch.float32, "cpu")
    assert len(m.groups) == 2 and m.groups[0].entries == [0, 2] and m.groups[1].entries == [1]
    assert [e.kind for e in m.entries] == ["paged", "paged", "paged", "paged", "state"]
    assert m.entries[3].writes is False and m.entries[3].k is m.entries[0].k            # reads entry 0's cache
    assert m.entries[0].k.shape == (7, 2, 16, 16) and m.entries[0].v.shape == (7, 2, 16, 16)
    assert m.entries[4].state.shape == (4, 5)
    assert m.bytes_per_page() == (2 + 1) * 2 * 2 * 16 * 16 * 4
    with pytest.raises(ValueError, match="page_size"):
        CacheManager([PagedKV(1, 16)], [None], 4, 24, 1, torch.float32, "cpu", allocate=False)


def test_state_slot_is_cleared_at_admission():
    m = CacheManager([FixedState((3,), torch.float32)], [None], 2, 16, 2, torch.float32, "cpu")
    rc = m.admit(7)
    m.entries[0].state[rc.slot] += 5.0
    m.release(rc)
    rc2 = m.admit(8)
    assert rc2.slot == rc.slot and not m.entries[0].state[rc2.slot].any()


# --------------------------------------------------------------------------
# manager under random orders
# --------------------------------------------------------------------------

@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 20])
def test_random_orders_keep_every_page_accounted_for(seed, window):
    rnd = random.Random(seed)
    m = manager(num_pages=12, max_requests=5, window=window, two_groups=True)
    live = {}
    next_id = 0
    G = len(m.groups)                     # the two entries share a group unless one has a window
    for _ in range(400):
        op = rnd.random()
        if op < 0.25 and m.num_free_slots():
            live[next_id] = m.admit(next_id)
            next_id += 1
        elif op < 0.8 and live:
            rid = rnd.choice(list(live))
            rc = live[rid]
            grow = rnd.choice([1, 1, 1, 2, 7, 16, 33])
            before = [m.num_free_pages(g) for g in range(G)]
            tables = [list(t) for t in rc.tables]
            if m.can_extend(rc, rc.length + grow):
                m.extend(rc, rc.length + grow)
                m.commit(rc, rc.length + grow)
            else:
                with pytest.raises(OutOfPages):
                    m.extend(rc, rc.length + grow)
                # all or nothing: a refused extension changes nothing
                assert [m.num_free_pages(g) for g in range(G)] == before and [list(t) for t in rc.tables] == tables
        elif live:
            rid = rnd.choice(list(live))
            m.release(live.pop(rid))
        m.check()
        for rc in live.values():
            # every position a further query may read lies on a held page
            for gid, g in enumerate(m.groups):
                lo = 0 if g.key.window is None else max(0, rc.length - g.key.window + 1)
                for pos in range(lo, rc.length):
                    assert rc.tables[gid][pos // 16] >= 0
    for rc in list(live.values()):
        m.release(rc)
    m.check()
    assert all(m.num_free_pages(g) == 12 for g in range(G)) and m.num_free_slots() == 5


def test_window_gives_pages_back_once_they_are_behind_it():
    m = manager(num_pages=8, window=20)
    rc = m.admit(0)
    m.extend(rc, 50)
    assert m.num_free_pages(0) == 4
    m.commit(rc, 50)                      # next query is at 50 and reads keys 31..: pages 0 (0-15) is behind, page 1 (16-31) is not
    assert rc.tables[0][:2] == [CacheManager.RELEASED, 1] and m.num_free_pages(0) == 5
    m.extend(rc, 52)
    m.commit(rc, 52)                      # reads 33..: page 1 is behind now
    assert rc.tables[0][1] == CacheManager.RELEASED and m.num_free_pages(0) == 6
    with pytest.raises(PoolError, match="given back"):
        m.slot_of(rc, 0, 20)
    assert m.slot_of(rc, 0, 40) == rc.tables[0][2] * 16 + 8
    m.release(rc)
    m.check()
    with pytest.raises(PoolError, match="not live"):
        m.release(rc)


# --------------------------------------------------------------------------
# scheduler
# --------------------------------------------------------------------------

def run(s: Scheduler, steps=10_000, token=lambda req: 1):
    """Drive the scheduler with a model that always answers ``token(request)``."""
    log = []
    for _ in range(steps):
        if not s.has_unfinished():
            break
        items = s.schedule()
        log.append([(it.request.id, it.start, it.count, it.wants_logits) for it in items])
        for it in items:                                    # what the step function does
            s.manager.commit(it.request.cache, it.start + it.count)
        s.update(items, [token(it.request) if it.wants_logits else None for it in items])
        s.manager.check()
    return log


def test_budget_portions_and_decode_first():
    m = manager(num_pages=64, max_requests=8)
    s = Scheduler(m, SchedulerConfig(max_num_seqs=8, max_tokens_per_step=24, prefill_chunk=16), 512)
    a = s.add_request(list(range(40)), 3)
    b = s.add_request(list(range(10)), 3)
    log = run(s)
    assert log[0] == [(a, 0, 16, False), (b, 0, 8, False)]             # portions under the budget of 24
    assert log[1] == [(a, 16, 16, False), (b, 8, 2, True)]             # b's prompt ends: its logits are wanted
    assert log[2] == [(b, 10, 1, True), (a, 32, 8, True)]              # decoding requests first, then portions
    assert all(sum(n for _, _, n, _ in step) <= 24 for step in log)
    assert s.requests[a].generated == [1, 1, 1] and s.requests[a].finish_reason == "length"
    assert m.num_free_pages(0) == 64 and m.num_free_slots() == 8


def test_admission_is_fifo_and_bounded():
    m = manager(num_pages=64, max_requests=2)
    s = Scheduler(m, SchedulerConfig(max_num_seqs=2, max_tokens_per_step=64, prefill_chunk=64), 512)
    ids = [s.add_request([1, 2, 3], 2) for _ in range(5)]
    log = run(s)
    first_seen = {}
    for i, step in enumerate(log):
        assert len(step) <= 2
        for rid, *_ in step:
            first_seen.setdefault(rid, i)
    assert [first_seen[r] for r in ids] == sorted(first_seen[r] for r in ids)
    assert all(s.requests[r].finished for r in ids)


def test_requests_that_can_never_fit_are_refused():
    m = manager(num_pages=4)
    s = Scheduler(m, SchedulerConfig(), 100)
    with pytest.raises(RequestRefused, match="positions"):
        s.add_request([1] * 90, 12)                    # 90 + 12 - 1 > 100 (python/llaisys/models/qwen2.py:342-346)
    s.add_request([1] * 60, 5)                         # 64 tokens: exactly the 4 pages
    with pytest.raises(RequestRefused, match="pages"):
        s.add_request([1] * 60, 6)
    with pytest.raises(RequestRefused, match="at least one"):
        s.add_request([], 4)
    big = Scheduler(manager(num_pages=64), SchedulerConfig(), 1024)
    assert big.requests[big.add_request([1], 0)].max_new_tokens == 512  # <= 0 means 512 (qwen2.cpp:795)


def test_when_pages_run_out_the_youngest_is_preempted_and_recomputed():
    m = manager(num_pages=5, max_requests=4)
    s = Scheduler(m, SchedulerConfig(max_num_seqs=4, max_tokens_per_step=64, prefill_chunk=32), 512)
    a = s.add_request([1] * 30, 30)        # grows to 59 tokens: 4 pages
    b = s.add_request([2] * 30, 30)
    log = run(s)
    ra, rb = s.requests[a], s.requests[b]
    assert ra.finished and rb.finished and len(ra.generated) == 30 and len(rb.generated) == 30
    assert s.num_preemptions >= 1 and rb.preemptions >= 1 and ra.preemptions == 0       # the oldest keeps running
    # after a preemption b starts again from position 0 with everything it has produced so far
    restarts = [step for step in log for rid, start, n, _ in step if rid == b and start == 0]
    assert len(restarts) == rb.preemptions + 1
    assert m.num_free_pages(0) == 5 and m.num_free_slots() == 4


def test_a_prompt_portion_shrinks_to_the_free_pages_and_never_preempts():
    m = manager(num_pages=4, max_requests=4)
    s = Scheduler(m, SchedulerConfig(max_num_seqs=4, max_tokens_per_step=256, prefill_chunk=256), 512)
    a = s.add_request([1] * 40, 2)         # 3 pages
    b = s.add_request([2] * 20, 2)         # 2 pages: only one is free at first
    items = s.schedule()
    assert [(it.request.id, it.count) for it in items] == [(a, 40), (b, 16)]
    assert s.num_preemptions == 0


def test_finishing_rules():
    m = manager(num_pages=16)
    s = Scheduler(m, SchedulerConfig(), 512, eos_token_ids=[9])
    a = s.add_request([1, 2, 3], 5)
    tokens = iter([4, 5, 9, 6])
    run(s, token=lambda req: next(tokens))
    r = s.requests[a]
    assert r.generated == [4, 5] and r.finish_reason == "eos"          # the end token is dropped (qwen2.cpp:1060-1062)
    b = s.add_request([1], 2)
    run(s)
    assert s.requests[b].generated == [1, 1] and s.requests[b].finish_reason == "length"   # exactly max_new_tokens
    c = s.add_request([1, 2], 50)
    s.schedule()
    s.abort(c)
    assert s.requests[c].finish_reason == "aborted" and m.num_free_pages(0) == 16
    s.forget(c)
    assert c not in s.requests


def test_sampling_params_greedy_rule():
    assert SamplingParams().greedy                                     # top_k = 1 by default (qwen2.py:305-311)
    assert SamplingParams(temperature=0.0, top_k=50).greedy            # temperature <= 0 (qwen2.cpp:893-895)
    assert not SamplingParams(temperature=0.8, top_k=0).greedy


# --------------------------------------------------------------------------
# the packer of a step's metadata (host runtime) against the plain one
# --------------------------------------------------------------------------

@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("window", [None, 20])
def test_packed_steps_equal_the_plain_packer(seed, window):
    """Random batches (portions, single tokens, requests with pages behind a window given back) packed by the host
    runtime and by the plain numpy packer of the tests: the same buffer and the same layout, plainly, padded to a decode
    bucket, padded to a captured shape, and as single tokens of one request."""
    import numpy as np

    import plain_pack
    from litinfer_b200.engine import StepItem
    from litinfer_b200.engine.batch import pack_step, split_into_tokens

    rnd = random.Random(seed)
    m = manager(num_pages=200, max_requests=24, window=window, two_groups=True)
    vocab = 500
    for _ in range(12):
        items = []
        for i in range(rnd.randint(1, 12)):
            rc = m.admit(i)
            had = rnd.choice([0, 0, 7, 16, 40, 65])
            if had:
                m.extend(rc, had)
                m.commit(rc, had)
            q = rnd.choice([1, 1, 1, 2, 9, 33])
            m.extend(rc, had + q)
            items.append(StepItem(rc, [rnd.randrange(vocab) for _ in range(q)], tuple(sorted(rnd.sample(range(q), rnd.randint(0, min(q, 3)))))))
        T, S, R = sum(len(it.tokens) for it in items), len(items), sum(len(it.want) for it in items)
        cases = [dict(), dict(max_blocks=16)]
        if all(len(it.tokens) == 1 for it in items):
            cases.append(dict(pad_seqs=16, max_blocks=16))
        cases.append(dict(pad_seqs=S + 2, max_blocks=16, pad_tokens=T + 21, pad_rows=max(R, S + 2)))
        cases.append(dict(pad_seqs=S, max_blocks=16, pad_tokens=T, pad_rows=R + 1))
        for kw in cases:
            kw = dict(kw, work_budget=rnd.choice([0, 3, 12, 40]))
            a, la = pack_step(items, m, vocab, **kw)
            b, lb = plain_pack.pack_step(items, m, vocab, **kw)
            assert np.array_equal(a, b), f"buffers differ for {kw}"
            assert la == lb, f"layouts differ for {kw}"
        singles = split_into_tokens([StepItem(it.cache, it.tokens, ()) for it in items])
        a, la = pack_step(singles, m, vocab, pad_seqs=len(singles) + 3, max_blocks=16, tokens_of_one_request=True)
        b, lb = plain_pack.pack_step(singles, m, vocab, pad_seqs=len(singles) + 3, max_blocks=16, tokens_of_one_request=True)
        assert np.array_equal(a, b) and la == lb
        for it in items:
            m.release(it.cache)
        m.check()


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 20])
def test_resident_tables_get_what_they_lack(seed, window):
    """Steps packed for resident block tables, over the life of random requests (admitted, extended in portions and
    single tokens, committed so that pages behind a window go back, released and their ids and slots used again): the
    changes a step carries are those of the plain restatement, and a copy of the tables kept up to date with them
    holds, for every sequence of the step, the table that the step would otherwise have carried."""
    import numpy as np

    import plain_pack
    from litinfer_b200.engine import StepItem
    from litinfer_b200.engine.batch import pack_step

    rnd = random.Random(100 + seed)
    m = manager(num_pages=120, max_requests=6, window=window, two_groups=True)
    plain = plain_pack.PlainResidentTables(m)
    G, vocab = len(m.groups), 300
    copy = [np.full((m.max_requests + 1, 64), m.trash_page, dtype=np.int32) for _ in range(G)]
    live, next_id = {}, 0
    for step in range(60):
        while len(live) < 6 and rnd.random() < 0.5:
            rid = next_id % 9                                      # ids come back
            next_id += 1
            if rid in live:
                continue
            live[rid] = m.admit(rid)
            if rnd.random() < 0.3:                                 # extended before its first step
                n = rnd.choice([5, 16, 33])
                m.extend(live[rid], n)
                m.commit(live[rid], n)
        if not live:
            continue
        chosen = rnd.sample(sorted(live), rnd.randint(1, len(live)))
        items = []
        for rid in chosen:
            rc = live[rid]
            q = rnd.choice([1, 1, 1, 2, 17, 40])
            if rc.length + q > 64 * 16 - 1:
                continue
            m.extend(rc, rc.length + q)
            items.append(StepItem(rc, [rnd.randrange(vocab) for _ in range(q)], ()))
        if not items:
            continue
        want = plain.updates(items)
        full, lf = plain_pack.pack_step(items, m, vocab, max_blocks=64)
        buf, lay = pack_step(items, m, vocab, max_blocks=64, resident=True)
        S = lay["S"]
        for name in ("token_ids", "positions", "q_start", "ctx_lens", "state_slots", "slot_mapping0"):
            o, n = lay["fields"][name]
            o2, _ = lf["fields"][name]
            assert np.array_equal(buf[o:o + n], full[o2:o2 + n]), name
        for g in range(G):
            o, n = lay["fields"][f"table_updates{g}"]
            count = int(buf[o])
            got = [tuple(int(x) for x in buf[o + 1 + 3 * i:o + 4 + 3 * i]) for i in range(count)]
            assert got == want[g], f"step {step} group {g}"
            for slot, block, page in got:
                copy[g][slot, block] = page
            o2, _ = lf["fields"][f"block_table{g}"]
            tables = full[o2:o2 + S * 64].reshape(S, 64)
            for s_, it in enumerate(items):
                nb = -(-(it.cache.length + len(it.tokens)) // 16)
                assert np.array_equal(copy[g][it.cache.slot, :nb], tables[s_, :nb]), f"step {step} group {g} sequence {s_}"
        # nothing is sent twice
        again, la = pack_step(items, m, vocab, max_blocks=64, resident=True)
        assert all(int(again[la["fields"][f"table_updates{g}"][0]]) == 0 for g in range(G))
        for it in items:
            m.commit(it.cache, it.cache.length + len(it.tokens))
        for rid in list(live):
            if rnd.random() < 0.15:
                m.release(live.pop(rid))
                plain.forget(rid)
        m.check()


def test_the_packer_refuses_what_the_plain_one_refuses():
    from litinfer_b200.engine import StepItem
    from litinfer_b200.engine.batch import pack_step

    m = manager(num_pages=8, window=20)
    a, b = m.admit(0), m.admit(1)
    m.extend(a, 40)
    m.commit(a, 37)
    m.extend(b, 5)
    with pytest.raises(ValueError, match="at least one item"):
        pack_step([], m, 100)
    with pytest.raises(ValueError, match="without tokens"):
        pack_step([StepItem(a, [], ())], m, 100)
    with pytest.raises(ValueError, match="twice"):
        pack_step([StepItem(a, [1], ()), StepItem(a, [2], ())], m, 100)
    with pytest.raises(IndexError, match="token id"):
        pack_step([StepItem(a, [100], ())], m, 100)
    with pytest.raises(IndexError, match="wanted place"):
        pack_step([StepItem(a, [1, 2], (2,))], m, 100)
    with pytest.raises(RuntimeError, match="not allocated"):
        pack_step([StepItem(a, [1] * 12, ())], m, 100)                # 37 + 12 tokens need a fourth page
    with pytest.raises(ValueError, match="cannot be padded"):
        pack_step([StepItem(b, [1, 2], ())], m, 100, pad_seqs=1, pad_tokens=8, pad_rows=1)
    with pytest.raises(ValueError, match="wanted rows"):
        pack_step([StepItem(b, [1, 2], (0, 1))], m, 100, pad_seqs=2, pad_tokens=8, pad_rows=1)
    m.release(a)
    with pytest.raises(PoolError, match="not live"):
        pack_step([StepItem(a, [1], ())], m, 100)


@pytest.mark.parametrize("seed", range(10))
@pytest.mark.parametrize("window", [None, 24])
def test_the_scheduler_decides_like_the_plain_one(seed, window):
    """Random streams of requests (arrivals while others run, small pools so that requests are preempted, budgets that
    cut prompts into portions, end-of-sequence tokens, aborts) through the scheduler of the host runtime and through
    the plain Python one of the tests, each over a cache manager of its own: the same items every step, the same
    outputs, reasons and preemptions."""
    import plain_scheduler

    rnd = random.Random(1000 + seed)
    pages, slots = rnd.choice([6, 8, 14]), rnd.choice([2, 4, 6])
    cfg = dict(max_num_seqs=rnd.choice([2, 3, 8]), max_tokens_per_step=rnd.choice([8, 24, 64]), prefill_chunk=rnd.choice([5, 16, 64]))
    pair = []
    for mod in (None, plain_scheduler):
        m = manager(num_pages=pages, max_requests=slots, window=window, two_groups=True)
        if mod is None:
            s = Scheduler(m, SchedulerConfig(**cfg), 200, eos_token_ids=[7])
        else:
            s = mod.Scheduler(m, mod.SchedulerConfig(**cfg), 200, eos_token_ids=[7])
        pair.append((m, s))
    ids = []
    for step in range(300):
        if rnd.random() < 0.25 and len(ids) < 25:
            n, new = rnd.randint(1, 40), rnd.choice([1, 3, 20, 45, 45])
            got = []
            for m, s in pair:
                try:
                    got.append(s.add_request(list(range(n)), new))
                except ValueError as e:                         # refused by both, for the same reason
                    got.append(str(e))
            assert got[0] == got[1]
            if isinstance(got[0], int):
                ids.append(got[0])
        if ids and rnd.random() < 0.03:
            victim = rnd.choice(ids)
            for m, s in pair:
                s.abort(victim)
        draws = {}
        logs = []
        for m, s in pair:
            items = s.schedule()
            logs.append([(it.request.id, it.start, it.count, it.wants_logits) for it in items])
            for it in items:
                m.commit(it.request.cache, it.start + it.count)
            toks = []
            for it in items:
                if it.wants_logits and it.request.id not in draws:
                    draws[it.request.id] = rnd.choice([1, 2, 3, 7]) if rnd.random() < 0.3 else 1
                toks.append(draws.get(it.request.id) if it.wants_logits else None)
            done = s.update(items, toks)
            logs.append(sorted(r.id for r in done))
            m.check()
        assert logs[0] == logs[2] and logs[1] == logs[3], f"step {step}: {logs}"
        a, b = pair[0][1], pair[1][1]
        assert [r.id for r in a.running] == [r.id for r in b.running] and [r.id for r in a.waiting] == [r.id for r in b.waiting]
        assert a.num_preemptions == b.num_preemptions
        assert all(pair[0][0].num_free_pages(g) == pair[1][0].num_free_pages(g) for g in range(len(pair[0][0].groups)))
    a, b = pair[0][1], pair[1][1]
    for rid in ids:
        ra, rb = a.requests[rid], b.requests[rid]
        assert (ra.generated, ra.finish_reason, ra.status, ra.preemptions) == (rb.generated, rb.finish_reason, rb.status, rb.preemptions)
