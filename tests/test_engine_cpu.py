"""The host side of the engine (cache manager, block tables, slot mapping, step
metadata, schedule, page release behind a window) checked on the CPU: the
kernels are replaced by their plain references, everything else is the
product code, and the logits are compared with the plain model."""

from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import plain_qwen2 as P
from conftest import TINY
from helpers import check_logits, plain_logits, random_tokens, stack
from test_replay_gpu import build_trace


def replay_in_process(model_dir, dtype, trace, max_tokens, vocab, tmp_path, spec=None):
    from litinfer_b200.engine.replay import replay
    from litinfer_b200.models import DecoderModel

    model = DecoderModel.from_dir(model_dir, dtype, "cpu", spec=spec)
    replay(model, trace.lines().splitlines(), tmp_path, max_tokens, use_graphs=False)
    res = {}
    for i, rows in enumerate(trace.where):
        if not rows:
            continue
        lg = torch.from_numpy(np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(len(rows), vocab).copy())
        for (rid, pos), row in zip(rows, lg):
            res.setdefault(rid, {})[pos] = row
    return res


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_on_cpu_references(name, dtype, model_dirs, tmp_path, cpu_kernels):
    cfg = TINY[name]
    vocab = cfg["vocab_size"]
    tr, seqs, need = build_trace(vocab, cfg["max_position_embeddings"])
    got = replay_in_process(model_dirs[name], dtype, tr, need, vocab, tmp_path)
    for rid, toks in seqs.items():
        check_logits(stack(got[rid]), plain_logits(model_dirs[name], toks, dtype), dtype, f"{name} {dtype} {rid}")


def test_pool_too_small_is_an_error(model_dirs, tmp_path, cpu_kernels):
    from litinfer_b200.cache import OutOfPages
    from helpers import Trace

    tr = Trace()
    tr.step([("a", random_tokens(70, 256, 1), True)])
    with pytest.raises(OutOfPages):
        replay_in_process(model_dirs["A"], "float32", tr, 64, 256, tmp_path)


def test_schedule_with_repeated_block_and_shared_cache(model_dirs, tmp_path, cpu_kernels):
    """The order of layers is data: block 0 twice, and an entry that reads the
    keys and values of an earlier entry instead of its own."""
    from litinfer_b200.config import ScheduleEntry, load_config
    from helpers import Trace

    spec = load_config(model_dirs["A"]).to_model_spec()
    spec = spec.with_schedule([ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_from=1)])
    plain_schedule = [(0, None), (1, None), (0, None), (1, 1)]
    toks = random_tokens(45, 256, 3)
    tr = Trace()
    tr.step([("s", toks[:17], True)])
    tr.step([("s", toks[17:19], True)])
    for t in toks[19:30]:
        tr.step([("s", [t], True)])
    tr.step([("s", toks[30:], True)])
    got = replay_in_process(model_dirs["A"], "float32", tr, 64, 256, tmp_path, spec=spec)
    ref = plain_logits(model_dirs["A"], toks, "float32", plain_schedule)
    check_logits(stack(got["s"]), ref, "float32", "custom schedule")


def test_engine_greedy_matches_plain(model_dirs, cpu_kernels):
    from litinfer_b200.engine import Engine, EngineConfig
    from litinfer_b200.models import DecoderModel

    for name, lens, n_new in (("A", [5, 11, 17], 8), ("B", [1, 9, 33, 40], 12)):
        cfg, w = P.read_model_folder(model_dirs[name])
        model = DecoderModel.from_dir(model_dirs[name], "float32", "cpu")
        eng = Engine(model, EngineConfig(num_pages=10, max_num_seqs=4, max_tokens_per_step=24, prefill_chunk=16, use_graphs=False))
        prompts = [random_tokens(n, cfg["vocab_size"], 100 + n) for n in lens]
        ids = [eng.add_request(p, n_new) for p in prompts]
        eng.run_to_completion()
        eng.manager.check()
        assert eng.manager.num_free_pages(0) == 10 and eng.manager.num_free_slots() == 4
        for rid, p in zip(ids, prompts):
            ref, margin = P.plain_greedy(cfg, w, p, n_new)
            assert margin > 1e-5, "the plain model's own choice is a near-tie; pick another seed"
            assert eng.get_output(rid) == ref, f"config {name}, prompt of {len(p)}"


def test_engine_run_ahead_gives_the_same_tokens(model_dirs, cpu_kernels):
    """Steps launched before the tokens of the step before them are read: the same outputs as step by step, with requests
    of different lengths (some end by length while others go on), with an end-of-sequence token that cuts requests short
    (the token computed ahead for them is dropped), with too few pages for everybody, and with sampling."""
    from litinfer_b200.engine import Engine, EngineConfig
    from litinfer_b200.models import DecoderModel
    from litinfer_b200.sampling.sampler import SamplingParams

    cfg, w = P.read_model_folder(model_dirs["A"])
    model = DecoderModel.from_dir(model_dirs["A"], "float32", "cpu")
    prompts = [random_tokens(n, cfg["vocab_size"], 300 + n) for n in (5, 11, 17, 3)]
    new = [9, 14, 6, 20]

    def run(run_ahead, eos, pages, params):
        eng = Engine(model, EngineConfig(num_pages=pages, max_num_seqs=4, max_tokens_per_step=24, prefill_chunk=16, use_graphs=False,
                                         run_ahead=run_ahead))
        eng.scheduler.eos = set(eos)
        ids = [eng.add_request(p, n, params) for p, n in zip(prompts, new)]
        steps = 0
        while eng.has_unfinished():
            eng.step()
            steps += 1
            assert steps < 500
        assert eng.drain() == []
        eng.manager.check()
        assert eng.manager.num_free_pages(0) == pages and eng.manager.num_free_slots() == 4
        return [(eng.get_output(i), eng.finish_reason(i)) for i in ids], eng.scheduler.num_preemptions

    plain, _ = run(False, (), 12, None)
    assert [len(o) for o, _ in plain] == new
    # an end-of-sequence token: one that some request produces in the middle of its output
    eos = plain[1][0][5]
    preempted = 0
    for params in (None, SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=7)):
        for e in ((), (eos,)):
            for pages in (12, 5, 4, 3):
                a, pre_a = run(False, e, pages, params)
                b, pre_b = run(True, e, pages, params)
                assert a == b, f"run_ahead changes the outputs (eos {e}, pages {pages}, params {params})"
                if e and params is None:
                    assert any(r == "eos" for _, r in a)
                preempted += min(pre_a, pre_b)
    assert preempted > 0, "the small pools were meant to force preemptions in both modes"


def test_abort_while_a_step_is_in_flight(model_dirs, cpu_kernels):
    """With run_ahead a step is unread between calls.  Ending a request then, through the engine or straight through the
    scheduler, must not cost the other requests of that step their tokens."""
    from litinfer_b200.engine import Engine, EngineConfig
    from litinfer_b200.models import DecoderModel

    cfg, _ = P.read_model_folder(model_dirs["A"])
    model = DecoderModel.from_dir(model_dirs["A"], "float32", "cpu")
    prompts = [random_tokens(n, cfg["vocab_size"], 400 + n) for n in (5, 9, 12)]

    def run(abort_how):
        eng = Engine(model, EngineConfig(num_pages=16, max_num_seqs=4, max_tokens_per_step=32, use_graphs=False, run_ahead=True))
        ids = [eng.add_request(p, 10) for p in prompts]
        calls = 0
        while eng.has_unfinished():
            eng.step()
            calls += 1
            if calls == 5 and abort_how:
                assert eng._ahead is not None, "the test wants a step in flight here"
                if abort_how == "engine":
                    eng.abort(ids[1])
                else:
                    eng.scheduler.abort(ids[1])
            assert calls < 200
        eng.drain()
        eng.manager.check()
        assert eng.manager.num_free_pages(0) == 16 and eng.manager.num_free_slots() == 4
        return [eng.get_output(i) for i in ids], [eng.finish_reason(i) for i in ids]

    whole, _ = run(None)
    for how in ("engine", "scheduler"):
        outs, reasons = run(how)
        assert reasons[1] == "aborted" and reasons[0] == reasons[2] == "length"
        assert outs[0] == whole[0] and outs[2] == whole[2], how
        assert outs[1] == whole[1][:len(outs[1])] and len(outs[1]) < 10


def test_toy_mixer_with_state_on_cpu_references(model_dirs, cpu_kernels):
    from test_engine_gpu import run_toy_mixer

    run_toy_mixer(model_dirs, "cpu")


def test_toy_routed_feed_forward_and_positions_on_cpu_references(model_dirs, cpu_kernels):
    from test_engine_gpu import run_toy_feed_forward_and_positions

    run_toy_feed_forward_and_positions(model_dirs, "cpu", "float32")



@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_as_single_tokens_are_the_same_step(name, model_dirs, cpu_kernels):
    """A step with portions of prompts, packed with every token as an item of its own (as the captured decode step
    takes it), asks for the same work: same logits at the wanted places, in the order of the items and their wants."""
    from litinfer_b200.cache import CacheManager
    from litinfer_b200.engine import ModelRunner, StepItem
    from litinfer_b200.engine.batch import context_from, pack_step, split_into_tokens
    from litinfer_b200.models import DecoderModel

    cfg = TINY[name]
    vocab = cfg["vocab_size"]
    model = DecoderModel.from_dir(model_dirs[name], "float32", "cpu")
    spec = model.spec
    manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], 24, 16, 4, model.dtype, model.device)
    runner = ModelRunner(model, manager)
    a, b, c = random_tokens(60, vocab, 1), random_tokens(30, vocab, 2), random_tokens(9, vocab, 3)
    ra, rb, rc = manager.admit(1), manager.admit(2), manager.admit(3)
    manager.extend(ra, 41)
    manager.extend(rb, 29)
    runner.step([StepItem(ra, a[:41], ()), StepItem(rb, b[:29], ())])
    # a: a portion over a page's edge, far enough for the window of configuration B; b: one token; c: a whole short prompt
    manager.extend(ra, 60)
    manager.extend(rb, 30)
    manager.extend(rc, 9)
    items = [StepItem(ra, a[41:], (18, 0, 7)), StepItem(rb, b[29:], (0,)), StepItem(rc, c, (8,))]
    buf, layout = pack_step(items, manager, vocab)
    whole = model.forward(context_from(torch.from_numpy(buf), layout, manager.page_size), manager.entries)
    singles = split_into_tokens(items)
    assert [len(it.tokens) for it in singles] == [1] * 29
    buf, layout = pack_step(singles, manager, vocab, pad_seqs=32, tokens_of_one_request=True)
    assert layout["S"] == 32 and layout["max_q_len"] == 1
    f = layout["fields"]
    old = buf[f["old_lens"][0]:f["old_lens"][0] + 29].tolist()
    assert old == [41] * 19 + [29] + [0] * 9                      # the keys that were there before the step
    ctx_lens = buf[f["ctx_lens"][0]:f["ctx_lens"][0] + 29].tolist()
    assert ctx_lens == list(range(42, 61)) + [30] + list(range(1, 10))
    split = model.forward(context_from(torch.from_numpy(buf), layout, manager.page_size), manager.entries)
    rows = [18, 0, 7, 19, 20 + 8]
    assert torch.allclose(split[rows], whole, atol=1e-6, rtol=0)
    with pytest.raises(ValueError):
        pack_step(singles, manager, vocab)                        # one request twice, unless said so
    with pytest.raises(IndexError):
        split_into_tokens([StepItem(rc, c, (9,))])


@pytest.mark.parametrize("name", ["A", "B"])
def test_a_step_padded_to_a_fixed_shape_is_the_same_step(name, model_dirs, cpu_kernels):
    """A step with portions of prompts, padded to a fixed count of tokens, sequences and logit rows (as a captured step
    takes it): the padding writes to the sink page only, and the real rows come first and are unchanged."""
    from litinfer_b200.cache import CacheManager
    from litinfer_b200.engine import ModelRunner, StepItem
    from litinfer_b200.engine.batch import context_from, pack_step
    from litinfer_b200.models import DecoderModel

    cfg = TINY[name]
    vocab = cfg["vocab_size"]
    model = DecoderModel.from_dir(model_dirs[name], "float32", "cpu")
    spec = model.spec
    manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], 24, 16, 4, model.dtype, model.device)
    runner = ModelRunner(model, manager)
    a, b = random_tokens(70, vocab, 1), random_tokens(30, vocab, 2)
    ra, rb = manager.admit(1), manager.admit(2)
    manager.extend(ra, 21)
    manager.extend(rb, 29)
    runner.step([StepItem(ra, a[:21], ()), StepItem(rb, b[:29], ())])
    manager.extend(ra, 70)
    manager.extend(rb, 30)
    items = [StepItem(ra, a[21:], (48, 3)), StepItem(rb, b[29:], (0,))]
    buf, layout = pack_step(items, manager, vocab)
    plain = model.forward(context_from(torch.from_numpy(buf), layout, manager.page_size), manager.entries)
    buf, layout = pack_step(items, manager, vocab, pad_seqs=4, max_blocks=8, pad_tokens=64, pad_rows=4)
    assert (layout["T"], layout["S"], layout["R"], layout["R_real"]) == (64, 4, 4, 3)
    assert layout["singles"] == 1                                 # b's one token beside a's portion
    f = layout["fields"]
    q_start = buf[f["q_start"][0]:f["q_start"][0] + 5].tolist()
    assert q_start == [0, 49, 50, 50, 64]                         # an empty padding sequence, and one with the padding tokens
    sm = buf[f["slot_mapping0"][0]:f["slot_mapping0"][0] + 64]
    trash = manager.trash_page
    assert (sm[50:] // 16 == trash).all() and (sm[:50] // 16 != trash).all()
    padded = model.forward(context_from(torch.from_numpy(buf), layout, manager.page_size), manager.entries)
    assert padded.shape[0] == 4
    assert torch.equal(padded[:3], plain)
    with pytest.raises(ValueError):
        pack_step(items, manager, vocab, pad_seqs=2, pad_tokens=64, pad_rows=4)     # no sequence for the padding tokens
    with pytest.raises(ValueError):
        pack_step(items, manager, vocab, pad_seqs=4, pad_tokens=64, pad_rows=2)     # three rows wanted


@pytest.mark.parametrize("seed", range(6))
def test_padded_steps_keep_their_invariants_under_random_batches(seed, model_dirs, cpu_kernels):
    """Random batches of portions and single tokens, padded to the shape the runner would capture them under: the real
    tokens, sequences and rows come first and unchanged, the padding sits on the sink page, and the shape only grows."""
    import random

    import numpy as np

    from litinfer_b200.cache import CacheManager
    from litinfer_b200.engine import ModelRunner, StepItem
    from litinfer_b200.engine.batch import pack_step
    from litinfer_b200.models import DecoderModel

    rnd = random.Random(seed)
    cfg = TINY["C"]
    vocab = cfg["vocab_size"]
    model = DecoderModel.from_dir(model_dirs["C"], "float32", "cpu")
    manager = CacheManager(model.cache_requirements(), [e.cache_from for e in model.spec.schedule], 400, 16, 40, model.dtype, model.device)
    runner = ModelRunner(model, manager)
    runner.step_graph_after = 0
    for _ in range(8):
        n = rnd.randint(1, 20)
        items = []
        for i in range(n):
            rc = manager.admit(i)
            had = rnd.choice([0, 0, 5, 16, 33])
            if had:
                manager.extend(rc, had)
                manager.commit(rc, had)
            q = rnd.choice([1, 1, 1, 2, 7, 64, 100])
            manager.extend(rc, had + q)
            want = tuple(sorted(rnd.sample(range(q), rnd.randint(0, min(q, 2)))))
            items.append(StepItem(rc, random_tokens(q, vocab, seed * 100 + i), want))
        T, S, R = sum(len(it.tokens) for it in items), len(items), sum(len(it.want) for it in items)
        shape = runner._step_shape(items)
        if all(len(it.tokens) == 1 for it in items):
            shape = None                                            # a step of single tokens is the decode graph's
        if shape is not None:
            Tp, Sp, Rp, singles = shape
            assert Tp >= T and Sp >= S and Rp >= R and Tp - T < max(64, T // 4) and (Tp == T or Sp > S)
            assert singles == any(len(it.tokens) == 1 for it in items)
            plain, _ = pack_step(items, manager, vocab)
            buf, lay = pack_step(items, manager, vocab, pad_seqs=Sp, max_blocks=64, pad_tokens=Tp, pad_rows=Rp)
            f = lay["fields"]
            get = lambda name, n: buf[f[name][0]:f[name][0] + n]
            assert (lay["T"], lay["S"], lay["R"], lay["R_real"]) == (Tp, Sp, Rp, R)
            q_start = get("q_start", Sp + 1)
            assert q_start[S] == T and q_start[Sp] == Tp and (np.diff(q_start) >= 0).all()
            assert (np.diff(q_start)[S:Sp - 1] == 0).all() if Sp - S > 1 else True
            assert (get("slot_mapping0", Tp)[T:] // 16 == manager.trash_page).all()
            assert (get("block_table0", Sp * 64).reshape(Sp, 64)[S:] == manager.trash_page).all()
            assert (get("logit_rows", Rp)[R:] == Tp - 1).all() and (get("logit_rows", Rp)[:R] < T).all()
            assert (get("ctx_lens", Sp)[S:] == np.diff(q_start)[S:]).all()
            assert lay["singles"] == sum(1 for it in items if len(it.tokens) == 1)
        for it in items:
            manager.release(it.cache)
        manager.check()


def test_which_steps_are_captured_and_under_which_shape(model_dirs, cpu_kernels):
    """The runner's rule for steps with portions of prompts: a shape is captured when it comes back, the shape rounds
    tokens, sequences and rows up, and what does not fit a captured shape is launched plainly."""
    from litinfer_b200.cache import CacheManager
    from litinfer_b200.engine import ModelRunner, StepItem
    from litinfer_b200.models import DecoderModel

    model = DecoderModel.from_dir(model_dirs["C"], "float32", "cpu")
    manager = CacheManager(model.cache_requirements(), [e.cache_from for e in model.spec.schedule], 8, 16, 4, model.dtype, model.device)
    runner = ModelRunner(model, manager)

    class Cache:
        def __init__(self, length):
            self.length = length

    def items(*portions):
        return [StepItem(Cache(had), [0] * n, want) for had, n, want in portions]

    step = items((0, 130, (129,)))
    assert runner._step_shape(step) is None                          # first sight: launched plainly
    assert runner._step_shape(step) == (192, 2, 2, False)            # it came back
    runner._step_graphs[(192, 2, 2, False)] = object()
    assert runner._step_shape(items((40, 150, (149,)))) == (192, 2, 2, False)      # another step of the same shape
    runner.step_graph_after = 0
    assert runner._step_shape(items((0, 512, (511,)))) == (512, 1, 1, False)       # nothing to pad: no padding sequence
    assert runner._step_shape(items((0, 500, (499,)), *[(700, 1, (0,))] * 12)) == (512, 16, 16, True)
    assert runner._step_shape(items((0, 544, (543,)))) == (640, 2, 2, False)       # steps of 128 beyond 512 tokens
    assert runner._step_shape(items((0, 80, tuple(range(80))))) == (128, 2, 128, False)    # every token's logits: rows padded to the tokens
    assert runner._step_shape(items((0, 2049, (0,)))) is None                       # too many tokens
    assert runner._step_shape(items((runner.max_context - 50, 100, (0,)))) is None  # beyond the captured attention's context
    runner.STEP_GRAPH_LOGITS = 1000
    assert runner._step_shape(items((0, 80, tuple(range(80))))) is None             # too many logits to keep per shape
    runner.STEP_GRAPH_LOGITS = ModelRunner.STEP_GRAPH_LOGITS
    runner._step_graphs.update({i: None for i in range(ModelRunner.STEP_GRAPH_LIMIT)})
    assert runner._step_shape(items((0, 300, (299,)))) is None                      # enough shapes are kept already
    runner._may_split = False
    assert runner._step_shape(step) is None                                         # a mixer with state of its own


@pytest.mark.parametrize("name", ["A", "B"])
def test_captured_paths_of_the_runner_with_the_capture_emulated(name, model_dirs, tmp_path, cpu_kernels):
    """Everything the runner does around a captured graph, on the CPU: single-token steps padded to a bucket, small
    steps with portions as single tokens of one request, larger ones padded to a shape, the rows picked out of the
    captured layout.  The capture itself is emulated (replaying runs the forward pass on the captured metadata
    buffer again), so that the packed, padded metadata and the bookkeeping are checked against the plain model."""
    from litinfer_b200.engine import step as step_module
    from litinfer_b200.engine.batch import context_from
    from litinfer_b200.engine.replay import Replayer
    from litinfer_b200.models import DecoderModel

    class Emulated(step_module.ModelRunner):
        def _capture(self, B, max_blocks, buf, layout, max_q_len=1, singles=0):
            meta = torch.zeros(buf.shape[0], dtype=torch.int32)
            self._upload(buf, meta)
            lay = dict(layout, max_ctx_len=self.max_context, max_q_len=max_q_len, singles=singles)
            ctx = context_from(meta, lay, self.manager.page_size, self.manager)
            runner = self

            class Graph:
                def replay(self):
                    ctx.scratch.clear()
                    ctx.sync_tables()
                    g.logits.copy_(runner.model.forward(ctx, runner.manager.entries))

            ctx.sync_tables()
            g = step_module._DecodeGraph(Graph(), meta, self.model.forward(ctx, self.manager.entries).clone(), lay)
            if B is not None:
                self._graphs[B] = g
            return g

    cfg = TINY[name]
    vocab = cfg["vocab_size"]
    tr, seqs, need = build_trace(vocab, cfg["max_position_embeddings"])
    model = DecoderModel.from_dir(model_dirs[name], "float32", "cpu")
    rp = Replayer(model, need, use_graphs=False)
    rp.runner = Emulated(model, rp.manager, max_context=rp.runner.max_context, step_graph_after=0)
    rp.runner.use_graphs = True
    got = {}
    for i, line in enumerate(tr.lines().splitlines()):
        logits = rp.step(json.loads(line)).clone()
        for (rid, pos), row in zip(tr.where[i], logits):
            got.setdefault(rid, {})[pos] = row
    for rid, toks in seqs.items():
        check_logits(stack(got[rid]), plain_logits(model_dirs[name], toks, "float32"), "float32", f"{name} {rid} through emulated captures")
    r = rp.runner
    assert r.graph_replays == len(tr.steps), "every step of the trace fits a captured path"
    assert len(r._graphs) >= 2 and len(r._step_graphs) >= 1
    rp.manager.check()


def test_toy_mixer_with_state_through_the_engine_on_cpu_references(model_dirs, cpu_kernels):
    from test_engine_gpu import run_toy_mixer_through_engine

    run_toy_mixer_through_engine(model_dirs, "cpu")


def test_toy_mixer_that_decodes_from_the_device_on_cpu_references(model_dirs, cpu_kernels):
    from test_engine_gpu import run_toy_mixer_in_captured_steps

    run_toy_mixer_in_captured_steps(model_dirs, "cpu")


@pytest.mark.parametrize("name", ["A", "B0"])
def test_toy_architecture_from_a_folder_on_cpu_references(name, model_dirs, cpu_kernels, tmp_path):
    from test_engine_gpu import run_toy_architecture

    run_toy_architecture(name, "float32", model_dirs, tmp_path, "cpu")


def test_toy_positions_and_block_arrangements_on_cpu_references(model_dirs, cpu_kernels):
    from test_engine_gpu import run_toy_positions_and_blocks

    run_toy_positions_and_blocks(model_dirs, "cpu", "float32")


def test_profile_switch_reports_per_phase_and_op(model_dirs, cpu_kernels, monkeypatch, capsys):
    """LLAISYS_PROFILE (LitInfer: src/utils/profiler.cpp): every kernel call is recorded under phase/op and a table is
    printed; on the CPU twin there is no device to time, so calls are counted through the same wrapper with timing off."""
    import io

    from litinfer_b200 import kernels

    prof = kernels.Profile()
    prof.enabled = True
    calls = []
    wrapped = prof.wrap("linear", lambda *a, **k: calls.append(a))
    prof.phase = "prefill"
    wrapped(1, 2)
    assert calls == [(1, 2)]                               # without a CUDA device the call goes straight through
    prof.total_ms = {"prefill/linear": 3.0, "decode/linear": 1.0}
    prof.calls = {"prefill/linear": 2, "decode/linear": 5}
    out = io.StringIO()
    prof.report(out)
    text = out.getvalue()
    assert "LLAISYS PROFILE" in text and "total op time: 4.000 ms" in text
    assert text.index("prefill/linear") < text.index("decode/linear")          # sorted by time
    assert "75.00" in text and "25.00" in text
