"""Trace replay through bin/trace_run, as a user runs it, against the plain model.

For each tiny configuration and both dtypes one trace holds: a request whole;
the same tokens with the last 32 decoded one by one; the same in portions of
changing size down to two tokens; the first tokens of a sequence; and a mixed
phase with up to four live requests, portions of some beside decoded tokens of
others, in a pool so small that pages are used again.
"""

from __future__ import annotations

import pytest
import torch

from conftest import MID, TINY
from helpers import Trace, check_logits, plain_logits, random_tokens, run_trace, stack

pytestmark = pytest.mark.gpu

PORTIONS = [7, 16, 2, 33, 5, 2, 17, 3, 2, 11, 2, 29]
MIX_PORTIONS = [5, 2, 16, 9, 3, 21, 2, 13]


def round64(n):
    return -(-n // 64) * 64


def build_trace(vocab: int, max_pos: int, main_len: int = 100, portions=PORTIONS, mix_portions=MIX_PORTIONS, mix_lens=None):
    tr = Trace()
    seqs = {}
    main_len = min(main_len, max_pos - 4)
    main = random_tokens(main_len, vocab, 11)
    # whole
    seqs["whole"] = main
    tr.step([("whole", main, True)], end=["whole"])
    # most of it in one step, the last 32 one by one
    seqs["tail"] = main
    tr.step([("tail", main[:-32], True)])
    for i in range(main_len - 32, main_len):
        tr.step([("tail", [main[i]], True)], end=["tail"] if i == main_len - 1 else [])
    # portions of changing size
    seqs["cut"] = main
    pos, i = 0, 0
    while pos < main_len:
        n = min(portions[i % len(portions)], main_len - pos)
        last = pos + n == main_len
        tr.step([("cut", main[pos:pos + n], True)], end=["cut"] if last else [])
        pos += n
        i += 1
    # the first tokens of a sequence
    for n in (1, 2, 3):
        seqs[f"first{n}"] = random_tokens(n, vocab, 20 + n)
        tr.step([(f"first{n}", seqs[f"first{n}"], True)], end=[f"first{n}"])
    need = round64(main_len)
    # mixed: up to four live requests
    lens = [main_len] + list(mix_lens or [60, min(90, max_pos - 2), 40, 75, 50, 33])
    queue = [(f"mix{j}", main if j == 0 else random_tokens(n, vocab, 40 + j)) for j, n in enumerate(lens)]
    for rid, toks in queue:
        seqs[rid] = toks
    live = []          # [rid, tokens, fed, slot]
    step_no, slot = 0, 0
    while queue or live:
        while queue and len(live) < 4:
            rid, toks = queue.pop(0)
            live.append([rid, toks, 0, slot])
            slot += 1
        entries, ending = [], []
        for item in live:
            rid, toks, fed, sl = item
            if (step_no + sl) % 5 == 4 and fed > 0:
                continue                                   # left out of this step, goes on later
            if fed < int(0.6 * len(toks)):
                n = min(mix_portions[(step_no + sl) % len(mix_portions)], len(toks) - fed)
            else:
                n = 1
            entries.append((rid, toks[fed:fed + n], True))
            item[2] = fed + n
            if item[2] == len(toks):
                ending.append(rid)
        need = max(need, sum(round64(it[2]) for it in live))
        if entries:
            tr.step(entries, end=ending)
        live = [it for it in live if it[0] not in ending]
        step_no += 1
    return tr, seqs, need


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "B0"])
def test_replay_all_cuts(name, dtype, model_dirs, tmp_path):
    cfg = TINY[name]
    vocab = cfg["vocab_size"]
    tr, seqs, need = build_trace(vocab, cfg["max_position_embeddings"])
    got = run_trace(model_dirs[name], dtype, tr, tmp_path / "out", need, vocab)
    refs = {}
    for rid, toks in seqs.items():
        key = tuple(toks)
        if key not in refs:
            refs[key] = plain_logits(model_dirs[name], toks, dtype)
        lg = stack(got[rid])
        assert lg.shape[0] == len(toks), f"{rid}: {lg.shape[0]} rows for {len(toks)} tokens"
        check_logits(lg, refs[key], dtype, f"config {name} {dtype} request {rid}")
    # the same tokens cut in different ways: beyond rounding nothing may differ, and in
    # float32 every reduction runs in an order that does not depend on the cut
    whole = stack(got["whole"])
    for rid in ("tail", "cut", "mix0"):
        other = stack(got[rid])
        if dtype == "float32":
            assert torch.equal(whole, other), f"float32: '{rid}' differs from 'whole' by {(whole - other).abs().max():.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MID))
def test_replay_other_sizes(name, dtype, tmp_path):
    """Sizes at which the engine takes other kernels than at the tiny ones: head sizes of 128 and 64 with portions of 64
    tokens and more (tensor-core attention and products, rotary encoding in the product's epilogue), a window of 100 keys,
    and widths that are no multiple of 8 (no fused activation, no 16-byte loads)."""
    from litinfer_b200.weights import write_model_folder

    cfg = MID[name]
    vocab = cfg["vocab_size"]
    write_model_folder(tmp_path / "model", dict(cfg), seed=4321 + len(name), store_dtype="float32")
    tr, seqs, need = build_trace(vocab, cfg["max_position_embeddings"], main_len=300, portions=[70, 2, 130, 5, 64, 17, 3, 9, 66],
                                 mix_portions=[65, 2, 100, 9, 33, 128, 2, 71], mix_lens=[150, 210, 90, 170, 120])
    got = run_trace(tmp_path / "model", dtype, tr, tmp_path / "out", need, vocab)
    refs = {}
    for rid, toks in seqs.items():
        key = tuple(toks)
        if key not in refs:
            refs[key] = plain_logits(tmp_path / "model", toks, dtype)
        lg = stack(got[rid])
        assert lg.shape[0] == len(toks), f"{rid}: {lg.shape[0]} rows for {len(toks)} tokens"
        check_logits(lg, refs[key], dtype, f"config {name} {dtype} request {rid}")
    if dtype == "float32":
        whole = stack(got["whole"])
        for rid in ("tail", "cut", "mix0"):
            assert torch.equal(whole, stack(got[rid])), f"float32: '{rid}' differs from 'whole'"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_long_decode(dtype, model_dirs, tmp_path):
    """A short prompt and then 560 tokens one by one: many pages, a long context."""
    cfg = TINY["C"]
    vocab = cfg["vocab_size"]
    toks = random_tokens(600, vocab, 77)
    tr = Trace()
    tr.step([("long", toks[:40], True)])
    for i in range(40, 600):
        tr.step([("long", [toks[i]], True)], end=["long"] if i == 599 else [])
    got = run_trace(model_dirs["C"], dtype, tr, tmp_path / "out", round64(600), vocab)
    check_logits(stack(got["long"]), plain_logits(model_dirs["C"], toks, dtype), dtype, f"long decode {dtype}")


def test_replay_without_graphs_matches(model_dirs, tmp_path):
    """Captured decode steps and plainly launched ones give the same logits."""
    cfg = TINY["A"]
    vocab = cfg["vocab_size"]
    toks = random_tokens(50, vocab, 5)
    tr = Trace()
    tr.step([("a", toks[:20], True)])
    for i in range(20, 50):
        tr.step([("a", [toks[i]], True)])
    a = run_trace(model_dirs["A"], "bfloat16", tr, tmp_path / "g", 64, vocab)
    b = run_trace(model_dirs["A"], "bfloat16", tr, tmp_path / "n", 64, vocab, extra=["--no-graphs"])
    assert torch.equal(stack(a["a"]), stack(b["a"]))


REAL_SIZES = dict(
    architectures=["Qwen2ForCausalLM"], torch_dtype="float32", num_hidden_layers=2, hidden_size=1536,
    num_attention_heads=12, num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=32000,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096,
    eos_token_id=None, use_sliding_window=False)


@pytest.fixture(scope="module")
def real_size_dir(tmp_path_factory):
    """Two layers with the layer sizes of the 1.5B shape (the vocabulary cut to 32,000 to keep the file small)."""
    from litinfer_b200.weights import write_model_folder

    d = tmp_path_factory.mktemp("real_sizes")
    write_model_folder(d, dict(REAL_SIZES), seed=99, store_dtype="float32")
    return d


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_real_layer_sizes(dtype, real_size_dir, tmp_path):
    """The kernels at the sizes they are built for: a 300-token prompt whole, then decoded on while a second
    request comes in portions beside it."""
    vocab = REAL_SIZES["vocab_size"]
    a = random_tokens(324, vocab, 201)
    b = random_tokens(160, vocab, 202)
    tr = Trace()
    tr.step([("a", a[:300], list(range(280, 300)))])
    tr.step([("a", [a[300]], True), ("b", b[:100], [99])])
    tr.step([("a", [a[301]], True), ("b", b[100:137], [0, 36])])
    tr.step([("a", [a[302]], True), ("b", b[137:139], True)])
    for i in range(303, 324):
        tr.step([("a", [a[i]], True), ("b", [b[139 + i - 303]], True)])
    got = run_trace(real_size_dir, dtype, tr, tmp_path / "out", 384 + 192, vocab)
    ref_a = plain_logits(real_size_dir, a, dtype)
    ref_b = plain_logits(real_size_dir, b[:139 + 21], dtype)
    for rid, ref in (("a", ref_a), ("b", ref_b)):
        rows = sorted(got[rid])
        check_logits(stack(got[rid]), ref[rows], dtype, f"real layer sizes {dtype} request {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_real_layer_sizes_four_live_requests(dtype, real_size_dir, tmp_path):
    """Every cut at the sizes the kernels are built for: whole, the last 32 tokens one by one, portions of changing size
    (some of 64 tokens and more, where the tensor-memory kernels run), and up to four live requests with portions of some
    beside decoded tokens of others, in a pool so small that pages are used again."""
    vocab = REAL_SIZES["vocab_size"]
    tr, seqs, need = build_trace(vocab, REAL_SIZES["max_position_embeddings"], main_len=200, portions=[70, 2, 33, 5, 64, 17, 3, 6],
                                 mix_portions=[65, 2, 40, 9, 33, 70, 2, 21], mix_lens=[150, 130, 100, 90, 70])
    got = run_trace(real_size_dir, dtype, tr, tmp_path / "out", need, vocab)
    refs = {}
    for rid, toks in seqs.items():
        key = tuple(toks)
        if key not in refs:
            refs[key] = plain_logits(real_size_dir, toks, dtype)
        lg = stack(got[rid])
        assert lg.shape[0] == len(toks), f"{rid}: {lg.shape[0]} rows for {len(toks)} tokens"
        check_logits(lg, refs[key], dtype, f"real layer sizes {dtype} request {rid}")
    if dtype == "float32":
        whole = stack(got["whole"])
        for rid in ("tail", "cut", "mix0"):
            assert torch.equal(whole, stack(got[rid])), f"float32: '{rid}' differs from 'whole'"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_at_the_benchmark_length(dtype, real_size_dir, tmp_path):
    """What the benchmark times, held to the plain model: a prompt of 2,048 tokens in one step, then 32 tokens one by
    one at contexts of 2,049 to 2,080 keys."""
    vocab = REAL_SIZES["vocab_size"]
    toks = random_tokens(2080, vocab, 301)
    tr = Trace()
    tr.step([("a", toks[:2048], list(range(2040, 2048)))])
    for i in range(2048, 2080):
        tr.step([("a", [toks[i]], True)], end=["a"] if i == 2079 else [])
    got = run_trace(real_size_dir, dtype, tr, tmp_path / "out", round64(2080), vocab)
    ref = plain_logits(real_size_dir, toks, dtype)
    rows = sorted(got["a"])
    assert rows == list(range(2040, 2080))
    check_logits(stack(got["a"]), ref[rows], dtype, f"2,048-token prompt and 32 decoded tokens, {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["head128", "head64_window", "B"])
def test_steps_with_portions_through_captured_shapes(name, dtype, model_dirs, tmp_path):
    """Steps with portions of prompts replayed from graphs of their padded shapes (captured at first sight here) give
    what the same steps give when launched plainly: padding tokens, padding sequences and padding rows change nothing,
    a captured shape serves other requests at other places of the cache, and two shapes share their memory."""
    from litinfer_b200.engine.replay import Replayer
    from litinfer_b200.models import DecoderModel
    from litinfer_b200.weights import write_model_folder

    if name in MID:
        cfg = MID[name]
        folder = tmp_path / "model"
        write_model_folder(folder, dict(cfg), seed=77, store_dtype="float32")
    else:
        cfg, folder = TINY[name], model_dirs[name]
    vocab = cfg["vocab_size"]
    lens = dict(a=230, b=152, c=90, d=203, e=80)
    lens = {k: min(v, cfg["max_position_embeddings"] - 2) for k, v in lens.items()}
    toks = {k: random_tokens(n, vocab, 500 + i) for i, (k, n) in enumerate(lens.items())}
    a, b, c, d, e = (toks[k] for k in "abcde")
    nd = len(d)
    records = [
        dict(entries=[dict(id="a", tokens=a[:130], want=[129])]),
        dict(entries=[dict(id="a", tokens=a[130:200], want=[0, 69]), dict(id="b", tokens=b[:70], want=[69])]),
        dict(entries=[dict(id="a", tokens=a[200:201], want=[0]), dict(id="b", tokens=b[70:150], want=[79]),
                      dict(id="c", tokens=c, want=[3, len(c) - 1])]),
        dict(entries=[dict(id="a", tokens=a[201:202], want=[0]), dict(id="b", tokens=b[150:151], want=[0]),
                      dict(id="d", tokens=d[:100], want=[99])], end=["c"]),
        # the same shape again, with other requests' tokens and a page that c gave back
        dict(entries=[dict(id="b", tokens=b[151:152], want=[0]), dict(id="a", tokens=a[202:203], want=[0]),
                      dict(id="d", tokens=d[100:nd], want=[nd - 101])], end=["b"]),
        # the logits of every token: rows padded to the tokens
        dict(entries=[dict(id="e", tokens=e, want=list(range(len(e))))], end=["e"]),
        dict(entries=[dict(id="a", tokens=a[203:], want=[len(a) - 204])], end=["a", "d"]),
    ]
    where = [[("a", 129)], [("a", 130), ("a", 199), ("b", 69)], [("a", 200), ("b", 149), ("c", 3), ("c", len(c) - 1)],
             [("a", 201), ("b", 150), ("d", 99)], [("b", 151), ("a", 202), ("d", nd - 1)], [("e", i) for i in range(len(e))],
             [("a", len(a) - 1)]]
    model = DecoderModel.from_dir(folder, dtype, torch.device("cuda:0"))
    need = sum(round64(n) for n in lens.values())
    plainly = Replayer(model, need, use_graphs=False)
    captured = Replayer(model, need, use_graphs=True, step_graph_after=0)
    refs = {k: plain_logits(folder, toks[k], dtype) for k in toks}
    for i, rec in enumerate(records):
        rec = dict(rec, step=i)
        x = plainly.step(rec).clone()
        y = captured.step(rec).clone()
        ref = torch.stack([refs[k][p] for k, p in where[i]])
        check_logits(x.cpu(), ref, dtype, f"{name} {dtype} step {i} launched plainly")
        check_logits(y.cpu(), ref, dtype, f"{name} {dtype} step {i} from a captured shape")
        if dtype == "float32":
            assert torch.equal(x, y), f"float32: step {i} differs between a captured shape and plain launches"
    r = captured.runner
    assert r.graph_replays == len(records)
    assert 4 <= len(r._step_graphs) <= 6 and plainly.runner.graph_replays == 0
    # a shape that has not come back yet is launched plainly by default
    later = Replayer(model, need, use_graphs=True)
    later.step(dict(records[0], step=0))
    assert later.runner.graph_replays == 0 and not later.runner._step_graphs


def test_captured_decode_step_of_many_requests(tmp_path):
    """Seventy requests decoding together (a captured step of 128 single tokens, where the products take the tensor-memory
    kernel and the rotation angles come from the step's table): the same logits as launched plainly, step after step."""
    from litinfer_b200.engine.replay import Replayer
    from litinfer_b200.models import DecoderModel
    from litinfer_b200.weights import write_model_folder

    cfg = MID["head128"]
    folder = tmp_path / "model"
    write_model_folder(folder, dict(cfg), seed=78, store_dtype="float32")
    vocab = cfg["vocab_size"]
    n = 70
    prompts = [random_tokens(5 + (i * 7) % 23, vocab, 900 + i) for i in range(n)]
    model = DecoderModel.from_dir(folder, "bfloat16", torch.device("cuda:0"))
    plainly = Replayer(model, 64 * n, max_live=n, use_graphs=False)
    captured = Replayer(model, 64 * n, max_live=n, use_graphs=True)
    refs = [plain_logits(folder, p, "bfloat16") for p in prompts]
    first = dict(step=0, entries=[dict(id=str(i), tokens=p[:-4], want=[]) for i, p in enumerate(prompts)])
    plainly.step(first)
    captured.step(first)
    for j in range(4, 0, -1):
        rec = dict(step=5 - j, entries=[dict(id=str(i), tokens=[p[-j]], want=[0]) for i, p in enumerate(prompts)])
        x = plainly.step(rec).clone()
        y = captured.step(rec).clone()
        ref = torch.stack([r[len(p) - j] for r, p in zip(refs, prompts)])
        check_logits(x.cpu(), ref, "bfloat16", f"70 requests, token -{j}, launched plainly")
        check_logits(y.cpu(), ref, "bfloat16", f"70 requests, token -{j}, from the captured step")
    assert captured.runner.graph_replays == 4


def test_captured_decode_steps_at_a_context_beyond_8192(tmp_path):
    """A model that allows 32,768 positions: the captured decode step is made for contexts up to that bound, and decode
    attention cuts every sequence's own context (9,000 keys here, beside a request of 40) into units of several rounds.
    The same logits as with every kernel launched plainly for the contexts as they are; for the short request, whose
    plain logits cost little, the plain model's."""
    from litinfer_b200.engine.replay import Replayer
    from litinfer_b200.models import DecoderModel
    from litinfer_b200.weights import write_model_folder

    cfg = dict(MID["head128"], max_position_embeddings=32768)
    folder = tmp_path / "model"
    write_model_folder(folder, cfg, seed=79, store_dtype="float32")
    vocab = cfg["vocab_size"]
    long_one, short_one = random_tokens(9006, vocab, 950), random_tokens(46, vocab, 951)
    model = DecoderModel.from_dir(folder, "bfloat16", torch.device("cuda:0"))
    need = round64(len(long_one)) + round64(len(short_one))
    plainly = Replayer(model, need, max_live=2, use_graphs=False)
    captured = Replayer(model, need, max_live=2, use_graphs=True)
    assert captured.runner.max_context > 9006
    step = 0
    for start in range(0, 9000, 1500):
        rec = dict(step=step, entries=[dict(id="long", tokens=long_one[start:start + 1500], want=[])])
        plainly.step(rec)
        captured.step(rec)
        step += 1
    rec = dict(step=step, entries=[dict(id="short", tokens=short_one[:40], want=[])])
    plainly.step(rec)
    captured.step(rec)
    before = captured.runner.graph_replays
    ref_short = plain_logits(folder, short_one, "bfloat16")
    for j in range(6):
        step += 1
        rec = dict(step=step, entries=[dict(id="long", tokens=[long_one[9000 + j]], want=[0]), dict(id="short", tokens=[short_one[40 + j]], want=[0])])
        x = plainly.step(rec).clone().cpu()
        y = captured.step(rec).clone().cpu()
        check_logits(y, x, "bfloat16", f"9,000 keys and 40 keys, decoded token {j}: captured against launched plainly")
        check_logits(y[1:2], ref_short[40 + j:41 + j], "bfloat16", f"the request of 40 keys beside one of 9,000, decoded token {j}")
    assert captured.runner.graph_replays == before + 6 and plainly.runner.graph_replays == 0


def test_a_request_across_the_kernel_choices_of_a_step(tmp_path):
    """In bfloat16 which kernels run depends on the step's size: up to 16 tokens the norms ride on the products, from 17 on
    they are kernels of their own; from 120 (sequence, key head) pairs on decode attention walks a whole context per CTA
    instead of splitting it; from 65 tokens on the products go to the tensor-memory kernels.  The same request decoded alone
    and among 15, 16, 70 and 127 others must give the plain model's logits every time, and the same logits up to rounding."""
    from litinfer_b200.engine.replay import Replayer
    from litinfer_b200.models import DecoderModel
    from litinfer_b200.weights import write_model_folder

    cfg = MID["head128"]
    folder = tmp_path / "model"
    write_model_folder(folder, dict(cfg), seed=79, store_dtype="float32")
    vocab = cfg["vocab_size"]
    model = DecoderModel.from_dir(folder, "bfloat16", torch.device("cuda:0"))
    main = random_tokens(203, vocab, 1000)
    ref = plain_logits(folder, main, "bfloat16")[200:203]
    seen = {}
    for others in (0, 15, 16, 70, 127):
        rp = Replayer(model, 256 + 64 * others, max_live=others + 1, use_graphs=False)
        rp.step(dict(step=0, entries=[dict(id="main", tokens=main[:200], want=[])]))
        side = [random_tokens(9 + (i * 5) % 30, vocab, 2000 + i) for i in range(others)]
        if others:
            rp.step(dict(step=1, entries=[dict(id=f"o{i}", tokens=p[:-3], want=[]) for i, p in enumerate(side)]))
        rows = []
        for j in range(3):
            entries = [dict(id="main", tokens=[main[200 + j]], want=[0])] + [dict(id=f"o{i}", tokens=[p[len(p) - 3 + j]], want=[]) for i, p in enumerate(side)]
            rows.append(rp.step(dict(step=2 + j, entries=entries))[0].clone().cpu())
        seen[others] = torch.stack(rows)
        check_logits(seen[others], ref, "bfloat16", f"the request among {others} others")
    scale = float(ref.abs().max())
    for others, lg in seen.items():
        assert (lg - seen[0]).abs().max() <= 0.02 * scale, f"among {others} others the logits move by {(lg - seen[0]).abs().max()} (scale {scale})"
