"""Benchmark of the engine on one B200: decode tokens per second.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of the step function.  The default run has the layer
sizes of the DeepSeek-R1-Distill-Qwen-1.5B shape (LitInfer's own benchmark
model) with random weights, a batch of 8 sequences that each hold a 2,048-token
prompt and decode on from there, 16-token pages, context capped at 4,096.
One JSON line is printed:

* ``value``: decoded tokens per second over exactly K steps, timed with CUDA
  events on the device (metadata of every step staged on the device beforehand);
* ``e2e``: the same through the Python entry point (``Qwen2.engine_*``): prompts
  in as host lists, real prefill, and per step the host-to-device copy of the
  step's metadata from pinned memory and the device-to-host read of the sampled
  tokens inside the timed region;
* ``prefill``: one 2,048-token prompt in one step;
* ``roofline``: bytes a decode step has to read (every weight once and the cache
  of the live requests) over its time, against the measured copy bandwidth;
* ``points``: decode tokens per second at batch 1 and 64.

Weights (3 GB) are larger than L2, so nothing stays cached between steps.

``--only decode|prefill|mixed|kernels-decode|kernels-prefill|kernels-mixed`` measures one part and prints a short line (for
profiling runs and the summaries under ``profiles/``); ``mixed`` is a step of ``--batch`` requests decoding at
``--context`` beside a portion of ``--prefill-tokens`` prompt tokens.

``--shape 1.5b|7b|14b`` chooses the layer sizes (default 1.5b, the headline; the other two are the larger workloads of
the benchmark description and run behind the flag only):

* ``--shape 7b --only serve``: continuous batching through ``Engine`` of 64 requests with prompts of 128 to 2,048
  tokens and 128 to 512 new tokens each under a real page budget: total tokens per second, mean and 95th-percentile
  step time, preemptions, steps by launch path.  LitInfer's own harness likewise times whole generations with the
  warm-up excluded (scripts/benchmark_cpu.py:202-253).
* ``--shape 14b --only chunked``: a 2,048-token prompt fed in portions of 512 tokens beside 32 requests decoding at a
  context of 4,096: milliseconds per step and the fractions of the roofline of its bytes and of its flops.

The default line also carries ``fp32_check``: the largest difference between the engine's float32 logits and the plain
implementation of the tests (tests/plain_qwen2.py) on two layers of the benchmark's sizes with the same random weights,
which the device draws with the library's kernel and the host restates bit for bit.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.is_file():
        try:
            d = json.loads(f.read_text())
            hbm = float(d.get("hbm_gbs") or d.get("hbm_gb_s") or 0)
            tf = float(d.get("bf16_tflops") or 0)
            if hbm > 0 and tf > 0:
                return {"hbm_gbs": hbm, "bf16_tflops": tf, "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS)


SHAPES = {
    # configs[2] of the benchmark description: the 1.5B shape (LitInfer's own benchmark model)
    "1.5b": dict(name="DeepSeek-R1-Distill-Qwen-1.5B shape (Qwen2)", num_hidden_layers=28, hidden_size=1536, num_attention_heads=12,
                 num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=151936, rope_theta=10000.0, rms_norm_eps=1e-6,
                 max_position_embeddings=4096),
    # configs[3]: the Qwen2-7B shape
    "7b": dict(name="Qwen2-7B shape", num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
               intermediate_size=18944, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=4096),
    # configs[4]: the Qwen2.5-14B shape
    "14b": dict(name="Qwen2.5-14B shape", num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                intermediate_size=13824, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-5, max_position_embeddings=8192),
}


def bench_config(shape: str = "1.5b"):
    """The configuration of a shape of the benchmark description (default: configs[2], the 1.5B shape)."""
    d = dict(SHAPES[shape])
    d.pop("name")
    return dict(architectures=["Qwen2ForCausalLM"], torch_dtype="bfloat16", tie_word_embeddings=False, eos_token_id=None,
                use_sliding_window=False, **d)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(model):
    """Bytes of every matrix a decode step reads once: all blocks and the lm_head
    (of the embedding only one row per token is read)."""
    total = 0
    for b in model.blocks:
        for p in b.all_params():
            n = 1
            for s in p.shape:
                n *= s
            total += n * (model.embedding.element_size() if p.role == "matrix" else 4)
    total += model.lm_head.numel() * model.lm_head.element_size()
    return total


def decode_flops_and_prefill_flops(cfg, T):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, dh = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_token_linear = 2 * (H * (nh + 2 * nkv) * dh + nh * dh * H + 3 * H * I) * L
    attn = 2 * 2 * nh * dh * (T * (T + 1) // 2) * L          # causal q k^T and p v
    return per_token_linear * T + attn + 2 * H * V


def make_decode_state(model, batch, context, steps_total, seed=0):
    """Cache manager and runner with ``batch`` requests that already hold ``context``
    tokens (cache filled with random values: decode timing does not need a real prefill)."""
    import torch

    from litinfer_b200.cache import CacheManager
    from litinfer_b200.engine import ModelRunner

    spec = model.spec
    per_seq = -(-(context + steps_total + 1) // 16)
    manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], per_seq * batch, 16, batch,
                           model.dtype, model.device)
    for g in manager.groups:
        g.kv.normal_(0.0, 0.5)
    runner = ModelRunner(model, manager, use_graphs=True, max_context=min(spec.max_position_embeddings, context + steps_total + 1))
    reqs = []
    for b in range(batch):
        rc = manager.admit(b)
        manager.extend(rc, context)
        manager.commit(rc, context)
        reqs.append(rc)
    return manager, runner, reqs


def time_decode(model, batch, context, steps, warmup, graphs=True):
    """Device time of exactly ``steps`` decode steps (tokens per second, ms per step,
    launches per step, mean context)."""
    import numpy as np
    import torch

    from litinfer_b200 import kernels
    from litinfer_b200.engine import StepItem
    from litinfer_b200.engine.batch import pack_step

    total = steps + warmup
    manager, runner, reqs = make_decode_state(model, batch, context, total)
    vocab = model.spec.vocab_size
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, vocab, (total + 1, batch), generator=g).tolist()
    if not graphs:
        # every kernel launched from the host, one by one: what a profiler can list
        runner.use_graphs = False
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = 0
        for k in range(total):
            if k == warmup:
                torch.cuda.synchronize()
                before = kernels.launches
                start.record()
            for rc in reqs:
                manager.extend(rc, rc.length + 1)
            runner.step([StepItem(rc, [toks[k][b]], (0,)) for b, rc in enumerate(reqs)])
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop)
        return dict(tok_s=batch * steps / (ms / 1e3), ms_per_step=ms / steps, launches_per_step=(kernels.launches - before) // steps,
                    mean_ctx=context + warmup + (steps + 1) / 2)
    # first step through the ordinary path: captures the graph for this batch size
    for rc in reqs:
        manager.extend(rc, rc.length + 1)
    before = kernels.launches
    runner.step([StepItem(rc, [toks[0][b]], (0,)) for b, rc in enumerate(reqs)])
    graph = runner._graphs[runner._bucket(batch)]
    # launches of one forward = those of the capture pass (two warm-ups and the capture itself ran the same sequence)
    launches_per_step = (kernels.launches - before) // 3
    out = torch.empty(batch, dtype=torch.int32, device=model.device)
    max_blocks = graph.layout["max_blocks"]
    staged = []
    for k in range(total):
        for rc in reqs:
            manager.extend(rc, rc.length + 1)
        items = [StepItem(rc, [toks[k + 1][b]], (0,)) for b, rc in enumerate(reqs)]
        bucket = runner._bucket(batch)
        # as the runner packs a captured decode step: the block tables are resident, a step carries their changes
        buf, layout = pack_step(items, manager, vocab, pad_seqs=bucket, max_blocks=max_blocks, resident=runner.resident,
                                update_cap=runner._update_room(items, bucket, bucket))
        assert layout["fields"] == graph.layout["fields"]
        staged.append(torch.from_numpy(buf))
        for rc in reqs:
            manager.commit(rc, rc.length + 1)
    staged = torch.stack(staged).to(model.device)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def run(k):
        graph.meta_buf[:staged.shape[1]].copy_(staged[k], non_blocking=True)
        graph.graph.replay()
        kernels.argmax(graph.logits[:batch], out)

    for k in range(warmup):
        run(k)
    torch.cuda.synchronize()
    start.record()
    for k in range(warmup, total):
        run(k)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    mean_ctx = context + 1 + warmup + (steps + 1) / 2
    del staged, graph
    return dict(tok_s=batch * steps / (ms / 1e3), ms_per_step=ms / steps, launches_per_step=launches_per_step + 1, mean_ctx=mean_ctx)


def time_prefill(model, tokens, repeats=3, graphs=True):
    """Median device time of one step that holds a whole prompt of ``tokens`` tokens and wants its last logits.  With
    ``graphs`` the step runs as the engine runs it: launched plainly when its shape comes first, captured when it comes
    back, replayed from then on (the timed repeats); the upload of the step's metadata is inside the timed region."""
    import torch

    from litinfer_b200.cache import CacheManager
    from litinfer_b200.engine import ModelRunner, StepItem

    spec = model.spec
    manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], -(-tokens // 16) + 1, 16, 1,
                           model.dtype, model.device)
    runner = ModelRunner(model, manager, use_graphs=graphs)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, spec.vocab_size, (tokens,), generator=g).tolist()
    times = []
    for i in range(repeats + 2):
        rc = manager.admit(i)
        manager.extend(rc, tokens)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepItem(rc, prompt, (tokens - 1,))])
        stop.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(start.elapsed_time(stop))
        manager.release(rc)
    return statistics.median(times)


def time_e2e(model, cfg, batch, prompt_len, new_tokens, steps):
    """Through the Python entry point: host token lists in, host token lists out."""
    import torch

    from litinfer_b200 import Qwen2

    # run_ahead: a decode step is launched before the tokens of the one before it are read back (they stay on the device as
    # its inputs); every step still uploads its metadata from pinned memory and every step's tokens are read to the host
    front = Qwen2(None, model=model, max_num_seqs=batch, max_tokens_per_step=4096, prefill_chunk=2048, run_ahead=True,
                  num_pages=(-(-(prompt_len + new_tokens + 1) // 16)) * batch)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab_size"], (prompt_len,), generator=g).tolist() for _ in range(batch)]
    front.engine_start()
    ids = [front.engine_add_request(p, new_tokens) for p in prompts]
    eng = front._eng()
    # prefill and the first decode steps (graph capture) are outside the timed region
    while any(r.num_cached < prompt_len for r in eng.scheduler.requests.values()):
        front.engine_step()
    for _ in range(4):
        front.engine_step()
    done_before = sum(len(front.engine_get_output(i)) for i in ids)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = 0
    while front.engine_has_unfinished() and n < steps:
        front.engine_step()
        n += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    outs = [front.engine_get_output(i) for i in ids]
    produced = sum(len(o) for o in outs) - done_before
    h2d = eng.runner._graphs[eng.runner._bucket(batch)].meta_buf.numel() * 4
    front.engine_stop()
    return dict(value=produced / dt, steps=n, h2d=h2d, d2h=4 * batch, run_ahead=True)


def time_first_token(model, cfg, prompt_len=16, repeats=7):
    """Milliseconds from ``Qwen2.generate(prompt, 1)`` with a short prompt to its token on the host: LitInfer's own
    headline figure (TTFT of prompts of 10-17 tokens, README.md:69-76, scripts/benchmark_cpu.py:202-253)."""
    import torch

    from litinfer_b200 import Qwen2

    front = Qwen2(None, model=model, max_num_seqs=1, num_pages=16)
    g = torch.Generator().manual_seed(5)
    times = []
    for i in range(repeats + 3):
        prompt = torch.randint(0, cfg["vocab_size"], (prompt_len,), generator=g).tolist()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = front.generate(prompt, max_new_tokens=1)
        dt = time.perf_counter() - t0
        assert len(out) == 1
        if i >= 3:
            times.append(dt * 1e3)
    return statistics.median(times)


def time_mixed(model, batch, context, portion, repeats=4, graphs=True, profiler=None):
    """Median device time of a step that holds ``batch`` requests decoding at about ``context`` tokens beside a portion of
    ``portion`` prompt tokens of another request (what a continuous-batching engine runs while a prompt comes in): as the
    engine runs it, from the captured graph of its shape once that has come back (``graphs``).  ``profiler``: a context
    manager factory entered around the timed steps (for the table of kernels, with the launches made plainly)."""
    import contextlib

    import torch

    from litinfer_b200.cache import CacheManager
    from litinfer_b200.engine import ModelRunner, StepItem

    spec = model.spec
    pages = (batch * (context + 64) + 2 * portion + 4096) // 16
    manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], pages, 16, batch + 2, model.dtype, model.device)
    runner = ModelRunner(model, manager, use_graphs=graphs)
    watch = contextlib.ExitStack()
    g = torch.Generator().manual_seed(4)
    live = []
    for i in range(batch):
        rc = manager.admit(i)
        manager.extend(rc, context)
        toks = torch.randint(0, spec.vocab_size, (context,), generator=g).tolist()
        for lo in range(0, context, 2048):
            runner.step([StepItem(rc, toks[lo:lo + 2048], ())])
        live.append(rc)
    incoming, next_id = manager.admit(batch), batch + 1
    times = []
    for it in range(repeats + 3):
        items = []
        for rc in live:
            manager.extend(rc, rc.length + 1)
            items.append(StepItem(rc, [5], (0,)))
        if incoming.length + portion > min(4000, spec.max_position_embeddings - 1):
            manager.release(incoming)
            incoming, next_id = manager.admit(next_id), next_id + 1
        manager.extend(incoming, incoming.length + portion)
        items.append(StepItem(incoming, torch.randint(0, spec.vocab_size, (portion,), generator=g).tolist(), (portion - 1,)))
        torch.cuda.synchronize()
        if it == 3 and profiler is not None:
            watch.enter_context(profiler())
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step(items)
        stop.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(start.elapsed_time(stop))
    watch.close()
    return statistics.median(times)


def time_serve(model, cfg, requests=64, seed=11, max_tokens_per_step=4096, page_budget_tokens=None):
    """Continuous batching of ``requests`` requests with prompts of 128 to 2,048 tokens and 128 to 512 new tokens each
    through the engine (scheduler, step function, sampler), host tokens in and out.  The pool holds
    ``page_budget_tokens`` tokens (default: three quarters of what all requests would need at their longest, so that
    admission and preemption have to work).  A warm-up pass with the same requests comes first and is not timed."""
    import torch

    from litinfer_b200.engine import Engine, EngineConfig

    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(128, 2049, (requests,), generator=g).tolist()
    news = torch.randint(128, 513, (requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    need = sum(-(-(n + m) // 16) for n, m in zip(lens, news)) * 16
    budget = int(page_budget_tokens or need * 3 // 4)
    eng = Engine(model, EngineConfig(num_pages=budget // 16, max_num_seqs=requests, max_tokens_per_step=max_tokens_per_step,
                                     prefill_chunk=2048, run_ahead=True))
    out = {}
    # a step that does not come back within the limit ends the run with what is known: the status word of the kernels'
    # bounded waits, and the step that was running
    watch = {"at": time.perf_counter(), "what": "start", "stop": False}

    def watchdog(limit=float(os.environ.get("LITINFER_BENCH_STEP_LIMIT_S", "45"))):
        from litinfer_b200 import kernels as K

        while not watch["stop"]:
            time.sleep(1.0)
            if time.perf_counter() - watch["at"] > limit:
                print(f"[serve] no step for {limit:.0f} s; kernels' status word {K.library().li_tcgen05_status()}; last: {watch['what']}",
                      file=sys.stderr, flush=True)
                os._exit(7)

    threading.Thread(target=watchdog, daemon=True).start()
    for timed in (False, True):
        ids = [eng.add_request(p, m) for p, m in zip(prompts, news)]
        steps, pre0, replay0 = [], eng.scheduler.num_preemptions, eng.runner.graph_replays
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while eng.has_unfinished():
            t = time.perf_counter()
            running = eng.scheduler.running
            watch["at"], watch["what"] = t, (f"{'timed' if timed else 'warm-up'} step {len(steps)}: {len(running)} running "
                                             f"(cached {[r.num_cached for r in running][:70]}), {len(eng.scheduler.waiting)} waiting, "
                                             f"graph replays {eng.runner.graph_replays}")
            eng.step()
            steps.append(time.perf_counter() - t)
            if len(steps) % 200 == 0:
                print(f"[serve] {'timed' if timed else 'warm-up'} pass: step {len(steps)}, {len(eng.scheduler.running)} running, "
                      f"{len(eng.scheduler.waiting)} waiting, {eng.tokens_run} tokens run, {time.perf_counter() - t0:.1f} s",
                      file=sys.stderr, flush=True)
        eng.drain()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        produced = sum(len(eng.get_output(i)) for i in ids)
        for i in ids:
            eng.scheduler.forget(i)
        steps.sort()
        out = dict(seconds=dt, generated=produced, prompt_tokens=sum(lens), tok_s=produced / dt, total_tok_s=(produced + sum(lens)) / dt,
                   steps=len(steps), mean_step_ms=1e3 * sum(steps) / len(steps), p95_step_ms=1e3 * steps[int(0.95 * (len(steps) - 1))],
                   preemptions=eng.scheduler.num_preemptions - pre0, steps_from_graphs=eng.runner.graph_replays - replay0,
                   steps_launched_plainly=len(steps) - (eng.runner.graph_replays - replay0), pool_tokens=budget, needed_tokens=need)
    watch["stop"] = True
    return out


def time_chunked(model, cfg, decoding=32, context=4096, prompt=2048, portion=512, peaks=None):
    """A prompt of ``prompt`` tokens fed in portions of ``portion`` beside ``decoding`` requests that decode at a context of
    ``context``: device milliseconds of each of the prompt's steps (median over three prompts, after one for warm-up and
    graph capture), and what fraction of the roofline of its bytes (weights once, the caches read) and of its flops that is."""
    import torch

    from litinfer_b200.cache import CacheManager
    from litinfer_b200.engine import ModelRunner, StepItem

    spec = model.spec
    pages = (decoding * (context + 64) + 2 * prompt + 4096) // 16
    manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], pages, 16, decoding + 2, model.dtype, model.device)
    for grp in manager.groups:
        grp.kv.normal_(0.0, 0.5)
    runner = ModelRunner(model, manager, use_graphs=True, max_context=min(spec.max_position_embeddings, context + 64))
    g = torch.Generator().manual_seed(4)
    live = []
    for i in range(decoding):
        rc = manager.admit(i)
        manager.extend(rc, context)
        manager.commit(rc, context)                         # the cache holds random values: a decode step's time does not depend on them
        live.append(rc)
    next_id = decoding
    per_step = [[] for _ in range(prompt // portion)]
    for rep in range(4):
        incoming = manager.admit(next_id)
        next_id += 1
        toks = torch.randint(0, spec.vocab_size, (prompt,), generator=g).tolist()
        for k in range(prompt // portion):
            items = []
            for rc in live:
                if rc.length + 1 > context + 48:              # keep the decoding requests near the context asked for
                    manager.commit(rc, context)
                manager.extend(rc, rc.length + 1)
                items.append(StepItem(rc, [5], (0,)))
            manager.extend(incoming, incoming.length + portion)
            items.append(StepItem(incoming, toks[k * portion:(k + 1) * portion], (portion - 1,)))
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step(items)
            stop.record()
            torch.cuda.synchronize()
            if rep >= 1:
                per_step[k].append(start.elapsed_time(stop))
        manager.release(incoming)
    ms = [statistics.median(x) for x in per_step]
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    nh, nkv, dh = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    wbytes = weight_bytes(model)
    kv_token = 2 * L * nkv * dh * 2
    out = []
    for k, m in enumerate(ms):
        cached = k * portion
        tokens = decoding + portion
        flops = 2 * (H * (nh + 2 * nkv) * dh + nh * dh * H + 3 * H * I) * L * tokens + 2 * H * cfg["vocab_size"] * (decoding + 1)
        flops += 2 * 2 * nh * dh * L * (decoding * context + portion * cached + portion * (portion + 1) // 2)
        nbytes = wbytes + kv_token * (decoding * context + cached + portion)
        out.append(dict(step=k, cached_prompt_tokens=cached, ms=round(m, 3), hbm_frac=round(nbytes / (m / 1e3) / (peaks["hbm_gbs"] * 1e9), 4),
                        flops_frac=round(flops / (m / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)))
    return out


def fp32_check(cfg, layers=2, tokens=48, seed=3):
    """The largest |difference| between the engine's float32 logits and the plain implementation of the tests on ``layers``
    layers of the benchmark's sizes: the same random weights on both sides (drawn on the device by the library's kernel,
    restated on the host bit for bit), a prompt of ``tokens`` tokens whole."""
    import torch

    sys.path.insert(0, str(ROOT / "tests"))
    import plain_qwen2 as P

    from litinfer_b200.cache import CacheManager
    from litinfer_b200.config import config_from_dict
    from litinfer_b200.engine import ModelRunner, StepItem
    from litinfer_b200.models import DecoderModel
    from litinfer_b200.models.decoder import declared_params
    from litinfer_b200.weights.random_init import random_tensor

    small = dict(cfg, num_hidden_layers=layers, torch_dtype="float32")
    spec = config_from_dict(small).to_model_spec()
    model = DecoderModel.from_random(spec, seed, "float32", "cuda:0")
    manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], -(-tokens // 16) + 1, 16, 1, model.dtype, model.device)
    runner = ModelRunner(model, manager)
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, small["vocab_size"], (tokens,), generator=g).tolist()
    rc = manager.admit(0)
    manager.extend(rc, tokens)
    got = runner.step([StepItem(rc, toks, list(range(tokens)))]).cpu()
    del model, runner, manager
    torch.cuda.empty_cache()
    weights = {p.name: random_tensor(p, seed, "cpu", torch.float32) for p in declared_params(spec) if p.draw}
    ref = P.plain_forward(dict(small), weights, toks)
    return dict(layers=layers, tokens=tokens, max_abs_err=float((got - ref).abs().max()), max_abs_logit=float(ref.abs().max()))


def run_reference(args):
    """The reference arm: the unmodified LitInfer (built with g++ by baseline/build_reference.py, since its own build
    needs xmake) through its stock ``Qwen2(...).engine_*`` path on the CPU, which is the only device it runs on, for
    the same metric and configuration.  A one-layer run comes first; if the full run would not fit the time this arm
    may take (LITINFER_REF_BUDGET_S, default 900 s) the line says `unavailable` with the measured extrapolation."""
    import shutil
    import tempfile

    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        import build_reference

        build_reference.build(verbose=True)
    except Exception as e:                                   # no sources, no compiler, a compile error
        return {"impl": "reference", "unavailable": f"LitInfer's native library could not be built here: {str(e)[:300]}"}
    from litinfer_b200.weights import write_model_folder      # writes files only: no model, kernel or engine of this repository

    budget = float(os.environ.get("LITINFER_REF_BUDGET_S", "900"))
    cfg = bench_config(args.shape)
    cfg["eos_token_id"] = -1                                  # LitInfer wants an integer; no token has this id
    warmup = max(args.warmup, 3)
    cores = os.cpu_count() or 1

    def run(layers, batch, context, steps, warm):
        d = tempfile.mkdtemp(prefix="litinfer_ref_")
        try:
            write_model_folder(d, dict(cfg, num_hidden_layers=layers), seed=0, store_dtype="bfloat16")
            pages = batch * (-(-(context + steps + warm + 4) // 16)) + 8
            env = dict(os.environ, LLAISYS_NUM_BLOCKS=str(pages))          # LitInfer's own knob for the size of its page pool
            r = subprocess.run([sys.executable, str(ROOT / "baseline" / "run_reference.py"), "--model", d, "--batch", str(batch), "--context",
                                str(context), "--steps", str(steps), "--warmup", str(warm), "--vocab", str(cfg["vocab_size"])],
                               capture_output=True, text=True, env=env, timeout=max(budget * 2, 600))
            if r.returncode != 0:
                raise RuntimeError((r.stderr or r.stdout)[-400:])
            return json.loads(r.stdout.strip().splitlines()[-1])
        finally:
            shutil.rmtree(d, ignore_errors=True)

    try:
        cal = run(1, args.batch, 256, 3, 1)
    except Exception as e:
        return {"impl": "reference", "unavailable": f"LitInfer's CPU engine failed on a one-layer model of this configuration: {str(e)[:300]}"}
    L = cfg["num_hidden_layers"]
    est_prefill = cal["prefill_s"] * (args.batch * args.context / cal["prefill_tokens"]) * L
    est_decode = cal["ms_per_step"] / 1e3 * L * (args.steps + warmup)
    est = cal["load_s"] * L / 2 + est_prefill + est_decode
    calibration = {"layers": 1, "cpu_cores": cores, "prefill_tok_s": round(cal["prefill_tokens"] / cal["prefill_s"], 1),
                   "decode_ms_per_step": round(cal["ms_per_step"], 2), "estimated_full_run_s": round(est, 0)}
    if est > budget:
        return {"impl": "reference", "calibration": calibration, "unavailable":
                f"LitInfer has no GPU path; its CPU engine, measured here on one layer of this configuration ({cores} cores: "
                f"{calibration['prefill_tok_s']} prompt tokens/s, {calibration['decode_ms_per_step']} ms a decode step at batch {args.batch}), would need "
                f"about {est:.0f} s for the {L}-layer run (prefill of {args.batch} x {args.context} tokens, then {args.steps + warmup} steps): "
                f"beyond the {budget:.0f} s this arm may take"}
    try:
        full = run(L, args.batch, args.context, args.steps, warmup)
    except Exception as e:
        return {"impl": "reference", "calibration": calibration, "unavailable": f"LitInfer's CPU engine failed on the full configuration: {str(e)[:300]}"}
    return {
        "metric": f"decode tok/s @ batch {args.batch} ({args.shape.upper()} shape, context {args.context}+)", "value": round(full["tok_s"], 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(full["ms_per_step"], 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (LitInfer runs bfloat16 files as float16)",
        "data": "synthetic: random-init weights N(0, 0.02), random token ids", "impl": "reference", "device": f"cpu ({cores} cores)",
        "config": {"model": SHAPES[args.shape]["name"], "layers": L, "global_batch": args.batch, "seq_len": args.context,
                   "new_tokens": args.steps + warmup, "page_size": 16, "parallelism": "CPU, OpenMP"},
        "prefill": {"value": round(full["prefill_tokens"] / full["prefill_s"], 1), "tokens": full["prefill_tokens"], "ms": round(full["prefill_s"] * 1e3, 1)},
        "calibration": calibration,
    }


def main() -> int:
    if os.environ.get("LITINFER_BENCH_STACKS"):          # where the program is, every so many seconds, on stderr
        import faulthandler

        faulthandler.dump_traceback_later(float(os.environ["LITINFER_BENCH_STACKS"]), repeat=True)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (named in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--shape", default="1.5b", choices=sorted(SHAPES), help="layer sizes: the headline 1.5B shape, or the 7B / 14B shapes of the larger workloads")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "mixed", "kernels-decode", "kernels-prefill", "kernels-mixed", "serve", "chunked", "fp32"],
                    help="measure one part and print a short line (for profiling runs); kernels-*: a table of the "
                         "kernels' device times from torch.profiler; mixed: --batch requests decoding at --context beside "
                         "a portion of --prefill-tokens prompt tokens")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel from the host (so that a profiler lists them)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    import torch

    from litinfer_b200 import kernels
    from litinfer_b200.config import config_from_dict
    from litinfer_b200.models import DecoderModel

    cfg = bench_config(args.shape)
    full_layers = cfg["num_hidden_layers"]
    if args.only == "fp32":
        print(json.dumps({"only": "fp32", "shape": args.shape, **fp32_check(cfg)}))
        return 0
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    if args.only in ("decode", "kernels-decode") and args.context + 4096 > cfg["max_position_embeddings"]:
        # a longer context than the shape's own limit, on request: the measurement's model allows it
        cfg["max_position_embeddings"] = args.context + 4096
    peaks = load_peaks()
    spec = config_from_dict(cfg).to_model_spec()
    model = DecoderModel.from_random(spec, 0, "bfloat16", "cuda:0")
    wbytes = weight_bytes(model)
    kv_per_token = 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2

    if args.only in ("kernels-decode", "kernels-prefill", "kernels-mixed"):
        from torch.profiler import ProfilerActivity, profile

        if args.only == "kernels-decode":
            time_decode(model, args.batch, args.context, 8, warmup)             # builds the graph, warms up
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                r = time_decode(model, args.batch, args.context, args.steps, warmup)
            print(json.dumps({"only": args.only, "batch": args.batch, "steps": args.steps + warmup, **{k: round(v, 4) for k, v in r.items()}}))
        elif args.only == "kernels-mixed":
            holder = {}

            def watching():
                holder["prof"] = profile(activities=[ProfilerActivity.CUDA])
                return holder["prof"]

            ms = time_mixed(model, args.batch, args.context, args.prefill_tokens, graphs=False, profiler=watching)
            prof = holder["prof"]
            print(json.dumps({"only": args.only, "decoding": args.batch, "context": args.context, "portion": args.prefill_tokens,
                              "ms_launched_plainly": round(ms, 3), "steps_in_table": 4}))
        else:
            time_prefill(model, args.prefill_tokens, repeats=1, graphs=False)
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                ms = time_prefill(model, args.prefill_tokens, repeats=1, graphs=False)
            print(json.dumps({"only": args.only, "tokens": args.prefill_tokens, "ms": round(ms, 3), "runs_in_table": 3}))
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=16, max_name_column_width=70))
        return 0
    if args.only == "decode":
        r = time_decode(model, args.batch, args.context, args.steps, warmup, graphs=not args.no_graphs)
        print(json.dumps({"only": "decode", "batch": args.batch, "context": args.context, "layers_run": cfg["num_hidden_layers"],
                          "graphs": not args.no_graphs, **{k: round(v, 4) for k, v in r.items()}}))
        return 0
    if args.only == "serve":
        r = time_serve(model, cfg)
        print(json.dumps({"only": "serve", "shape": args.shape, "model": SHAPES[args.shape]["name"], "layers_run": cfg["num_hidden_layers"],
                          "requests": 64, **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()}}))
        return 0
    if args.only == "chunked":
        r = time_chunked(model, cfg, peaks=peaks)
        print(json.dumps({"only": "chunked", "shape": args.shape, "model": SHAPES[args.shape]["name"], "layers_run": cfg["num_hidden_layers"],
                          "decoding": 32, "context": 4096, "prompt": 2048, "portion": 512, "peaks": peaks["source"], "steps": r}))
        return 0
    if args.only == "mixed":
        ms = time_mixed(model, args.batch, args.context, args.prefill_tokens)
        print(json.dumps({"only": "mixed", "decoding": args.batch, "context": args.context, "portion": args.prefill_tokens,
                          "layers_run": cfg["num_hidden_layers"], "ms": round(ms, 3),
                          "tok_s": round((args.batch + args.prefill_tokens) / ms * 1e3, 1)}))
        return 0
    if args.only == "prefill":
        ms = time_prefill(model, args.prefill_tokens, graphs=not args.no_graphs)
        fl = decode_flops_and_prefill_flops(cfg, args.prefill_tokens)
        print(json.dumps({"only": "prefill", "tokens": args.prefill_tokens, "graphs": not args.no_graphs, "layers_run": cfg["num_hidden_layers"], "ms": round(ms, 3),
                          "tok_s": round(args.prefill_tokens / ms * 1e3, 1), "frac": round(fl / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    main_run = time_decode(model, args.batch, args.context, args.steps, warmup)
    clock_info = clocks.stop()

    step_bytes = wbytes + args.batch * main_run["mean_ctx"] * kv_per_token
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    prefill_tokens = 2048
    pf_ms = time_prefill(model, prefill_tokens)
    pf_flops = decode_flops_and_prefill_flops(cfg, prefill_tokens)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(time_decode(model, b, args.context, min(args.steps, 64), warmup)["tok_s"], 1)
        points["first_token_ms_prompt16"] = round(time_first_token(model, cfg), 3)
    e2e = time_e2e(model, cfg, args.batch, args.context, 256, args.steps)
    del model
    torch.cuda.empty_cache()
    check = fp32_check(cfg)

    line = {
        "metric": f"decode tok/s @ batch {args.batch} ({args.shape.upper()} shape, context {args.context}+)",
        "value": round(main_run["tok_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random-init weights N(0, 0.02), random token ids",
        "impl": "ours",
        "config": {
            "model": SHAPES[args.shape]["name"], "layers": full_layers, "layers_run": cfg["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": args.batch, "seq_len": args.context, "new_tokens": args.steps + warmup, "context_cap": 4096,
            "page_size": 16, "parallelism": "single GPU", "cache_refresh": f"inputs larger than L2 ({wbytes / 1e9:.1f} GB of weights per step)",
            "peaks": peaks["source"],
        },
        "e2e": {"value": round(e2e["value"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                "steps": e2e["steps"], "run_ahead": True},
        "gpu_launches": int(main_run["launches_per_step"] * args.steps),
        "clocks": clock_info,
        "prefill": {"value": round(prefill_tokens / (pf_ms / 1e3), 1), "tokens": prefill_tokens, "ms": round(pf_ms, 3),
                    "frac": round(pf_flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "fp32_check": {k: (round(v, 7) if isinstance(v, float) else v) for k, v in check.items()},
        "kernel_library": kernels.library_file(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
