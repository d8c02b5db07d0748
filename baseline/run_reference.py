"""Drives the unmodified LitInfer (its Python layer and native library under ``baseline/_ref``) through its own public
interface for the benchmark's decode measurement, and prints one JSON object.

    python baseline/run_reference.py --model DIR --batch 8 --context 2048 --steps K --warmup W

It follows LitInfer's stock path: ``Qwen2(model_path)`` (python/llaisys/models/qwen2.py:25-208), ``engine_start``,
``engine_add_request`` for every prompt, then ``engine_step`` (qwen2.py:458-496 -> src/llaisys/models/qwen2.cpp:922-1080),
whose first call takes in all the prompts and every further call decodes one token per request.  Timed: exactly K such
decode steps after W untimed ones, with the host's clock (LitInfer runs on the CPU and its calls return when the work is
done).  Nothing of this repository's engine is imported here.
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--vocab", type=int, required=True)
    args = ap.parse_args()
    sys.path.insert(0, str(HERE / "_ref"))
    import llaisys                                           # noqa: F401  (LitInfer's package)
    from llaisys.models.qwen2 import Qwen2

    t0 = time.perf_counter()
    model = Qwen2(args.model)
    load_s = time.perf_counter() - t0
    rng = random.Random(3)
    prompts = [[rng.randrange(args.vocab) for _ in range(args.context)] for _ in range(args.batch)]
    model.engine_start()
    for p in prompts:
        model.engine_add_request(p, args.steps + args.warmup + 2)
    def step():
        if model.engine_step() < 0:
            raise RuntimeError("LitInfer's engine_step failed (see its message above; the page pool is sized by LLAISYS_NUM_BLOCKS)")

    t0 = time.perf_counter()
    step()                                                   # takes in the prompts and produces each request's first token
    prefill_s = time.perf_counter() - t0
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    decode_s = time.perf_counter() - t0
    model.engine_stop()
    print(json.dumps({"load_s": load_s, "prefill_s": prefill_s, "prefill_tokens": args.batch * args.context, "decode_s": decode_s,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * decode_s / args.steps,
                      "tok_s": args.batch * args.steps / decode_s}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
