"""Command line: token ids in, token ids out.

    python -m litinfer_b200 --model DIR --prompt "151646 1986 374" --max_steps 32

LitInfer has no generation program of its own; its scripts take ``--model``,
``--device``, ``--prompt``, ``--max_steps``, ``--top_k``, ``--top_p``,
``--temperature``, ``--test`` (test/test_infer.py:172-183) and ``--repeats``,
``--output`` (scripts/benchmark_cpu.py:176-187).  Those names and meanings are
kept.  There is no tokenizer here (LitInfer's core has none either; its
scripts borrow one), so ``--prompt`` holds token ids.  ``--random-config``
writes a model folder with random weights first, from a config.json and a seed.
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
from pathlib import Path


def parse_ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="litinfer_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", help="folder with config.json and *.safetensors")
    ap.add_argument("--random-config", help="a config.json: make a model folder with random weights from it (see --random-seed, --save-model)")
    ap.add_argument("--random-seed", type=int, default=0)
    ap.add_argument("--save-model", help="where --random-config writes the folder (default: a temporary one)")
    ap.add_argument("--device", default="nvidia", choices=["nvidia", "cuda", "cuda:0"], help="LitInfer's scripts say cpu|nvidia; this engine runs on the GPU")
    ap.add_argument("--dtype", default=None, choices=["bfloat16", "float32"], help="default: from config.json's torch_dtype")
    ap.add_argument("--prompt", action="append", dest="prompts", help="token ids, separated by spaces or commas; may be given several times")
    ap.add_argument("--prompt-file", help="a file with one prompt (token ids) per line")
    ap.add_argument("--max_steps", default=128, type=int, help="new tokens per prompt")
    ap.add_argument("--top_p", default=0.8, type=float)
    ap.add_argument("--top_k", default=50, type=int)
    ap.add_argument("--temperature", default=1.0, type=float)
    ap.add_argument("--seed", default=0, type=int, help="seed of the sampling draws (per request)")
    ap.add_argument("--test", action="store_true", help="greedy decoding (top_k 1, top_p 1, temperature 1), as LitInfer's --test")
    ap.add_argument("--repeats", default=1, type=int, help="run each prompt this many times; timings are of the last run")
    ap.add_argument("--batch", action="store_true", help="run all prompts together through the continuous-batching engine")
    ap.add_argument("--num-pages", type=int, default=None, help="pages of 16 tokens in the cache pool (LLAISYS_NUM_BLOCKS also works)")
    ap.add_argument("--max-tokens-per-step", type=int, default=2048)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--output", help="write the results as JSON here as well")
    args = ap.parse_args(argv)

    if bool(args.model) == bool(args.random_config):
        ap.error("give exactly one of --model and --random-config")
    prompts = [parse_ids(p) for p in (args.prompts or [])]
    if args.prompt_file:
        prompts += [parse_ids(l) for l in Path(args.prompt_file).read_text().splitlines() if l.strip()]
    if not prompts:
        ap.error("no prompt: give --prompt or --prompt-file")
    if args.max_steps <= 0 or args.repeats <= 0:
        ap.error("--max_steps and --repeats must be positive")
    top_k, top_p, temperature = (1, 1.0, 1.0) if args.test else (args.top_k, args.top_p, args.temperature)

    from . import Qwen2
    from .weights import write_model_folder

    tmp = None
    model_dir = args.model
    if args.random_config:
        cfg = json.loads(Path(args.random_config).read_text())
        if args.save_model:
            model_dir = args.save_model
        else:
            tmp = tempfile.TemporaryDirectory()
            model_dir = tmp.name
        write_model_folder(model_dir, cfg, args.random_seed, store_dtype="bfloat16" if cfg.get("torch_dtype") != "float32" else "float32")
    model = Qwen2(model_dir, device="cuda:0", dtype=args.dtype, num_pages=args.num_pages, max_tokens_per_step=args.max_tokens_per_step,
                  prefill_chunk=args.prefill_chunk)
    results = []
    if args.batch:
        model.engine_start()
        ids = [model.engine_add_request(p, args.max_steps, top_k, top_p, temperature, args.seed + i) for i, p in enumerate(prompts)]
        steps = 0
        while model.engine_has_unfinished():
            model.engine_step()
            steps += 1
        for p, i in zip(prompts, ids):
            results.append({"prompt_tokens": len(p), "tokens": model.engine_get_output(i)})
        model.engine_stop()
        summary = {"engine_steps": steps}
    else:
        for i, p in enumerate(prompts):
            for _ in range(args.repeats):
                toks, metrics = model.generate_profile(p, args.max_steps, top_k, top_p, temperature, args.seed + i)
            results.append({"prompt_tokens": len(p), "tokens": toks, **metrics})
        summary = {}
    out = {"model": str(model_dir), "dtype": str(model.model.dtype).replace("torch.", ""), "top_k": top_k, "top_p": top_p,
           "temperature": temperature, "results": results, **summary}
    for r in results:
        print(" ".join(str(t) for t in r["tokens"]), flush=True)
    if args.output:
        Path(args.output).write_text(json.dumps(out, indent=1))
    if tmp is not None:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
