"""The Python entry point, in the manner of LitInfer's ``llaisys.models.Qwen2``
(python/llaisys/models/qwen2.py:23-501): token ids in, token ids out.

    model = Qwen2(model_path)
    tokens = model.generate(input_ids, max_new_tokens=32)

Names and meanings of methods and options are LitInfer's where it has them:
``generate / generate_profile / generate_stream`` with ``max_new_tokens``,
``top_k``, ``top_p``, ``temperature`` (defaults 1, 1.0, 1.0: greedy), and the
``engine_*`` methods of its continuous-batching interface.  Differences, all
deliberate: ``seed`` makes sampling reproducible per request; the first token
is sampled like every other one (LitInfer always takes it greedily,
qwen2.py:359); sampling options may be given per request in
``engine_add_request``; the class is chosen by config.json's ``architectures``
through the registry, so :func:`load_model` works for any registered one.
"""

from __future__ import annotations

import os
import time
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from .config import load_config
from .engine import Engine, EngineConfig
from .models import DecoderModel
from .sampling import SamplingParams


def _default_dtype(config) -> str:
    # float32 checkpoints run in float32, everything else in bfloat16 (LitInfer runs
    # bfloat16 checkpoints as float16, python/llaisys/models/qwen2.py:253-264)
    return "float32" if getattr(config, "torch_dtype", "bfloat16") in ("float32", "fp32") else "bfloat16"


class CausalLM:
    """A model folder (config.json + safetensors) of any registered architecture, ready to generate on one GPU.
    :data:`Qwen2` is this class under LitInfer's name for it."""

    def __init__(self, model_path, device="cuda:0", quantize=None, dtype: Optional[str] = None,
                 num_pages: Optional[int] = None, max_num_seqs: int = 64, max_tokens_per_step: int = 2048,
                 prefill_chunk: int = 2048, use_graphs: bool = True, run_ahead: bool = True,
                 model: Optional[DecoderModel] = None) -> None:
        if quantize is not None:
            raise ValueError("quantized weights are not supported by this engine")
        dev = torch.device(device)
        if model is None:
            if dev.type != "cuda":
                raise RuntimeError(f"this engine runs on a CUDA device (B200) only, got device '{device}'")
            config = load_config(model_path)
            model = DecoderModel.from_dir(model_path, dtype or _default_dtype(config), dev)
        self.model = model
        self.spec = model.spec
        self.device = model.device
        self._engine_options = dict(max_num_seqs=max_num_seqs, max_tokens_per_step=max_tokens_per_step,
                                    prefill_chunk=prefill_chunk, use_graphs=use_graphs, run_ahead=run_ahead)
        self._num_pages = num_pages
        self._engine: Optional[Engine] = None
        self._single: Optional[Engine] = None

    # ------------------------------------------------------------------
    @property
    def end_token(self) -> int:
        return self.spec.eos_token_ids[0] if self.spec.eos_token_ids else -1

    def _default_pages(self, max_num_seqs: int) -> int:
        env = os.environ.get("LLAISYS_NUM_BLOCKS")              # LitInfer's override (src/llaisys/models/qwen2.cpp:121-125)
        if env and int(env) > 0:
            return int(env)
        if self._num_pages:
            return int(self._num_pages)
        per_seq = -(-self.spec.max_position_embeddings // 16)
        want = per_seq * max_num_seqs
        if self.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.device)
            probe = Engine.bytes_per_page(self.model, 16)
            want = max(per_seq, min(want, int(free * 0.4) // max(probe, 1)))
        return want

    def _make_engine(self, **overrides) -> Engine:
        opts = dict(self._engine_options)
        opts.update(overrides)
        pages = self._default_pages(opts["max_num_seqs"])
        cfg = EngineConfig(num_pages=pages, page_size=16, max_num_seqs=opts["max_num_seqs"],
                           max_tokens_per_step=opts["max_tokens_per_step"], prefill_chunk=opts["prefill_chunk"],
                           use_graphs=opts["use_graphs"], run_ahead=bool(opts.get("run_ahead", True)))
        return Engine(self.model, cfg)

    # ------------------------------------------------------------------
    # single request
    # ------------------------------------------------------------------
    def generate(self, inputs: Sequence[int], max_new_tokens: Optional[int] = None, top_k: int = 1, top_p: float = 1.0,
                 temperature: float = 1.0, seed: int = 0) -> List[int]:
        tokens, _ = self.generate_profile(inputs, max_new_tokens, top_k, top_p, temperature, seed)
        return tokens

    def generate_profile(self, inputs: Sequence[int], max_new_tokens: Optional[int] = None, top_k: int = 1, top_p: float = 1.0,
                         temperature: float = 1.0, seed: int = 0) -> Tuple[List[int], Dict[str, float]]:
        """Tokens and the timing dictionary of LitInfer's ``generate_profile`` (qwen2.py:399-407)."""
        tokens: List[int] = []
        t0 = time.perf_counter()
        first = None
        for tok in self.generate_stream(inputs, 1 if max_new_tokens is None else max_new_tokens, top_k, top_p, temperature, seed):
            if first is None:
                first = time.perf_counter() - t0
            tokens.append(tok)
        total = time.perf_counter() - t0
        prefill = first if first is not None else total
        decode_seconds = total - prefill
        decode_tokens = max(len(tokens) - 1, 0)
        return tokens, {
            "prefill_seconds": prefill if max_new_tokens is None or max_new_tokens > 0 else 0.0,
            "first_token_seconds": prefill if max_new_tokens is None or max_new_tokens > 0 else 0.0,
            "decode_seconds": decode_seconds,
            "decode_tokens": decode_tokens,
            "decode_tokens_per_second": decode_tokens / decode_seconds if decode_seconds > 0 and decode_tokens else 0.0,
            "time_per_decode_token_seconds": decode_seconds / decode_tokens if decode_tokens else 0.0,
            "generated_tokens": len(tokens),
        }

    def generate_stream(self, inputs: Sequence[int], max_new_tokens: int = 128, top_k: int = 1, top_p: float = 1.0,
                        temperature: float = 1.0, seed: int = 0) -> Iterator[int]:
        """Yield token ids as they are produced; the end-of-sequence token is not yielded."""
        max_new_tokens = 1 if max_new_tokens is None else max_new_tokens
        if max_new_tokens <= 0:
            return
        prompt = [int(t) for t in inputs]
        if not prompt:
            raise ValueError("generate: inputs must not be empty")
        if len(prompt) + max_new_tokens - 1 > self.spec.max_position_embeddings:
            raise ValueError(
                f"generate: requested prompt and output exceed model max sequence length ({self.spec.max_position_embeddings})")
        if self._single is None:
            self._single = self._make_engine(max_num_seqs=1)
        eng = self._single
        from . import kernels as K

        if K.TRACE:                                  # LitInfer prints the same kind of line (python/llaisys/models/qwen2.py:351-357)
            import sys

            print(f"[LLAISYS] Calling generate ntokens={len(prompt)} max_new_tokens={max_new_tokens}", file=sys.stderr, flush=True)
        rid = eng.add_request(prompt, max_new_tokens, SamplingParams(temperature, top_k, top_p, seed))
        sent = 0
        try:
            while not eng.is_finished(rid):
                eng.step()
                out = eng.scheduler.requests[rid].generated
                while sent < len(out):
                    yield out[sent]
                    sent += 1
        finally:
            eng.abort(rid)                       # reads a step launched ahead, then frees pages if the caller stopped early; no-op when finished
            eng.scheduler.forget(rid)

    # ------------------------------------------------------------------
    # continuous batching
    # ------------------------------------------------------------------
    def engine_start(self, **options) -> None:
        self._engine = self._make_engine(**options)

    def _eng(self) -> Engine:
        if self._engine is None:
            raise RuntimeError("engine_start() has not been called")
        return self._engine

    def engine_add_request(self, inputs: Sequence[int], max_new_tokens: int = 128, top_k: int = 1, top_p: float = 1.0,
                           temperature: float = 1.0, seed: int = 0) -> int:
        return self._eng().add_request(inputs, max_new_tokens, SamplingParams(temperature, top_k, top_p, seed))

    def engine_step(self) -> int:
        """One scheduling iteration; returns how many requests finished in it."""
        return len(self._eng().step())

    def engine_has_unfinished(self) -> bool:
        return self._eng().has_unfinished()

    def engine_num_seqs(self) -> int:
        return self._eng().num_seqs()

    def engine_is_finished(self, req_id: int) -> bool:
        return self._eng().is_finished(req_id)

    def engine_get_output(self, req_id: int) -> List[int]:
        return self._eng().get_output(req_id)

    def engine_stop(self) -> None:
        self._engine = None


Qwen2 = CausalLM            # LitInfer's name (python/llaisys/models/qwen2.py:23); the class itself serves any registered architecture


def load_model(model_path, **kwargs) -> CausalLM:
    """The front end for whatever registered architecture config.json names."""
    return CausalLM(model_path, **kwargs)
