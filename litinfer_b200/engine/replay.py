"""Trace replay: given token ids through the model step by step, logits out.

The program ``bin/trace_run`` is a thin wrapper around :func:`replay`.  It
samples nothing and has no forward pass, cache or loader of its own: it admits
requests to the engine's cache manager, allocates their pages, calls the
engine's step function and gives the pages back when told so.  LitInfer has
nothing like it; its closest test compares one argmax token of a 3-token
prompt fed whole and one by one (test/test_kv_cache.py:52-66).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, IO, Iterable, Optional

import torch

from ..cache.manager import CacheManager, RequestCache
from ..models.decoder import DecoderModel
from .batch import StepItem
from .step import ModelRunner


class Replayer:
    def __init__(self, model: DecoderModel, max_tokens: int, page_size: int = 16, max_live: int = 8, use_graphs: bool = True,
                 step_graph_after: int = 1) -> None:
        spec = model.spec
        self.model = model
        num_pages = max(1, -(-int(max_tokens) // page_size))
        self.manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], num_pages, page_size,
                                    max_live, model.dtype, model.device)
        max_context = min(spec.max_position_embeddings, num_pages * page_size)
        # (the runner captures nothing for a model with a mixer that has state of its own)
        self.runner = ModelRunner(model, self.manager, use_graphs=use_graphs, max_context=max_context,
                                  step_graph_after=step_graph_after)
        self.live: Dict[str, RequestCache] = {}
        self._next_id = 0

    def step(self, record: dict) -> torch.Tensor:
        """Run one step record; returns float32 logits [wanted, vocab] (possibly empty)."""
        items = []
        for e in record.get("entries", []):
            rid = str(e["id"])
            if rid not in self.live:
                self.live[rid] = self.manager.admit(self._next_id)
                self._next_id += 1
            rc = self.live[rid]
            toks = [int(t) for t in e["tokens"]]
            self.manager.extend(rc, rc.length + len(toks))
            items.append(StepItem(rc, toks, [int(w) for w in e.get("want", [])]))
        if items:
            logits = self.runner.step(items)
        else:
            logits = torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.model.device)
        for rid in record.get("end", []):
            rc = self.live.pop(str(rid), None)
            if rc is not None:
                self.manager.release(rc)
        return logits


def replay(model: DecoderModel, lines: Iterable[str], out_dir, max_tokens: int, page_size: int = 16, max_live: int = 8,
           use_graphs: bool = True, report: Optional[IO[str]] = None, step_graph_after: int = 1) -> None:
    """Feed the step records in ``lines``; write ``<step>.f32`` files; print ``done <step>`` to ``report``."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    rp = Replayer(model, max_tokens, page_size, max_live, use_graphs, step_graph_after)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = rp.step(record)
        if logits.shape[0]:
            logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4").tofile(out_dir / f"{record['step']}.f32")
        if report is not None:
            print(f"done {record['step']}", file=report, flush=True)
