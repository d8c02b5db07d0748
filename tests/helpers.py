"""Helpers of the tests: traces for replay, tolerances, plain logits."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_qwen2 as P

ROOT = Path(__file__).resolve().parent.parent

# Float32: two independent float32 implementations of these tiny models differ by a few
# 1e-7 in the logits (measured between LitInfer's ops and a plain forward); 1e-4 leaves
# room for the longer sums of real layer sizes (rows of 8,960 products) and is still far
# below any real fault (a wrong key moves logits by 1e-2).
F32_ATOL = 1e-4
# bfloat16 against the plain model in float32 on the same (bfloat16-rounded) weights:
# activations are rounded to 8 bits of mantissa (relative step 2^-8) at roughly ten places
# per layer; the bound is relative to the largest logit of the sequence.
BF16_REL = 0.03
BF16_MEAN_REL = 0.006


def bf16_round(w: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """What the bfloat16 engine holds: matrices rounded to bfloat16, vectors kept in float32."""
    return {k: (v.to(torch.bfloat16).float() if v.dim() >= 2 else v) for k, v in w.items()}


def check_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "") -> None:
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    err = (got - ref).abs()
    if dtype == "float32":
        worst = int(err.max(dim=-1).values.argmax()) if err.dim() == 2 else 0
        assert err.max() <= F32_ATOL, f"{what}: max |diff| {err.max():.3e} at row {worst} (float32 bound {F32_ATOL})"
    else:
        scale = ref.abs().max()
        worst = int(err.max(dim=-1).values.argmax()) if err.dim() == 2 else 0
        assert err.max() <= BF16_REL * scale, f"{what}: max |diff| {err.max():.3e} at row {worst}, scale {scale:.3f} (bound {BF16_REL} * scale)"
        assert err.mean() <= BF16_MEAN_REL * scale, f"{what}: mean |diff| {err.mean():.3e}, scale {scale:.3f}"


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# --------------------------------------------------------------------------
# traces
# --------------------------------------------------------------------------

class Trace:
    """Builds the JSON lines for bin/trace_run and remembers which rows of which
    step file hold which (request, position)."""

    def __init__(self) -> None:
        self.steps: List[dict] = []
        self.where: List[List[tuple]] = []      # per step: (request, position) per wanted row
        self.fed: Dict[str, int] = {}

    def step(self, entries: Sequence[tuple], end: Sequence[str] = ()) -> None:
        """entries: (request id, tokens, want-all flag or list of places)."""
        es, rows = [], []
        for rid, tokens, want in entries:
            tokens = list(tokens)
            if want is True:
                want = list(range(len(tokens)))
            elif want is False:
                want = []
            base = self.fed.get(rid, 0)
            es.append({"id": rid, "tokens": tokens, "want": list(want)})
            rows.extend((rid, base + w) for w in want)
            self.fed[rid] = base + len(tokens)
        self.steps.append({"step": len(self.steps), "entries": es, "end": list(end)})
        self.where.append(rows)
        for rid in end:
            self.fed.pop(rid, None)

    def lines(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def run_trace(model_dir, dtype: str, trace: Trace, out_dir, max_tokens: int, vocab: int, extra=()) -> Dict[str, Dict[int, torch.Tensor]]:
    """Run bin/trace_run as a user would and collect logits per request and position."""
    out_dir = Path(out_dir)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra]
    r = subprocess.run(cmd, input=trace.lines(), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == list(range(len(trace.steps))), "trace_run did not report every step"
    res: Dict[str, Dict[int, torch.Tensor]] = {}
    for i, rows in enumerate(trace.where):
        f = out_dir / f"{i}.f32"
        if not rows:
            assert not f.exists(), f"step {i} wanted nothing but wrote a file"
            continue
        data = np.fromfile(f, dtype="<f4")
        assert data.size == len(rows) * vocab, f"step {i}: {data.size} floats for {len(rows)} rows of {vocab}"
        lg = torch.from_numpy(data.reshape(len(rows), vocab).copy())
        for (rid, pos), row in zip(rows, lg):
            res.setdefault(rid, {})[pos] = row
    return res


def stack(rows: Dict[int, torch.Tensor]) -> torch.Tensor:
    return torch.stack([rows[p] for p in sorted(rows)])


def plain_logits(model_dir, tokens, dtype: str, schedule=None) -> torch.Tensor:
    cfg, w = P.read_model_folder(model_dir)
    if dtype != "float32":
        w = bf16_round(w)
    return P.plain_forward(cfg, w, tokens, schedule)
