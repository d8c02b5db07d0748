"""The plain implementation (tests/plain_qwen2.py), the oracle of every other
test, checked against LitInfer itself once: tests/golden/litinfer_tiny.npz holds
what LitInfer's own code computed on the CPU for two tiny random models (made
by tests/golden/make_golden.py, which compiles LitInfer unmodified)."""

from __future__ import annotations

import importlib.util
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as P

GOLDEN = Path(__file__).resolve().parent / "golden"


def _golden():
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod, np.load(GOLDEN / "litinfer_tiny.npz")


def _weights(mod, cfg):
    return {k: torch.from_numpy(v) for k, v in mod.make_weights(cfg).items()}


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_logits_equal_litinfers_ops(name):
    """A 33-token and a 9-token sequence, fed to LitInfer in portions, mixed, with scrambled
    pages; the plain model runs each sequence whole."""
    mod, gold = _golden()
    cfg = mod.CONFIGS[name]
    w = _weights(mod, cfg)
    for i, seq in enumerate(mod.logit_sequences(cfg)):
        mine = P.plain_forward(cfg, w, seq.tolist())
        ref = torch.from_numpy(gold[f"{name}.logits{i}"])
        assert mine.shape == ref.shape
        # two float32 implementations with different summation orders
        assert (mine - ref).abs().max() < 5e-6, f"config {name} sequence {i}: {(mine - ref).abs().max():.3e}"


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_greedy_tokens_equal_litinfers(name):
    mod, gold = _golden()
    cfg = mod.CONFIGS[name]
    w = _weights(mod, cfg)
    assert np.array_equal(gold[f"{name}.generate"], gold[f"{name}.engine"]), "LitInfer's two paths disagree with each other"
    for prompt, ref in zip(mod.make_prompts(cfg), gold[f"{name}.generate"]):
        mine, margin = P.plain_greedy(cfg, w, prompt, cfg["new_tokens"])
        assert margin > 1e-4, "a near-tie would make the comparison meaningless"
        assert mine == ref.tolist()


# ---- the parts on their own: properties that do not need a second implementation ----

def test_rmsnorm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0], [0.0, 0.0]])
    y = P.plain_rmsnorm(x, torch.tensor([2.0, 0.5]), 1e-6)
    r = 1 / math.sqrt(12.5 + 1e-6)
    assert torch.allclose(y[0], torch.tensor([6.0 * r, 2.0 * r]))
    assert not y[1].any()
    g, u = torch.tensor([0.0, 2.0, -2.0]), torch.tensor([3.0, 1.0, 1.0])
    assert torch.allclose(P.plain_swiglu(g, u), torch.tensor([0.0, 2 / (1 + math.exp(-2)), -2 / (1 + math.exp(2))]))


def test_rope_pairs_halves_and_keeps_position_zero():
    x = torch.randn(3, 2, 8)
    y = P.plain_rope(x, [0, 1, 5], 10000.0)
    assert torch.equal(y[0], x[0])                                   # angle 0
    a, b = x[1, 0, 0], x[1, 0, 4]                                    # pair (j, j + dh/2), j = 0: angle = pos
    assert torch.allclose(y[1, 0, 0], a * math.cos(1) - b * math.sin(1), atol=1e-6)
    assert torch.allclose(y[1, 0, 4], b * math.cos(1) + a * math.sin(1), atol=1e-6)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_attention_is_causal_grouped_and_windowed():
    T, nh, nkv, dh = 9, 4, 2, 8
    q, k, v = torch.randn(T, nh, dh), torch.randn(T, nkv, dh), torch.randn(T, nkv, dh)
    o = P.plain_attention(q, k, v, 0.3)
    assert torch.allclose(o[0, :2], v[0, 0].expand(2, dh)) and torch.allclose(o[0, 2:], v[0, 1].expand(2, dh))   # one key; heads 0,1 -> kv 0
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 7.0, -3.0
    assert torch.equal(P.plain_attention(q, k2, v2, 0.3)[:5], o[:5])       # later keys do not reach earlier queries
    w = P.plain_attention(q, k, v, 0.3, window=3)
    assert torch.equal(w[:3], o[:3]) and not torch.allclose(w[5], o[5])
    k3, v3 = k.clone(), v.clone()
    k3[:4], v3[:4] = 5.0, 9.0
    assert torch.equal(P.plain_attention(q, k3, v3, 0.3, window=3)[6:], w[6:])   # keys behind the window do not matter


def test_sampling_candidates_follow_litinfers_order_of_filters():
    lg = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0])
    ids, pr = P.plain_candidates(lg, 1.0, 3, 1.0)
    assert ids.tolist() == [0, 1, 2] and abs(float(pr.sum()) - 1) < 1e-6
    ids, pr = P.plain_candidates(lg, 1.0, 0, 0.6)                  # softmax: .53 .20 .12 ...: the prefix reaching 0.6 is {0, 1}
    assert ids.tolist() == [0, 1]
    ids, _ = P.plain_candidates(lg, 0.25, 0, 0.6)                  # a low temperature sharpens: token 0 alone reaches 0.6
    assert ids.tolist() == [0]
    assert P.plain_argmax(torch.tensor([1.0, 3.0, 3.0])) == 1      # the first maximum


def test_schedule_and_window_defaults_fall_back_to_litinfer(tmp_path):
    from conftest import TINY
    from litinfer_b200.weights import write_model_folder

    d = write_model_folder(tmp_path / "m", dict(TINY["A"]), seed=5)
    cfg, w = P.read_model_folder(d)
    toks = list(range(20))
    base = P.plain_forward(cfg, w, toks)
    assert torch.equal(base, P.plain_forward(cfg, w, toks, [(0, None), (1, None)]))
    assert P.layer_windows(cfg) == [None, None]
    assert P.layer_windows(dict(cfg, use_sliding_window=True, sliding_window=7, max_window_layers=1)) == [None, 7]
    other = P.plain_forward(cfg, w, toks, [(0, None), (1, 0)])       # layer 1 reads layer 0's keys and values
    assert not torch.allclose(other, base)
