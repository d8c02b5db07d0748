"""Shared fixtures: tiny configurations, model folders in temporary places,
and the switch that lets host-side logic run on the CPU against the plain
kernel references."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        # no GPU test takes more than seconds; one that sits for minutes ends the run (a thread ends the process: a
        # signal would not get through a call that waits for the device)
        try:
            import pytest_timeout  # noqa: F401
        except ImportError:
            return
        for item in items:
            if "gpu" in item.keywords and item.get_closest_marker("timeout") is None:
                item.add_marker(pytest.mark.timeout(300, method="thread"))
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny Qwen2 configurations that differ in every size and option: layers,
# width, heads and groups (2 per key head / 3 on a single key head), head size,
# feed-forward width, vocabulary (no power of two in B), rope base, norm eps,
# tied or own lm_head, position limit, and the window (none / 24 keys on the
# last two layers).
TINY_A = dict(
    architectures=["Qwen2ForCausalLM"], torch_dtype="float32", num_hidden_layers=2, hidden_size=64,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128,
    eos_token_id=None, use_sliding_window=False)
TINY_B = dict(
    architectures=["Qwen2ForCausalLM"], torch_dtype="float32", num_hidden_layers=3, hidden_size=96,
    num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=272, vocab_size=389,
    rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256,
    eos_token_id=None, use_sliding_window=True, sliding_window=24, max_window_layers=1)
# A third one for long sequences: more positions, a head size of 48 (a multiple of 16 that is no power of two).
TINY_C = dict(
    architectures=["Qwen2ForCausalLM"], torch_dtype="float32", num_hidden_layers=2, hidden_size=80,
    num_attention_heads=6, num_key_value_heads=2, head_dim=48, intermediate_size=176, vocab_size=300,
    rope_theta=50000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024,
    eos_token_id=None, use_sliding_window=False)

# The second configuration exactly as the benchmark description gives it (no window, round sizes): the variant above is
# the harder test, this one has nothing in it that LitInfer's own code does not pin.
TINY_B0 = dict(
    architectures=["Qwen2ForCausalLM"], torch_dtype="float32", num_hidden_layers=3, hidden_size=96,
    num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=384,
    rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256,
    eos_token_id=None, use_sliding_window=False)

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "B0": TINY_B0}


def _qwen2(layers, hidden, heads, kv_heads, head_dim, intermediate, vocab, theta=10000.0, eps=1e-6, tie=False, window=None,
           max_window_layers=0):
    cfg = dict(architectures=["Qwen2ForCausalLM"], torch_dtype="float32", num_hidden_layers=layers, hidden_size=hidden,
               num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=intermediate,
               vocab_size=vocab, rope_theta=theta, rms_norm_eps=eps, tie_word_embeddings=tie, max_position_embeddings=512,
               eos_token_id=None, use_sliding_window=window is not None)
    if window is not None:
        cfg.update(sliding_window=window, max_window_layers=max_window_layers)
    return cfg


# Still small, but with the head sizes of real checkpoints (the engine takes other kernels for them), and one whose widths
# are no multiple of 8.
MID = {
    "head128": _qwen2(2, 256, 2, 1, 128, 512, 1000),
    "head64_window": _qwen2(2, 512, 8, 2, 64, 1376, 3001, theta=1e6, eps=1e-5, window=100, max_window_layers=1),
    "odd_widths": _qwen2(1, 100, 5, 1, 20, 250, 333),
}


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations with random float32 weights."""
    from litinfer_b200.weights import write_model_folder

    out = {}
    for name, cfg in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny{name}")
        write_model_folder(d, dict(cfg), seed=1234 + sum(map(ord, name)), store_dtype="float32")
        out[name] = d
    return out


@pytest.fixture
def cpu_kernels(monkeypatch):
    """Replace every kernel by its plain reference, so that host-side logic runs on the CPU."""
    import kernel_refs
    from litinfer_b200 import kernels

    for name in kernel_refs.ALL:
        monkeypatch.setattr(kernels, name, getattr(kernel_refs, name))
    return kernels
