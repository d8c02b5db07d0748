"""The decode step as one persistent kernel (csrc/decode_step.cu) against the same step run part by part and against
the plain model: batches of 1 to 16 sequences at contexts from a few keys to beyond 2,048, with and without a window,
launched plainly and from captured graphs, at small sizes and at the layer sizes of the 1.5B shape."""

from __future__ import annotations

import pytest
import torch

from conftest import MID
from helpers import check_logits, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

REAL = dict(
    architectures=["Qwen2ForCausalLM"], torch_dtype="float32", num_hidden_layers=2, hidden_size=1536,
    num_attention_heads=12, num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=32000,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096,
    eos_token_id=None, use_sliding_window=False)
# heads of 64, more layers than two, a window on the upper ones, widths that make ragged chunks (hidden 1600 = 1024 + 576)
WIDE64 = dict(
    architectures=["Qwen2ForCausalLM"], torch_dtype="float32", num_hidden_layers=3, hidden_size=1600,
    num_attention_heads=10, num_key_value_heads=5, head_dim=64, intermediate_size=2072, vocab_size=5003,
    rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=1024,
    eos_token_id=None, use_sliding_window=True, sliding_window=300, max_window_layers=1)

CONFIGS = {"head128": MID["head128"], "head64_window": MID["head64_window"], "wide64": WIDE64, "real": REAL}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from litinfer_b200.weights import write_model_folder

    out = {}
    for name, cfg in CONFIGS.items():
        d = tmp_path_factory.mktemp(f"fused_{name}")
        write_model_folder(d, dict(cfg), seed=700 + len(name), store_dtype="float32")
        out[name] = d
    return out


def _decode(folder, cfg, lens, steps, use_graphs, fused):
    """Prompts of the given lengths in one step each (part by part: they are no decode steps), then ``steps`` decode steps of
    all of them together; returns the logits of every decode step, [steps, sequences, vocab]."""
    from litinfer_b200.engine.replay import Replayer
    from litinfer_b200.models import DecoderModel

    from litinfer_b200.models.fused_decode import FusedDecode

    model = DecoderModel.from_dir(folder, "bfloat16", torch.device("cuda:0"))
    model._fused = FusedDecode(model, enable=fused)        # off: every step goes part by part (the default)
    assert (model._fused.layers is not None) == fused
    need = sum(-(-(n + steps) // 64) * 64 for n in lens)
    rp = Replayer(model, need, max_live=len(lens), use_graphs=use_graphs)
    vocab = cfg["vocab_size"]
    toks = [random_tokens(n + steps, vocab, 40 + i) for i, n in enumerate(lens)]
    for i, n in enumerate(lens):
        rp.step(dict(step=i, entries=[dict(id=str(i), tokens=toks[i][:n], want=[])]))
    outs = []
    for j in range(steps):
        rec = dict(step=len(lens) + j, entries=[dict(id=str(i), tokens=[toks[i][n + j]], want=[0]) for i, n in enumerate(lens)])
        outs.append(rp.step(rec).clone().cpu())
    launches = model._fused.launches if model._fused is not None else 0
    return torch.stack(outs), toks, launches


@pytest.mark.parametrize("name,lens", [
    ("head128", [5]), ("head128", [300, 17, 64]), ("head128", [33, 255, 256, 257, 1, 16, 100, 490]),
    ("head128", [20 + 7 * i for i in range(16)]), ("head64_window", [5, 130, 400]), ("head64_window", [30 * (i + 1) for i in range(11)]),
    ("wide64", [700, 3, 299, 300, 301]), ("wide64", [40 + 50 * i for i in range(16)]),
])
def test_fused_decode_step_matches_parts_and_plain(name, lens, folders):
    cfg = CONFIGS[name]
    steps = 3
    fused, toks, launches = _decode(folders[name], cfg, lens, steps, use_graphs=False, fused=True)
    parts, _, none = _decode(folders[name], cfg, lens, steps, use_graphs=False, fused=False)
    assert launches >= steps and none == 0                 # a prompt of one token is a step of single tokens too
    for i, n in enumerate(lens):
        ref = plain_logits(folders[name], toks[i], "bfloat16")[n:n + steps]
        check_logits(fused[:, i], ref, "bfloat16", f"{name} lens={lens}: fused step, sequence {i}")
        check_logits(parts[:, i], ref, "bfloat16", f"{name} lens={lens}: part by part, sequence {i}")
    scale = float(parts.abs().max())
    assert (fused - parts).abs().max() <= 0.02 * scale, f"{name} lens={lens}: fused and part-by-part steps differ by {(fused - parts).abs().max()} (scale {scale})"


@pytest.mark.parametrize("name,lens", [("head128", [300, 170, 100]), ("wide64", [90 + 50 * i for i in range(12)])])
def test_fused_decode_step_from_a_captured_graph(name, lens, folders):
    # (prompts of more than 64 tokens: shorter ones run as single tokens when graphs are on, which rounds their keys differently)
    cfg = CONFIGS[name]
    plainly, _, _ = _decode(folders[name], cfg, lens, 4, use_graphs=False, fused=True)
    captured, _, launches = _decode(folders[name], cfg, lens, 4, use_graphs=True, fused=True)
    assert launches >= 1                                   # warm-up and capture run it; replays do not go through Python
    assert torch.equal(plainly, captured), f"captured and plainly launched fused steps differ by {(plainly - captured).abs().max()}"


def test_fused_decode_step_a_sequence_does_not_depend_on_the_others(folders):
    """One sequence alone, among seven others (the same tile of tokens) and among fifteen (the next tile): bit for bit the
    same within a tile, within rounding across tiles."""
    cfg = CONFIGS["head128"]
    alone, _, _ = _decode(folders["head128"], cfg, [120], 3, False, True)
    among8, _, _ = _decode(folders["head128"], cfg, [120] + [50 + 9 * i for i in range(7)], 3, False, True)
    among16, _, _ = _decode(folders["head128"], cfg, [120] + [50 + 9 * i for i in range(15)], 3, False, True)
    assert torch.equal(alone[:, 0], among8[:, 0])
    assert (alone[:, 0] - among16[:, 0]).abs().max() <= 0.02 * float(alone.abs().max())


@pytest.mark.parametrize("lens", [[2049], [2048, 300, 1111, 5, 2303, 64, 700, 2047]])
def test_fused_decode_step_at_real_layer_sizes(lens, folders):
    """The layer sizes of the 1.5B shape at the contexts the benchmark decodes at (nine splits of 256 keys and more)."""
    cfg = CONFIGS["real"]
    steps = 2
    fused, toks, launches = _decode(folders["real"], cfg, lens, steps, use_graphs=True, fused=True)
    assert launches >= 1
    for i, n in enumerate(lens):
        ref = plain_logits(folders["real"], toks[i], "bfloat16")[n:n + steps]
        check_logits(fused[:, i], ref, "bfloat16", f"real sizes lens={lens}: fused step, sequence {i}")
    from litinfer_b200 import kernels as K

    assert K.library().li_tcgen05_status() == 0
