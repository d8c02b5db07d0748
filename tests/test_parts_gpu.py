"""Each part of a layer alone on the GPU against the plain functions: norm,
position encoding, attention mixer, feed-forward, block, and the model's head.
Sizes differ from the tiny model configurations."""

from __future__ import annotations

import math

import pytest
import torch

import plain_qwen2 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return 2e-5 * max(scale, 1.0) if dtype == torch.float32 else 2.0 ** -6 * max(scale, 1e-3)


def check(got, ref, dtype, what):
    got, ref = got.float().cpu(), ref.float().cpu()
    scale = float(ref.abs().max())
    err = float((got - ref).abs().max())
    assert err <= tol(dtype, scale), f"{what}: max |diff| {err:.3e}, scale {scale:.3f}"


def bind_random(part, seed, dtype):
    """Random tensors for a part; returns them as float32 CPU tensors keyed by name (as the part holds them after rounding)."""
    from litinfer_b200.weights import random_tensors

    params = part.all_params()
    tensors = random_tensors(params, seed, dtype, DEV)
    plain = {k: v.float().cpu() for k, v in tensors.items()}
    part.bind_all(dict(tensors))
    return plain


def step_context(manager, requests, vocab=100):
    """(ctx, items) for a list of (RequestCache, number of new tokens)."""
    from litinfer_b200.engine import StepItem, context_from, pack_step

    items = [StepItem(rc, [1] * n, list(range(n))) for rc, n in requests]
    for rc, n in requests:
        manager.extend(rc, rc.length + n)
    buf, layout = pack_step(items, manager, vocab)
    return context_from(torch.from_numpy(buf).to(DEV), layout, manager.page_size)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from litinfer_b200.config import PartSpec
    from litinfer_b200.parts import NORMS

    H = 200
    norm = NORMS.build(PartSpec("rmsnorm", {"size": H, "eps": 3e-5}), "n.", dtype, DEV)
    w = bind_random(norm, 1, dtype)["n.weight"]
    x = torch.randn(6, H) * 2
    xd = x.to(DEV)
    check(norm.forward(xd), P.plain_rmsnorm(x, w, 3e-5), dtype, "forward")
    delta = torch.randn(6, H).to(dtype)
    y = norm.add_forward(xd, delta.to(DEV))
    check(xd, x + delta.float(), torch.float32, "residual after add_forward")
    check(y, P.plain_rmsnorm(x + delta.float(), w, 3e-5), dtype, "add_forward")
    rows = torch.tensor([5, 0, 2], dtype=torch.int32, device=DEV)
    check(norm.gather_forward(xd, rows), P.plain_rmsnorm((x + delta.float())[[5, 0, 2]], w, 3e-5), dtype, "gather_forward")


def test_rope_part_table_and_refusals():
    from litinfer_b200.config import PartSpec
    from litinfer_b200.parts import POSITIONS

    rope = POSITIONS.build(PartSpec("rope", {"theta": 50000.0, "rotary_dim": 48, "pairing": "half"}), "", torch.float32, DEV, head_dim=48)
    j = torch.arange(24, dtype=torch.float32)
    assert torch.allclose(rope.denominators.cpu(), torch.pow(torch.tensor(50000.0), 2 * j / 48))
    with pytest.raises(ValueError, match="pairing"):
        POSITIONS.build(PartSpec("rope", {"theta": 1e4, "rotary_dim": 16, "pairing": "interleaved"}), "", torch.float32, DEV, head_dim=16)
    with pytest.raises(ValueError, match="rotary_dim"):
        POSITIONS.build(PartSpec("rope", {"theta": 1e4, "rotary_dim": 32}), "", torch.float32, DEV, head_dim=16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_in_portions(dtype, window):
    """The mixer alone: a 45-token sequence in portions of 19, 2, 1, 23 beside another request, against
    projections, rotation and attention of the plain implementation over the whole sequence."""
    from litinfer_b200.cache import CacheManager
    from litinfer_b200.config import PartSpec
    from litinfer_b200.parts import MIXERS

    H, nh, nkv, dh = 72, 6, 2, 48
    spec = PartSpec("attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": dh, "qkv_bias": True, "out_bias": False,
                                  "scale": 1 / math.sqrt(dh), "window": window,
                                  "position": PartSpec("rope", {"theta": 1e4, "rotary_dim": dh, "pairing": "half"})})
    att = MIXERS.build(spec, "a.", dtype, DEV)
    w = bind_random(att, 2, dtype)
    manager = CacheManager([att.cache_requirement()], [None], 9, 16, 2, dtype, DEV)
    T = 45
    h = (torch.randn(T, H) * 0.5).to(dtype)
    other = (torch.randn(30, H) * 0.5).to(dtype)
    rc, rc2 = manager.admit(0), manager.admit(1)
    outs, pos = [], 0
    for n, n2 in ((19, 7), (2, 1), (1, 1), (23, 2)):
        ctx = step_context(manager, [(rc2, n2), (rc, n)])
        x = torch.cat([other[rc2.length:rc2.length + n2], h[pos:pos + n]]).to(DEV)
        y = att.forward(x, ctx, manager.entries[0])
        outs.append(y[n2:].cpu())
        manager.commit(rc, rc.length + n)
        manager.commit(rc2, rc2.length + n2)
        pos += n
    got = torch.cat(outs)
    hf = h.float()
    q = P.plain_linear(hf, w["a.q_proj.weight"], w["a.q_proj.bias"]).view(T, nh, dh)
    k = P.plain_linear(hf, w["a.k_proj.weight"], w["a.k_proj.bias"]).view(T, nkv, dh)
    v = P.plain_linear(hf, w["a.v_proj.weight"], w["a.v_proj.bias"]).view(T, nkv, dh)
    q, k = P.plain_rope(q, range(T), 1e4), P.plain_rope(k, range(T), 1e4)
    o = P.plain_attention(q, k, v, 1 / math.sqrt(dh), window)
    ref = P.plain_linear(o.reshape(T, nh * dh), w["a.o_proj.weight"])
    check(got, ref, dtype, f"attention part window={window}")
    if window is not None:
        assert rc.tables[0][0] == CacheManager.RELEASED          # pages behind the window were given back meanwhile


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    from litinfer_b200.config import PartSpec
    from litinfer_b200.parts import FEED_FORWARDS

    H, I = 72, 200
    ff = FEED_FORWARDS.build(PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}), "m.", dtype, DEV)
    w = bind_random(ff, 3, dtype)
    assert ff.gate_up.fused_activation == (dtype == torch.bfloat16)
    for T in (3, 70, 150):                     # the weight-streaming kernel, and the tensor-memory kernel with one and two row tiles
        h = (torch.randn(T, H)).to(dtype)
        got = ff.forward(h.to(DEV), None)
        ref = P.plain_mlp(h.float(), {"mlp." + k[2:]: v for k, v in w.items()}, "")
        check(got, ref, dtype, f"feed-forward T={T}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_and_head(dtype, model_dirs):
    """A whole block, then the model's tail (pending residual, final norm on wanted rows, lm_head)."""
    from conftest import TINY
    from litinfer_b200.cache import CacheManager
    from litinfer_b200.models import DecoderModel
    from helpers import bf16_round

    name = "C"
    cfg, w = P.read_model_folder(model_dirs[name])
    if dtype == torch.bfloat16:
        w = bf16_round(w)
    model = DecoderModel.from_dir(model_dirs[name], dtype, DEV)
    manager = CacheManager(model.cache_requirements(), [None, None], 8, 16, 1, dtype, DEV)
    rc = manager.admit(0)
    T = 37
    ctx = step_context(manager, [(rc, T)], cfg["vocab_size"])
    x = torch.randn(T, cfg["hidden_size"])
    xd = x.to(DEV).clone()
    xd, carry = model.blocks[1].forward(xd, ctx, manager.entries[1], None)
    pending = carry.delta
    ref, _ = P.plain_block(x, w, cfg, 1, torch.arange(T), None)
    check(xd + pending.float(), ref, dtype, "block")
    # the head on three wanted rows of a made-up residual stream
    from litinfer_b200 import kernels as K
    rows = torch.tensor([0, 36, 17], dtype=torch.int32, device=DEV)
    y = model.final_norm.gather_forward(x.to(DEV), rows)
    logits = torch.empty(3, cfg["vocab_size"], dtype=torch.float32, device=DEV)
    K.linear(y, model.lm_head, None, logits)
    ref = P.plain_linear(P.plain_rmsnorm(x[[0, 36, 17]], w["model.norm.weight"], cfg["rms_norm_eps"]), w["lm_head.weight"])
    check(logits, ref, dtype, "final norm and lm_head")
