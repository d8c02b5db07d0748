"""Plain, slow implementation of the Qwen2 dense decoder: the oracle of the tests.

Whole sequences, no cache, no batching, 32-bit floats on the CPU, one function
for each part.  It shares no code with the package (it has its own reader of
model folders) and is written from the formulas of the LitInfer sources; every
function cites the file and lines it restates (paths are relative to the
LitInfer project root).

Two things go beyond what LitInfer runs, both written so that they fall back
to LitInfer's behaviour when unused:

* a sliding window (``window`` keys, the query's own included) on chosen
  layers, which LitInfer never reads from config.json
  (python/llaisys/models/qwen2.py:243-299 has no such key);
* a layer *schedule*: the order in which blocks run, where a block may be
  named twice and an entry may read the keys and values that an earlier entry
  produced instead of making its own.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_ST_DTYPES = {
    "F32": (np.float32, 4),
    "F64": (np.float64, 8),
    "F16": (np.float16, 2),
    "BF16": (np.uint16, 2),
    "I32": (np.int32, 4),
    "I64": (np.int64, 8),
}


# --------------------------------------------------------------------------
# model folder
# --------------------------------------------------------------------------

def read_model_folder(path):
    """config.json as a dict and every tensor of model.safetensors as float32.

    File format as read by python/llaisys/models/qwen2.py:112-129: 8 bytes of
    little-endian header length, a JSON header of name -> dtype, shape,
    data_offsets, then the raw data.
    """
    path = Path(path)
    cfg = json.loads((path / "config.json").read_text())
    blob = (path / "model.safetensors").read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        np_dtype, _ = _ST_DTYPES[info["dtype"]]
        lo, hi = info["data_offsets"]
        arr = np.frombuffer(blob[base + lo:base + hi], dtype=np_dtype).copy()
        if info["dtype"] == "BF16":
            # widen: bfloat16 is the upper half of a float32
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        t = torch.from_numpy(arr.reshape(info["shape"]))
        tensors[name] = t.float() if t.is_floating_point() else t
    return cfg, tensors


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def plain_embedding(table, ids):
    """x[t, :] = E[id_t, :], ids checked against the table (src/ops/embedding/op.cpp:32-40)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= table.shape[0]):
        raise IndexError("token id out of range")
    return table[ids].clone()


def plain_rmsnorm(x, weight, eps):
    """y_j = w_j * x_j / sqrt(mean(x^2) + eps), per row (src/ops/rms_norm/op.cpp:13-24)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    r = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return (weight * x) * r


def plain_linear(x, weight, bias=None):
    """out = x W^T (+ b), W stored [out, in] (src/ops/linear/cpu/linear_cpu.cpp:45-60)."""
    out = x @ weight.t()
    if bias is not None:
        out = out + bias
    return out


def plain_rope(x, positions, theta):
    """Rotate-half position encoding on [T, heads, dh] (src/ops/rope/op.cpp:13-20, 33-39).

    phi = pos / theta^(2j/dh); (a, b) = (x[j], x[j + dh/2]);
    x'[j] = a cos - b sin; x'[j + dh/2] = b cos + a sin.
    """
    dh = x.shape[-1]
    half = dh // 2
    j = torch.arange(half, dtype=torch.float32)
    denom = torch.pow(torch.tensor(float(theta), dtype=torch.float32), (2.0 * j) / dh)
    phi = torch.as_tensor(positions, dtype=torch.float32)[:, None] / denom[None, :]
    cos, sin = torch.cos(phi)[:, None, :], torch.sin(phi)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def plain_attention(q, k, v, scale, window=None):
    """Causal grouped-query attention over a whole sequence.

    q [T, nh, dh], k and v [T, nkv, dh]; query head h reads key head
    h // (nh / nkv); the query at position p sees keys 0..p
    (src/ops/paged_attention/op.cpp:194-234), and with a window only the
    last ``window`` of them (p - t < window).  Softmax in the plain two-pass
    form; LitInfer's online recurrence gives the same value.
    """
    T, nh, dh = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    out = torch.empty_like(q)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= (pos[:, None] - pos[None, :]) < window
    for h in range(nh):
        s = (q[:, h] @ k[:, h // group].t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h] = p @ v[:, h // group]
    return out


def plain_swiglu(gate, up):
    """up * gate / (1 + exp(-gate)) (src/ops/swiglu/op.cpp:17-23)."""
    return up * (gate / (1.0 + torch.exp(-gate)))


def plain_mlp(h, w, prefix):
    """down(swiglu(gate(h), up(h))), no biases (src/llaisys/models/qwen2.cpp:744-759)."""
    gate = plain_linear(h, w[prefix + "mlp.gate_proj.weight"])
    up = plain_linear(h, w[prefix + "mlp.up_proj.weight"])
    return plain_linear(plain_swiglu(gate, up), w[prefix + "mlp.down_proj.weight"])


def plain_qkv(h, w, prefix, cfg):
    """q, k, v projections with optional biases (src/llaisys/models/qwen2.cpp:613-615)."""
    nh, nkv, dh = _heads(cfg)
    T = h.shape[0]
    p = prefix + "self_attn."
    q = plain_linear(h, w[p + "q_proj.weight"], w.get(p + "q_proj.bias")).view(T, nh, dh)
    k = plain_linear(h, w[p + "k_proj.weight"], w.get(p + "k_proj.bias")).view(T, nkv, dh)
    v = plain_linear(h, w[p + "v_proj.weight"], w.get(p + "v_proj.bias")).view(T, nkv, dh)
    return q, k, v


def _heads(cfg):
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    dh = cfg.get("head_dim") or cfg["hidden_size"] // nh
    return nh, nkv, dh


def layer_windows(cfg):
    """Window of each layer, None for full attention.

    With ``use_sliding_window`` the layers from ``max_window_layers`` on see
    ``sliding_window`` keys; the others, and every layer without it, see all.
    """
    L = cfg["num_hidden_layers"]
    if not cfg.get("use_sliding_window", False) or cfg.get("sliding_window") is None:
        return [None] * L
    first = cfg.get("max_window_layers", L)
    return [cfg["sliding_window"] if i >= first else None for i in range(L)]


def plain_block(x, w, cfg, layer, positions, window, shared_kv=None):
    """One pre-norm block: x += Attn(norm(x)); x += MLP(norm(x)) (src/llaisys/models/qwen2.cpp:272-316).

    Returns the new x and the (k, v) this entry used, so that a later entry of
    the schedule can read them.
    """
    nh, nkv, dh = _heads(cfg)
    eps = cfg.get("rms_norm_eps", 1e-6)
    theta = cfg.get("rope_theta", 10000.0)
    prefix = f"model.layers.{layer}."
    T = x.shape[0]
    h = plain_rmsnorm(x, w[prefix + "input_layernorm.weight"], eps)
    q, k, v = plain_qkv(h, w, prefix, cfg)
    q = plain_rope(q, positions, theta)
    if shared_kv is None:
        k = plain_rope(k, positions, theta)      # keys are cached after rotation (qwen2.cpp:626-673)
    else:
        k, v = shared_kv
    o = plain_attention(q, k, v, 1.0 / math.sqrt(dh), window)
    x = x + plain_linear(o.reshape(T, nh * dh), w[prefix + "self_attn.o_proj.weight"])
    h = plain_rmsnorm(x, w[prefix + "post_attention_layernorm.weight"], eps)
    x = x + plain_mlp(h, w, prefix)
    return x, (k, v)


def plain_forward(cfg, w, tokens, schedule=None):
    """Logits [T, V] of a whole sequence (src/llaisys/models/qwen2.cpp:261-361).

    ``schedule`` is a list of (layer, reads_entry) pairs: run block ``layer``;
    if ``reads_entry`` is not None, attend over the keys and values that
    schedule entry ``reads_entry`` produced.  Default: every layer once, in
    order, each with its own keys and values.
    """
    eps = cfg.get("rms_norm_eps", 1e-6)
    T = len(tokens)
    positions = torch.arange(T)
    windows = layer_windows(cfg)
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    x = plain_embedding(w["model.embed_tokens.weight"], tokens)
    produced = []
    for layer, reads in schedule:
        shared = produced[reads] if reads is not None else None
        x, kv = plain_block(x, w, cfg, layer, positions, windows[layer], shared)
        produced.append(kv)
    x = plain_rmsnorm(x, w["model.norm.weight"], eps)
    head = w.get("lm_head.weight")
    if head is None:                                  # tied (python/llaisys/models/qwen2.py:196-199)
        head = w["model.embed_tokens.weight"]
    return plain_linear(x, head)


# --------------------------------------------------------------------------
# sampling and generation
# --------------------------------------------------------------------------

def plain_argmax(logits):
    """Index of the first maximum (src/ops/argmax/op.cpp:28-33)."""
    logits = torch.as_tensor(logits, dtype=torch.float32)
    best, idx = float("-inf"), 0
    for i, v in enumerate(logits.tolist()):
        if v > best:
            best, idx = v, i
    return idx


def plain_candidates(logits, temperature, top_k, top_p):
    """The token ids LitInfer's sampler keeps, and their probabilities.

    logits / temperature; descending order; the first top_k if 0 < k < V;
    softmax over those; the shortest prefix whose cumulative probability
    reaches top_p if 0 < p < 1; softmax again over what is left
    (src/llaisys/models/qwen2.cpp:890-920).
    """
    z = torch.as_tensor(logits, dtype=torch.float32) / temperature
    order = torch.argsort(z, descending=True, stable=True)
    V = z.numel()
    if 0 < top_k < V:
        order = order[:top_k]
    if 0.0 < top_p < 1.0:
        pr = torch.softmax(z[order], dim=0)
        cum = torch.cumsum(pr, dim=0)
        reach = torch.nonzero(cum >= top_p)
        if reach.numel():
            order = order[: int(reach[0]) + 1]
    pr = torch.softmax(z[order], dim=0)
    return order, pr


def plain_greedy_margins(cfg, w, prompt, n_new, schedule=None):
    """n_new greedy tokens by recomputing the whole sequence each time, and for each of them the margin
    between the best and the second logit."""
    toks = list(prompt)
    out, margins = [], []
    for _ in range(n_new):
        lg = plain_forward(cfg, w, toks, schedule)[-1]
        top2 = torch.topk(lg, 2).values
        margins.append(float(top2[0] - top2[1]))
        t = plain_argmax(lg)
        out.append(t)
        toks.append(t)
    return out, margins


def plain_greedy(cfg, w, prompt, n_new, schedule=None):
    """The tokens of :func:`plain_greedy_margins` and the smallest margin that was seen."""
    out, margins = plain_greedy_margins(cfg, w, prompt, n_new, schedule)
    return out, min(margins, default=float("inf"))


def same_up_to_a_near_tie(got, ref, margins, small=0.05) -> bool:
    """Whether greedy tokens ``got`` of an implementation that rounds differently (bfloat16) are acceptable against
    the plain ``ref``: equal, or equal up to a position at which the plain model's own margin is below ``small``, where
    rounding may legitimately pick the runner-up (after that the two sequences are different texts and nothing can
    be said).  A difference at a position with a clear margin is a fault."""
    if len(got) != len(ref):
        return False
    for i, (a, b) in enumerate(zip(got, ref)):
        if a != b:
            return margins[i] < small
    return True
