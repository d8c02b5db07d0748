#!/usr/bin/env python3
"""Makes tests/golden/litinfer_tiny.npz: what LitInfer itself computes for two
tiny random Qwen2 models, so that the plain implementation of the tests
(tests/plain_qwen2.py) can be compared with it.

    python tests/golden/make_golden.py /path/to/LitInfer

LitInfer is compiled here on the CPU, unmodified, with g++ (its own build
needs xmake): every .cpp/.cc under src/ into one libllaisys.so, its Python
package copied beside it.  Its safetensors loader cannot read float32 files
(a view outlives the mapping, python/llaisys/models/qwen2.py:117-129), so the
weights are handed over through its C interface (tensorCreate / tensorLoad)
instead.  Recorded per configuration:

* greedy tokens of ``Qwen2.generate`` (single-sequence path) and of the
  ``engine_*`` path with all prompts submitted together;
* logits of a mixed, chunked schedule computed by composing LitInfer's exported
  ops in the order of src/llaisys/models/qwen2.cpp:967-1047 (the model
  interface returns token ids only), with scrambled page tables.

The weights are not stored: ``make_weights`` below draws them from a seed and
the test calls it again.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

CONFIGS = {
    "A": dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=128, prompts=(5, 11, 17), new_tokens=8),
    "B": dict(num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
              intermediate_size=256, vocab_size=384, rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=256, prompts=(1, 9, 33, 40), new_tokens=12),
}
SEED = 1234


def make_weights(cfg, seed=SEED):
    """Matrices and biases N(0, 0.02), norm weights 1 + N(0, 0.1), float32, by tensor name."""
    rng = np.random.default_rng(seed)
    H, nh, nkv, dh, I, V, L = (cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                                 "intermediate_size", "vocab_size", "num_hidden_layers"))
    n = lambda *s: (rng.standard_normal(s) * 0.02).astype(np.float32)
    g = lambda *s: (1 + rng.standard_normal(s) * 0.1).astype(np.float32)
    W = {"model.embed_tokens.weight": n(V, H)}
    for l in range(L):
        p = f"model.layers.{l}."
        W[p + "input_layernorm.weight"] = g(H)
        for nm, rows in (("q", nh * dh), ("k", nkv * dh), ("v", nkv * dh)):
            W[p + f"self_attn.{nm}_proj.weight"] = n(rows, H)
            W[p + f"self_attn.{nm}_proj.bias"] = n(rows)
        W[p + "self_attn.o_proj.weight"] = n(H, nh * dh)
        W[p + "post_attention_layernorm.weight"] = g(H)
        W[p + "mlp.gate_proj.weight"] = n(I, H)
        W[p + "mlp.up_proj.weight"] = n(I, H)
        W[p + "mlp.down_proj.weight"] = n(H, I)
    W["model.norm.weight"] = g(H)
    if not cfg["tie_word_embeddings"]:
        W["lm_head.weight"] = n(V, H)
    return W


def make_prompts(cfg):
    rng = np.random.default_rng(7)
    return [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in cfg["prompts"]]


def build_reference(src: Path, out: Path) -> Path:
    """Compile LitInfer's sources as they are; returns the folder to put on sys.path."""
    obj = out / "obj"
    obj.mkdir(parents=True)
    files = sorted(list((src / "src").rglob("*.cpp")) + list((src / "src").rglob("*.cc")))
    objs = []
    for i, f in enumerate(files):
        extra = []
        # the AVX files need the flags of xmake/cpu.lua:43-58; `-include immintrin.h` first, because
        # include/llaisys.h:13 defines __C, which GCC's intrinsics headers use as a parameter name
        if f.name == "linear_cpu_avx.cpp":
            extra = ["-include", "immintrin.h", "-mavx2", "-mfma", "-mf16c", "-DLLAISYS_COMPILE_AVX_LINEAR"]
        elif f.name == "quantize_cpu_avx.cpp":
            extra = ["-include", "immintrin.h", "-mavx2", "-mfma", "-mf16c", "-DLLAISYS_COMPILE_AVX_QUANT"]
        o = obj / f"{i}.o"
        subprocess.run(["g++", "-std=c++17", "-O2", "-fPIC", "-fopenmp", "-Wno-unknown-pragmas", f"-I{src / 'include'}", f"-I{src / 'src'}",
                        *extra, "-c", str(f), "-o", str(o)], check=True)
        objs.append(str(o))
    subprocess.run(["g++", "-shared", "-fopenmp", "-o", str(out / "libllaisys.so"), *objs], check=True)
    pkg = out / "pkg"
    shutil.copytree(src / "python" / "llaisys", pkg / "llaisys")
    for p in (pkg / "llaisys").rglob("*"):
        os.chmod(p, 0o755 if p.is_dir() else 0o644)
    shutil.copy(out / "libllaisys.so", pkg / "llaisys" / "libllaisys" / "libllaisys.so")
    return pkg


def load_direct(W, cfg):
    """A reference model with its weights set through the C interface."""
    from llaisys.libllaisys import LIB_LLAISYS as LIB, DataType, LlaisysQwen2Meta, llaisysDataType_t
    from llaisys.models.qwen2 import Qwen2

    m = Qwen2.__new__(Qwen2)
    m.meta = LlaisysQwen2Meta(llaisysDataType_t(DataType.F32), cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"],
                              cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"], cfg["max_position_embeddings"],
                              cfg["vocab_size"], cfg["rms_norm_eps"], cfg["rope_theta"], -1)
    ids = (ctypes.c_int * 1)(0)
    m.model = LIB.llaisysQwen2ModelCreate(ctypes.byref(m.meta), 0, ids, 1)
    w = LIB.llaisysQwen2ModelWeights(m.model).contents

    def T(a):
        a = np.ascontiguousarray(a)
        sh = (ctypes.c_size_t * a.ndim)(*a.shape)
        t = LIB.tensorCreate(sh, a.ndim, int(DataType.F32), 0, 0)
        LIB.tensorLoad(t, ctypes.c_void_p(a.ctypes.data))
        return t

    w.in_embed = T(W["model.embed_tokens.weight"])
    w.out_norm_w = T(W["model.norm.weight"])
    w.out_embed = w.in_embed if cfg["tie_word_embeddings"] else T(W["lm_head.weight"])
    names = dict(attn_norm_w="input_layernorm.weight", attn_q_w="self_attn.q_proj.weight", attn_q_b="self_attn.q_proj.bias",
                 attn_k_w="self_attn.k_proj.weight", attn_k_b="self_attn.k_proj.bias", attn_v_w="self_attn.v_proj.weight",
                 attn_v_b="self_attn.v_proj.bias", attn_o_w="self_attn.o_proj.weight", mlp_norm_w="post_attention_layernorm.weight",
                 mlp_gate_w="mlp.gate_proj.weight", mlp_up_w="mlp.up_proj.weight", mlp_down_w="mlp.down_proj.weight")
    for l in range(cfg["num_hidden_layers"]):
        for field, n in names.items():
            getattr(w, field)[l] = T(W[f"model.layers.{l}.{n}"])
    return m


def ops_logits(W, cfg, seqs, plan, tables):
    """Logits of every fed token by composing the reference's ops, batched and paged
    as its engine does (src/llaisys/models/qwen2.cpp:967-1047)."""
    from llaisys import DataType, Ops, Tensor

    H, nh, nkv, dh, I, V, NL = (cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                                  "intermediate_size", "vocab_size", "num_hidden_layers"))

    def L(a, dt=DataType.F32):
        a = np.ascontiguousarray(a)
        t = Tensor(shape=list(a.shape), dtype=dt)
        t.load(a.ctypes.data)
        t._keep = a
        return t

    def N(t):
        b = np.empty(t.shape(), np.float32)
        ctypes.memmove(b.ctypes.data, t.data_ptr(), b.nbytes)
        return b

    nblk = 1 + max(max(t) for t in tables)
    kp = [np.zeros((nblk, 16, nkv, dh), np.float32) for _ in range(NL)]
    vp = [np.zeros((nblk, 16, nkv, dh), np.float32) for _ in range(NL)]
    done = [0] * len(seqs)
    got = [[] for _ in seqs]
    for step in plan:
        toks = np.concatenate([seqs[s][done[s]:done[s] + n] for s, n in step]).astype(np.int64)
        pos = np.concatenate([np.arange(done[s], done[s] + n) for s, n in step]).astype(np.int64)
        T = len(toks)
        x = Tensor(shape=[T, H])
        Ops.embedding(x, L(toks, DataType.I64), L(W["model.embed_tokens.weight"]))
        maxb = max(len(tables[s]) for s, _ in step)
        bt = np.zeros((len(step), maxb), np.int32)
        for i, (s, _) in enumerate(step):
            bt[i, :len(tables[s])] = tables[s]
        cl = np.array([done[s] + n for s, n in step], np.int32)
        ql = np.array([n for _, n in step], np.int32)
        for l in range(NL):
            p = f"model.layers.{l}."
            h = Tensor(shape=[T, H])
            Ops.rms_norm(h, x, L(W[p + "input_layernorm.weight"]), cfg["rms_norm_eps"])
            q, k, v = Tensor(shape=[T, nh, dh]), Tensor(shape=[T, nkv, dh]), Tensor(shape=[T, nkv, dh])
            Ops.linear(q, h, L(W[p + "self_attn.q_proj.weight"]), L(W[p + "self_attn.q_proj.bias"]))
            Ops.linear(k, h, L(W[p + "self_attn.k_proj.weight"]), L(W[p + "self_attn.k_proj.bias"]))
            Ops.linear(v, h, L(W[p + "self_attn.v_proj.weight"]), L(W[p + "self_attn.v_proj.bias"]))
            qr, kr, pt = Tensor(shape=[T, nh, dh]), Tensor(shape=[T, nkv, dh]), L(pos, DataType.I64)
            Ops.rope(qr, q, pt, cfg["rope_theta"])
            Ops.rope(kr, k, pt, cfg["rope_theta"])
            kn, vn, g = N(kr), N(v), 0
            for s, n in step:
                for i in range(n):
                    t = done[s] + i
                    kp[l][tables[s][t // 16], t % 16] = kn[g]
                    vp[l][tables[s][t // 16], t % 16] = vn[g]
                    g += 1
            a = Tensor(shape=[T, nh, dh])
            Ops.batched_paged_self_attention(a, qr, L(kp[l]), L(vp[l]), L(bt, DataType.I32), L(cl, DataType.I32), L(ql, DataType.I32),
                                             1.0 / np.sqrt(dh))
            o = Tensor(shape=[T, H])
            Ops.linear(o, a.view(T, H), L(W[p + "self_attn.o_proj.weight"]), None)
            x1 = Tensor(shape=[T, H])
            Ops.add(x1, x, o)
            h2 = Tensor(shape=[T, H])
            Ops.rms_norm(h2, x1, L(W[p + "post_attention_layernorm.weight"]), cfg["rms_norm_eps"])
            gt, up = Tensor(shape=[T, I]), Tensor(shape=[T, I])
            Ops.linear(gt, h2, L(W[p + "mlp.gate_proj.weight"]), None)
            Ops.linear(up, h2, L(W[p + "mlp.up_proj.weight"]), None)
            sw = Tensor(shape=[T, I])
            Ops.swiglu(sw, gt, up)
            dn = Tensor(shape=[T, H])
            Ops.linear(dn, sw, L(W[p + "mlp.down_proj.weight"]), None)
            x = Tensor(shape=[T, H])
            Ops.add(x, x1, dn)
        xf = Tensor(shape=[T, H])
        Ops.rms_norm(xf, x, L(W["model.norm.weight"]), cfg["rms_norm_eps"])
        lg = Tensor(shape=[T, V])
        head = W["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else W["lm_head.weight"]
        Ops.linear(lg, xf, L(head), None)
        lg, g = N(lg), 0
        for s, n in step:
            got[s].append(lg[g:g + n])
            g += n
            done[s] += n
    return [np.concatenate(x) for x in got]


# the mixed, chunked schedule of the logits: (sequence, tokens) per step, and each sequence's (scrambled) pages
LOGIT_LENGTHS = (33, 9)
LOGIT_PLAN = [[(0, 16)], [(0, 15), (1, 7)], [(0, 2), (1, 1)], [(1, 1)]]
LOGIT_TABLES = [[5, 0, 7], [3]]


def logit_sequences(cfg):
    rng = np.random.default_rng(3)
    return [rng.integers(0, cfg["vocab_size"], size=n) for n in LOGIT_LENGTHS]


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/LitInfer")
    src = Path(sys.argv[1])
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        pkg = build_reference(src, Path(tmp))
        sys.path.insert(0, str(pkg))
        for name, cfg in CONFIGS.items():
            W = make_weights(cfg)
            m = load_direct(W, cfg)
            prompts = make_prompts(cfg)
            n = cfg["new_tokens"]
            out[f"{name}.generate"] = np.array([m.generate(p, max_new_tokens=n) for p in prompts], dtype=np.int64)
            m.engine_start()
            ids = [m.engine_add_request(p, n) for p in prompts]
            while m.engine_has_unfinished():
                m.engine_step(1, 1.0, 0.0)
            out[f"{name}.engine"] = np.array([m.engine_get_output(i) for i in ids], dtype=np.int64)
            m.engine_stop()
            for i, lg in enumerate(ops_logits(W, cfg, logit_sequences(cfg), LOGIT_PLAN, LOGIT_TABLES)):
                out[f"{name}.logits{i}"] = lg.astype(np.float32)
    dst = Path(__file__).resolve().parent / "litinfer_tiny.npz"
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
