"""Plain references of the package's kernels, one per function of
``litinfer_b200.kernels``, with the same signatures, in float32 torch on
whatever device the tensors are on.

Two uses: the GPU tests compare each kernel alone with its reference here;
the CPU tests patch these in place of the kernels, so that the cache manager,
the step function and the scheduler can be checked against the plain model
without a GPU.  They are test code: nothing in the package imports them.
"""

from __future__ import annotations

import math

import numpy as np
import torch


def _store(out, value):
    out.copy_(value.to(out.dtype))


def embedding(table, ids, out32):
    _store(out32, table[ids.long()].float())


def _rms(x, weight, eps):
    x = x.float()
    r = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return (weight * x) * r


def rmsnorm(x32, weight, eps, out):
    _store(out, _rms(x32, weight, eps))


def add_rmsnorm(x32, delta, weight, eps, out):
    x32.add_(delta.float())
    _store(out, _rms(x32, weight, eps))


def gather_rmsnorm(x32, rows, weight, eps, out):
    _store(out, _rms(x32[rows.long()], weight, eps))


def residual_add(x32, delta):
    x32.add_(delta.float())


def linear(a, weight, bias, out, epilogue=None, row_scale=None):
    y = a.float() @ weight.float().t()
    if row_scale is not None:
        y = y * _factor(row_scale)
    if bias is not None:
        y = y + bias
    if epilogue == "swiglu":
        # columns come as 8 gate, 8 up, 8 gate, 8 up, ...
        M, N = y.shape
        y = y.view(M, N // 16, 2, 8)
        g, u = y[:, :, 0, :], y[:, :, 1, :]
        y = (u * (g / (1.0 + torch.exp(-g)))).reshape(M, N // 2)
    _store(out, y)


def _factor(row_scale):
    ssq, width, eps = row_scale
    return (1.0 / torch.sqrt(ssq.sum(1) / width + eps)).unsqueeze(1)


def linear_scaled_accepts(a, weight, out):
    return True


def linear_add_scaled_parts(a, weight, x32, hprime):
    return 3


def linear_add_scaled(a, weight, bias, x32, norm_weight, hprime, ssq):
    y = a.float() @ weight.float().t()
    if bias is not None:
        y = y + bias
    x32.add_(y)
    _store(hprime, norm_weight * x32)
    # any split of the columns into parts gives the same sums; here: everything in part 0
    ssq.zero_()
    ssq[:, 0] = (x32 * x32).sum(-1)


def apply_row_scale(hprime, ssq, width, eps, out):
    _store(out, hprime.float() * _factor((ssq, width, eps)))


def interleave_gate_up(gate, up):
    I, Kd = gate.shape
    return torch.stack((gate.view(I // 8, 8, Kd), up.view(I // 8, 8, Kd)), dim=1).reshape(2 * I, Kd).contiguous()


def rope_kv_write(qkv, positions, denominators, rotary_dim, slot_mapping, k_cache, v_cache,
                  num_heads, num_kv_heads, head_dim, write=True):
    T = qkv.shape[0]
    q_dim, kv_dim = num_heads * head_dim, num_kv_heads * head_dim
    half = rotary_dim // 2
    if rotary_dim:
        phi = positions.float()[:, None] / denominators[None, :]
        cos, sin = torch.cos(phi)[:, None, :], torch.sin(phi)[:, None, :]

    def rot(x):
        x = x.float().clone()
        if not rotary_dim:
            return x
        a, b = x[..., :half].clone(), x[..., half:rotary_dim].clone()
        x[..., :half] = a * cos - b * sin
        x[..., half:rotary_dim] = b * cos + a * sin
        return x

    q = rot(qkv[:, :q_dim].reshape(T, num_heads, head_dim))
    qkv[:, :q_dim] = q.reshape(T, q_dim).to(qkv.dtype)
    if not write:
        return
    k = rot(qkv[:, q_dim:q_dim + kv_dim].reshape(T, num_kv_heads, head_dim)).to(qkv.dtype)
    v = qkv[:, q_dim + kv_dim:].reshape(T, num_kv_heads, head_dim)
    page_size = k_cache.shape[2]
    page = (slot_mapping // page_size).long()
    off = (slot_mapping % page_size).long()
    k_cache[page, :, off] = k
    v_cache[page, :, :, off] = v         # values are cached transposed: [page, kv_head, head_dim, slot]


def linear_rope_kv(a, weight, bias, qkv, positions, denominators, rotary_dim, slot_mapping, k_cache, v_cache,
                   num_heads, num_kv_heads, head_dim, write=True, fused=True, row_scale=None, cos_sin=None):
    linear(a, weight, bias, qkv, row_scale=row_scale)
    rope_kv_write(qkv, positions, denominators, rotary_dim, slot_mapping, k_cache, v_cache, num_heads, num_kv_heads, head_dim, write)


def rope_table(positions, denominators, out):
    phi = positions.float().unsqueeze(1) / denominators.unsqueeze(0)
    out[..., 0] = torch.cos(phi)
    out[..., 1] = torch.sin(phi)


def paged_attention(qkv, out, k_cache, v_cache, block_table, q_start, ctx_lens, seq_of_token, positions,
                    num_heads, num_kv_heads, head_dim, scale, window, max_q_len, max_ctx_len, implementation=None, old_lens=None, singles=0,
                    units=None, unit_slots=(0, 0)):
    # old_lens only tells a kernel which keys it may read early, singles which kernel takes which sequence, units how a
    # kernel shares its work out; the result does not depend on them
    T = qkv.shape[0]
    page_size = k_cache.shape[2]
    group = num_heads // num_kv_heads
    q = qkv[:, :num_heads * head_dim].reshape(T, num_heads, head_dim).float()
    res = torch.zeros(T, num_heads, head_dim, dtype=torch.float32, device=qkv.device)
    seqs = seq_of_token.tolist()
    poss = positions.tolist()
    for t in range(T):
        s, p = seqs[t], poss[t]
        lo = 0 if not window else max(0, p - window + 1)
        keys = torch.arange(lo, p + 1, device=qkv.device)
        pages = block_table[s].long()[keys // page_size]
        offs = keys % page_size
        k = k_cache[pages, :, offs].float()          # [n, kv_heads, dh]
        v = v_cache[pages, :, :, offs].float()
        for h in range(num_heads):
            sc = (k[:, h // group] @ q[t, h]) * scale
            pr = torch.softmax(sc, dim=0)
            res[t, h] = pr @ v[:, h // group]
    _store(out, res.reshape(T, num_heads * head_dim))


def paged_attention_dense(qkv, out, k_cache, v_cache, block_table, q_start, ctx_lens, seq_of_token, positions,
                          num_heads, num_kv_heads, head_dim, scale, window, max_q_len, max_ctx_len, implementation=None, old_lens=None,
                          singles=0, units=None, unit_slots=(0, 0)):
    """The same formula as :func:`paged_attention`, a sequence at a time instead of a token and a head at a time (for
    contexts of thousands of keys): scores of all the sequence's tokens against all its keys in float32, keys outside
    [p - window + 1, p] masked, softmax, weighted sum."""
    T = qkv.shape[0]
    page_size = k_cache.shape[2]
    group = num_heads // num_kv_heads
    q = qkv[:, :num_heads * head_dim].reshape(T, num_heads, head_dim).float()
    res = torch.zeros(T, num_heads, head_dim, dtype=torch.float32, device=qkv.device)
    starts, lens = q_start.tolist(), ctx_lens.tolist()
    for s, c in enumerate(lens):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        keys = torch.arange(c, device=qkv.device)
        pages = block_table[s].long()[keys // page_size]
        offs = keys % page_size
        k = k_cache[pages, :, offs].float().repeat_interleave(group, dim=1)          # [c, heads, dh]
        v = v_cache[pages, :, :, offs].float().repeat_interleave(group, dim=1)
        pos = positions[lo:hi].long()
        sc = torch.einsum("thd,chd->htc", q[lo:hi], k) * scale
        seen = keys[None, :] <= pos[:, None]
        if window:
            seen &= keys[None, :] > pos[:, None] - window
        sc = sc.masked_fill(~seen[None], float("-inf"))
        res[lo:hi] = torch.einsum("htc,chd->thd", torch.softmax(sc, dim=-1), v)
    _store(out, res.reshape(T, num_heads * head_dim))


def gather_rows(src, rows, out):
    out.copy_(src[rows.long()])


def scale_inplace(x32, factor):
    x32.mul_(factor)


def logit_cap(logits, cap):
    logits.copy_(cap * torch.tanh(logits / cap))


def swiglu(gate_up, out):
    I = gate_up.shape[1] // 2
    g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    _store(out, u * (g / (1.0 + torch.exp(-g))))


def argmax(logits, out):
    # first maximum
    m = logits.max(dim=1, keepdim=True).values
    idx = torch.where(logits == m, torch.arange(logits.shape[1], device=logits.device)[None, :], logits.shape[1]).min(dim=1).values
    out.copy_(idx.to(torch.int32))


# ---- sampling ---------------------------------------------------------------

_M64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform_for(seed: int, output_index: int, token: int) -> float:
    """The generator of the sample kernel: 23 bits of a hash of (seed, index, token), in (0, 1)."""
    key = _splitmix64((seed & _M64) ^ _splitmix64(output_index & _M64))
    bits = _splitmix64(key ^ ((token * 0xD1342543DE82EF95) & _M64)) >> 41
    return (bits + 0.5) / 8388608.0


def sample_row(logits_row, temperature, top_k, top_p, seed, output_index):
    """(token, kept ids) as the sample kernel computes them."""
    z = logits_row.float().cpu()
    V = z.numel()
    if temperature <= 0.0 or top_k == 1:
        m = z.max()
        return int(torch.nonzero(z == m)[0]), None
    z = z / np.float32(temperature)
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.topk(z, top_k).values[-1]
        keep &= z >= kth
    if 0.0 < top_p < 1.0:
        m = z[keep].max()
        e = torch.where(keep, torch.exp(z - m), torch.zeros(()))
        p = e / e.sum()
        # kept iff the probability mass of strictly larger candidates is below top_p
        order = torch.argsort(z, descending=True, stable=True)
        ps = p[order]
        zs = z[order]
        before = torch.cumsum(ps, 0) - ps
        # equal values share the mass before the first of them
        first_of_value = torch.ones(V, dtype=torch.bool)
        first_of_value[1:] = zs[1:] != zs[:-1]
        idx = torch.where(first_of_value, torch.arange(V), torch.zeros((), dtype=torch.long))
        idx = torch.cummax(idx, 0).values
        before = before[idx]
        ok = torch.zeros(V, dtype=torch.bool)
        ok[order] = before < top_p
        keep &= ok
    u = torch.tensor([uniform_for(seed, output_index, i) for i in range(V)], dtype=torch.float32)
    g = -torch.log(-torch.log(u))
    score = torch.where(keep, z + g, torch.full((), float("-inf")))
    m = score.max()
    return int(torch.nonzero(score == m)[0]), torch.nonzero(keep).flatten().tolist()


def sample(logits, params, out):
    host = params.cpu()
    f = host.view(torch.float32)
    res = []
    for r in range(logits.shape[0]):
        seed = (int(host[r, 3]) & 0xFFFFFFFF) | ((int(host[r, 4]) & 0xFFFFFFFF) << 32)
        tok, _ = sample_row(logits[r], float(f[r, 0]), int(host[r, 1]), float(f[r, 2]), seed, int(host[r, 5]))
        res.append(tok)
    out.copy_(torch.tensor(res, dtype=torch.int32))


def table_gather(resident, updates, slots, out, trash_page):
    """The resident block tables brought up to date and a row per sequence copied out: plain loops."""
    rows, cols = resident.shape
    n = int(updates[0])
    wanted = set(int(x) for x in slots.tolist())
    for i in range(n):
        slot, block, page = (int(x) for x in updates[1 + 3 * i:4 + 3 * i].tolist())
        if slot in wanted and slot != rows - 1 and 0 <= block < cols:
            resident[slot, block] = page
    for s, slot in enumerate(slots.tolist()):
        slot = slot if 0 <= slot < rows else rows - 1
        for b in range(out.shape[1]):
            out[s, b] = resident[slot, b] if b < cols else trash_page


ALL = ["table_gather", "gather_rows", "scale_inplace", "logit_cap", "rope_table", "linear_scaled_accepts", "linear_add_scaled_parts", "linear_add_scaled", "apply_row_scale", "linear_rope_kv", "interleave_gate_up", "embedding", "rmsnorm", "add_rmsnorm", "gather_rmsnorm", "residual_add", "linear", "rope_kv_write",
       "paged_attention", "swiglu", "argmax", "sample"]
