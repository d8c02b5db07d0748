"""Python face of the CUDA kernels in ``csrc/``: one function per kernel.

Each function checks its arguments (device, dtype, shape, contiguity) and
launches on the current CUDA stream of torch through the library's C
interface.  There is no other implementation behind these names: tensors that
are not on a CUDA device, a missing compiler or a failed build raise an error.

Conventions: the residual stream ``x32`` is float32; activations, matrices
and the cache are in the run dtype (bfloat16 or float32, never mixed in one
call); norm weights, biases and logits are float32; index tensors are int32.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Optional, Tuple

import torch

from .csrc.build import ensure_built

_lib = None
_lib_lock = threading.Lock()

_F32, _BF16 = 0, 1
launches = 0            # kernels launched through this module since import (bench reads it)


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The kernel library, built on first use."""
    global _lib
    if _lib is None:
        with _lib_lock:
            if _lib is None:
                path = ensure_built()
                lib = ctypes.CDLL(str(path))
                lib.li_last_error.restype = ctypes.c_char_p
                _lib = lib
    return _lib


def library_file() -> str:
    library()
    return str(ensure_built(verbose=False))


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"run dtype must be float32 or bfloat16, got {t.dtype}")


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise KernelError(f"{name}: the kernels run on CUDA devices only, tensor is on '{t.device}'")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if shape is not None and t.shape != tuple(shape):
        raise KernelError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# the current stream's handle without building a Stream object (a few hundred launches a step ask for it)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t: torch.Tensor):
    if _raw_stream is not None:
        index = t.device.index
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device() if index is None else index))
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _check(rc: int, what: str) -> None:
    global launches
    launches += 1
    if rc != 0:
        msg = library().li_last_error()
        raise KernelError(f"{what}: {msg.decode() if msg else 'error ' + str(rc)}")


_i = ctypes.c_int
_f = ctypes.c_float
_l = ctypes.c_longlong


# --------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids: torch.Tensor, out32: torch.Tensor) -> None:
    """out32[t, :] = float(table[ids[t], :])."""
    V, H = table.shape
    T = ids.shape[0]
    _need(table, "embedding table")
    _need(ids, "token ids", torch.int32)
    _need(out32, "embedding output", torch.float32, (T, H))
    _check(library().li_embedding(_p(table), _i(_dt(table)), _p(ids), _p(out32), _i(T), _i(H), _i(V), _stream(out32)), "embedding")


def rmsnorm(x32: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    T, H = x32.shape
    _need(x32, "rmsnorm input", torch.float32)
    _need(weight, "rmsnorm weight", torch.float32, (H,))
    _need(out, "rmsnorm output", None, (T, H))
    _check(library().li_rmsnorm(_p(x32), _p(weight), _f(eps), _p(out), _i(_dt(out)), _i(T), _i(H), _stream(out)), "rmsnorm")


def add_rmsnorm(x32: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """x32 += delta (float32 sum, kept in x32); out = rmsnorm(x32)."""
    T, H = x32.shape
    _need(x32, "add_rmsnorm residual", torch.float32)
    _need(delta, "add_rmsnorm delta", None, (T, H))
    _need(weight, "rmsnorm weight", torch.float32, (H,))
    _need(out, "add_rmsnorm output", delta.dtype, (T, H))
    _check(library().li_add_rmsnorm(_p(x32), _p(delta), _i(_dt(delta)), _p(weight), _f(eps), _p(out), _i(T), _i(H), _stream(out)),
           "add_rmsnorm")


def gather_rmsnorm(x32: torch.Tensor, rows: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out[r] = rmsnorm(x32[rows[r]])."""
    T, H = x32.shape
    R = rows.shape[0]
    _need(x32, "gather_rmsnorm input", torch.float32)
    _need(rows, "gather_rmsnorm rows", torch.int32)
    _need(weight, "rmsnorm weight", torch.float32, (H,))
    _need(out, "gather_rmsnorm output", None, (R, H))
    _check(library().li_gather_rmsnorm(_p(x32), _p(rows), _p(weight), _f(eps), _p(out), _i(_dt(out)), _i(R), _i(T), _i(H), _stream(out)),
           "gather_rmsnorm")


def residual_add(x32: torch.Tensor, delta: torch.Tensor) -> None:
    _need(x32, "residual", torch.float32)
    _need(delta, "delta", None, x32.shape)
    _check(library().li_residual_add(_p(x32), _p(delta), _i(_dt(delta)), _l(x32.numel()), _stream(x32)), "residual_add")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float) -> None:
    """``out[i] = mean + std * n(key, i)`` (flat index i) with n standard normal from the library's counter-based
    generator; float32 or bfloat16.  ``litinfer_b200.weights.random_init`` restates the recipe on the host."""
    _need(out, "fill_normal output")
    _check(library().li_fill_normal(_p(out), _i(_dt(out)), _l(out.numel()), ctypes.c_ulonglong(key & ((1 << 64) - 1)), _f(mean), _f(std),
                                    _stream(out)), "fill_normal")


def fill_randint(out: torch.Tensor, key: int, high: int) -> None:
    """``out[i]`` = an integer in [0, high) from (key, i); int32."""
    _need(out, "fill_randint output", torch.int32)
    _check(library().li_fill_randint(_p(out), _l(out.numel()), ctypes.c_ulonglong(key & ((1 << 64) - 1)), _i(high), _stream(out)),
           "fill_randint")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """``out[r] = src[rows[r]]`` for float32 rows (int32 ``rows`` on the device)."""
    _need(src, "gather source", torch.float32)
    _need(rows, "gather rows", torch.int32, (out.shape[0],))
    _need(out, "gather output", torch.float32, (rows.shape[0], src.shape[1]))
    _check(library().li_gather_rows(_p(src), _p(rows), _p(out), _i(src.shape[0]), _i(rows.shape[0]), _l(src.shape[1]), _stream(out)), "gather_rows")


def table_gather(resident: torch.Tensor, updates: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, trash_page: int) -> None:
    """Bring the resident block tables (int32 ``[slots + 1, cols]``, the last row all sink page) up to date with
    ``updates`` (a count, then triples of slot, logical page, page id) for the step's sequences (``slots`` int32 ``[S]``)
    and copy each sequence's row into the step's table ``out`` (int32 ``[S, max_blocks]``)."""
    _need(resident, "resident block tables", torch.int32)
    _need(updates, "table updates", torch.int32)
    _need(slots, "state slots", torch.int32)
    S = slots.shape[0]
    _need(out, "the step's block table", torch.int32, (S, out.shape[1]))
    if resident.dim() != 2 or updates.numel() < 1 or (updates.numel() - 1) % 3:
        raise KernelError(f"table_gather: resident {tuple(resident.shape)}, {updates.numel()} words of updates")
    _check(library().li_table_gather(_p(resident), _i(resident.shape[0]), _i(resident.shape[1]), _p(updates), _i((updates.numel() - 1) // 3),
                                     _p(slots), _p(out), _i(S), _i(out.shape[1]), _i(int(trash_page)), _stream(out)), "table_gather")


OVERLAP_KINDS = {"gemm": 1, "streaming_products": 2, "attention": 4, "rest": 8}


def allow_overlap(but: tuple = ()) -> None:
    """The launches that follow may begin while the kernel before them still runs (programmatic dependent launch),
    except the kinds of kernel named in ``but`` (keys of OVERLAP_KINDS).  The step function sets this per step."""
    library().li_pdl_allow(ctypes.c_int(sum(OVERLAP_KINDS[k] for k in but)))


def scale_inplace(x32: torch.Tensor, factor: float) -> None:
    """x32 *= factor (float32, in place)."""
    _need(x32, "scale operand", torch.float32)
    _check(library().li_scale_inplace(_p(x32), _l(x32.numel()), _f(factor), _stream(x32)), "scale")


def logit_cap(logits: torch.Tensor, cap: float) -> None:
    """logits = cap * tanh(logits / cap) (float32, in place)."""
    _need(logits, "logits", torch.float32)
    _check(library().li_logit_cap(_p(logits), _l(logits.numel()), _f(cap), _stream(logits)), "logit_cap")


EPILOGUES = {None: 0, "swiglu": 1}


def _linear_args(a, weight, bias, out, epilogue):
    M, Kd = a.shape
    N = weight.shape[0]
    _need(a, "linear input")
    _need(weight, "linear weight", a.dtype, (N, Kd))
    if bias is not None:
        _need(bias, "linear bias", torch.float32, (N,))
    if epilogue not in EPILOGUES:
        raise KernelError(f"linear: unknown epilogue {epilogue!r}")
    _need(out, "linear output", None, (M, N // 2 if epilogue == "swiglu" else N))
    if out.dtype not in (a.dtype, torch.float32):
        raise KernelError(f"linear output must be {a.dtype} or float32, got {out.dtype}")
    return M, N, Kd


def linear(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
           epilogue: Optional[str] = None, row_scale=None) -> None:
    """out[M, N] = a[M, K] weight[N, K]^T (+ bias[N]); float32 accumulation;
    out is in the run dtype or float32.

    ``row_scale=(ssq, width, eps)``: every token's row of the product is multiplied by
    ``1 / sqrt(sum_p ssq[t, p] / width + eps)`` before bias and epilogue (see :func:`linear_add_scaled`); an error
    unless :func:`linear_scaled_accepts`.

    ``epilogue="swiglu"`` (bfloat16 only): ``weight`` holds gate and up rows interleaved in
    groups of 8 (see :func:`interleave_gate_up`) and out[M, N / 2] = up * gate / (1 + exp(-gate))."""
    M, N, Kd = _linear_args(a, weight, bias, out, epilogue)
    if M == 0:
        return
    if row_scale is not None:
        _check(library().li_linear_scaled(_p(a), _p(weight), _p(bias), _p(out), _i(_dt(a)), _i(_dt(out)), _i(M), _i(N), _i(Kd),
                                          _i(EPILOGUES[epilogue]), *_row_scale_args(row_scale, M), _stream(out)), "linear (scaled)")
        return
    _check(library().li_linear(_p(a), _p(weight), _p(bias), _p(out), _i(_dt(a)), _i(_dt(out)), _i(M), _i(N), _i(Kd),
                               _i(EPILOGUES[epilogue]), _stream(out)), "linear")


def _row_scale_args(row_scale, M: int):
    ssq, width, eps = row_scale
    _need(ssq, "partial sums of squares", torch.float32)
    if ssq.dim() != 2 or ssq.shape[0] != M:
        raise KernelError(f"partial sums of squares of shape {tuple(ssq.shape)} for {M} tokens")
    return _p(ssq), _i(ssq.shape[1]), _i(int(width)), _f(float(eps))


def linear_scaled_accepts(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether :func:`linear` takes ``row_scale`` for these operands (bfloat16, at most 64 tokens)."""
    M, Kd = a.shape
    return bool(library().li_linear_scaled_accepts(_p(a), _p(weight), _p(out), _i(_dt(a)), _i(M), _i(weight.shape[0]), _i(Kd)))


def linear_add_scaled_parts(a: torch.Tensor, weight: torch.Tensor, x32: torch.Tensor, hprime: torch.Tensor) -> int:
    """How many partial sums per token :func:`linear_add_scaled` writes for these operands; 0 if no kernel takes them."""
    M, Kd = a.shape
    return int(library().li_linear_add_scaled_parts(_p(a), _p(weight), _p(x32), _p(hprime), _i(_dt(a)), _i(M), _i(weight.shape[0]), _i(Kd)))


def linear_add_scaled(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], x32: torch.Tensor,
                      norm_weight: torch.Tensor, hprime: torch.Tensor, ssq: torch.Tensor) -> None:
    """The product into the residual stream with the next RMSNorm half done, as one kernel (few bfloat16 tokens):
    ``x32 += a weight^T (+ bias)``; ``hprime = bfloat16(norm_weight * x32)``; ``ssq[t, p]`` = the sum of the new
    ``x32[t]^2`` over the columns of the product's tile p.  The normalised activation is
    ``hprime[t] / sqrt(sum_p ssq[t, p] / N + eps)``; :func:`linear` applies that factor to its own result
    (``row_scale``), :func:`apply_row_scale` to hprime itself."""
    M, Kd = a.shape
    N = weight.shape[0]
    _need(a, "linear input", torch.bfloat16)
    _need(weight, "linear weight", a.dtype, (N, Kd))
    if bias is not None:
        _need(bias, "linear bias", torch.float32, (N,))
    _need(x32, "residual stream", torch.float32, (M, N))
    _need(norm_weight, "rmsnorm weight", torch.float32, (N,))
    _need(hprime, "weighted sum", a.dtype, (M, N))
    parts = linear_add_scaled_parts(a, weight, x32, hprime)
    if parts == 0:
        raise KernelError(f"linear_add_scaled: no kernel for {M} tokens, N={N}, K={Kd}")
    _need(ssq, "partial sums of squares", torch.float32, (M, parts))
    _check(library().li_linear_add_scaled(_p(a), _p(weight), _p(bias), _p(x32), _p(norm_weight), _p(hprime), _p(ssq), _i(_dt(a)),
                                          _i(M), _i(N), _i(Kd), _stream(hprime)), "linear_add_scaled")


def apply_row_scale(hprime: torch.Tensor, ssq: torch.Tensor, width: int, eps: float, out: torch.Tensor) -> None:
    """``out[t] = hprime[t] / sqrt(sum_p ssq[t, p] / width + eps)`` (bfloat16)."""
    M, H = hprime.shape
    _need(hprime, "weighted sum", torch.bfloat16)
    _need(out, "normalised output", torch.bfloat16, (M, H))
    p_ssq, nparts, w, e = _row_scale_args((ssq, width, eps), M)
    _check(library().li_apply_row_scale(_p(hprime), p_ssq, nparts, w, e, _p(out), _i(M), _i(H), _stream(out)), "apply_row_scale")


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up rows as one [2 I, K] matrix in the order the swiglu epilogue reads:
    8 gate rows, the 8 up rows of the same outputs, the next 8 gate rows, ... (I a multiple of 8)."""
    I, Kd = gate.shape
    if I % 8 or up.shape != gate.shape:
        raise KernelError(f"interleave_gate_up: shapes {tuple(gate.shape)} / {tuple(up.shape)}, rows must be a multiple of 8")
    return torch.stack((gate.view(I // 8, 8, Kd), up.view(I // 8, 8, Kd)), dim=1).reshape(2 * I, Kd).contiguous()


LINEAR_IMPLEMENTATIONS = {"simt": 0, "gemv": 1, "tcgen05": 2, "gemv_tcgen05": 3}


def linear_with(which: str, a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                epilogue: Optional[str] = None) -> None:
    """:func:`linear` through one named kernel (``simt``, ``gemv``, ``tcgen05``, ``gemv_tcgen05``); an error
    if that kernel refuses the sizes.  For tests and measurements of a kernel alone."""
    M, N, Kd = _linear_args(a, weight, bias, out, epilogue)
    _check(library().li_linear_with(_i(LINEAR_IMPLEMENTATIONS[which]), _p(a), _p(weight), _p(bias), _p(out), _i(_dt(a)),
                                    _i(_dt(out)), _i(M), _i(N), _i(Kd), _i(EPILOGUES[epilogue]), _stream(out)), f"linear[{which}]")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, denominators: torch.Tensor, rotary_dim: int,
                  slot_mapping: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  num_heads: int, num_kv_heads: int, head_dim: int, write: bool = True) -> None:
    """Rotate q (in place in ``qkv``) and k; store rotated k and plain v at each
    token's slot of the caches: keys ``[pages, kv_heads, page_size, head_dim]``, values
    transposed ``[pages, kv_heads, head_dim, page_size]``.
    With ``write`` false only q is rotated.  ``rotary_dim`` 0 (``denominators`` may be None): nothing is
    rotated, keys and values are stored as they are."""
    T = qkv.shape[0]
    _need(qkv, "qkv", None, (T, (num_heads + 2 * num_kv_heads) * head_dim))
    _need(positions, "positions", torch.int32, (T,))
    if rotary_dim:
        _need(denominators, "rope denominators", torch.float32, (rotary_dim // 2,))
    _need(slot_mapping, "slot mapping", torch.int32, (T,))
    _need(k_cache, "key cache", qkv.dtype)
    pages, nkv, page_size, dh = k_cache.shape
    _need(v_cache, "value cache", qkv.dtype, (pages, nkv, dh, page_size))
    if nkv != num_kv_heads or dh != head_dim:
        raise KernelError(f"cache of {nkv} heads x {dh} does not match {num_kv_heads} x {head_dim}")
    _check(library().li_rope_kv_write(
        _p(qkv), _i(_dt(qkv)), _p(positions), _p(denominators if rotary_dim else None), _i(rotary_dim), _p(slot_mapping), _p(k_cache), _p(v_cache),
        _i(T), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(page_size), _i(pages), _i(1 if write else 0), _stream(qkv)),
        "rope_kv_write")


def linear_rope_kv(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], qkv: torch.Tensor,
                   positions: torch.Tensor, denominators: torch.Tensor, rotary_dim: int, slot_mapping: torch.Tensor,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                   write: bool = True, fused: bool = True, row_scale=None, cos_sin: Optional[torch.Tensor] = None) -> None:
    """The fused q|k|v projection followed by :func:`rope_kv_write`: ``qkv = a weight^T + bias``, q rotated in
    place, k rotated and v stored into the caches.  Keys and values are only guaranteed to be in the caches
    afterwards, not in ``qkv``.  For a few bfloat16 tokens both steps run as one kernel (the rotation is the
    product's epilogue); ``fused=False`` forces two kernels, for tests.  ``row_scale`` as in :func:`linear`.
    ``cos_sin``: the step's table from :func:`rope_table`; with it a long bfloat16 step (head_dim 128) rotates and
    writes the cache in the epilogue of the tensor-memory product too.  ``rotary_dim`` 0 (``denominators`` may be
    None): no rotation, as in :func:`rope_kv_write`."""
    T, Kd = a.shape
    N = (num_heads + 2 * num_kv_heads) * head_dim
    _need(a, "linear input")
    _need(weight, "qkv weight", a.dtype, (N, Kd))
    if bias is not None:
        _need(bias, "qkv bias", torch.float32, (N,))
    _need(qkv, "qkv", a.dtype, (T, N))
    _need(positions, "positions", torch.int32, (T,))
    if rotary_dim:
        _need(denominators, "rope denominators", torch.float32, (rotary_dim // 2,))
    _need(slot_mapping, "slot mapping", torch.int32, (T,))
    if cos_sin is not None:
        _need(cos_sin, "rope table", torch.float32, (T, rotary_dim // 2, 2))
    _need(k_cache, "key cache", a.dtype)
    pages, nkv, page_size, dh = k_cache.shape
    _need(v_cache, "value cache", a.dtype, (pages, nkv, dh, page_size))
    if nkv != num_kv_heads or dh != head_dim:
        raise KernelError(f"cache of {nkv} heads x {dh} does not match {num_kv_heads} x {head_dim}")
    _check(library().li_linear_rope_kv(
        _p(a), _p(weight), _p(bias), _p(qkv), _i(_dt(a)), _p(positions), _p(denominators if rotary_dim else None), _i(rotary_dim), _p(slot_mapping),
        _p(k_cache), _p(v_cache), _i(T), _i(Kd), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(page_size), _i(pages),
        _i(1 if write else 0), _i(1 if fused else 0),
        *(_row_scale_args(row_scale, T) if row_scale is not None else (_p(None), _i(0), _i(0), _f(0.0))), _p(cos_sin), _stream(qkv)),
        "linear_rope_kv")


def rope_table(positions: torch.Tensor, denominators: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, j] = (cos, sin)(float(positions[t]) / denominators[j])``: the angles of a step, for products that rotate in
    their epilogue (:func:`linear_rope_kv`)."""
    T = positions.shape[0]
    half = denominators.shape[0]
    _need(positions, "positions", torch.int32, (T,))
    _need(denominators, "rope denominators", torch.float32, (half,))
    _need(out, "rope table", torch.float32, (T, half, 2))
    _check(library().li_rope_table(_p(positions), _p(denominators), _i(half), _p(out), _i(T), _stream(out)), "rope_table")


ATTENTION_IMPLEMENTATIONS = {"general": 0, "decode": 1, "prefill": 2, "prefill_tcgen05": 3}


def paged_attention(qkv: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, q_start: torch.Tensor, ctx_lens: torch.Tensor,
                    seq_of_token: torch.Tensor, positions: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
                    max_q_len: int, max_ctx_len: int, implementation: Optional[str] = None,
                    old_lens: Optional[torch.Tensor] = None, singles: int = 0,
                    units: Optional[torch.Tensor] = None, unit_slots: Tuple[int, int] = (0, 0)) -> None:
    """Causal grouped-query attention of the step's tokens over the paged cache.

    Queries are the first ``num_heads * head_dim`` columns of ``qkv`` (already
    rotated).  The token at position p of sequence s sees the cached keys
    ``max(0, p - window + 1) .. p`` of s, found through ``block_table[s]``.
    ``implementation`` (``general``, ``decode``, ``prefill``, ``prefill_tcgen05``) forces one kernel, for
    tests and measurements; it is an error if that kernel refuses the sizes.
    ``old_lens`` (int32 ``[S]``): how many keys of each sequence were in the cache before this step; needed when
    several sequences of the step are tokens of one request (None: all but each sequence's last key).
    ``singles``: how many sequences of a step with longer portions have one token (negative: not known).  They then
    go to the decode kernel, the rest to the kernel for portions (bfloat16).
    ``units`` (int32, from ``engine.batch.attention_units``): the work list of the kernel for long portions, with
    ``unit_slots`` = how many entries to launch when the single tokens are the decode kernel's, and when not."""
    T = qkv.shape[0]
    S = ctx_lens.shape[0]
    _need(qkv, "qkv", None, (T, (num_heads + 2 * num_kv_heads) * head_dim))
    _need(out, "attention output", qkv.dtype, (T, num_heads * head_dim))
    _need(k_cache, "key cache", qkv.dtype)
    _need(v_cache, "value cache", qkv.dtype, (k_cache.shape[0], k_cache.shape[1], k_cache.shape[3], k_cache.shape[2]))
    _need(block_table, "block table", torch.int32)
    _need(q_start, "q_start", torch.int32, (S + 1,))
    _need(ctx_lens, "ctx_lens", torch.int32, (S,))
    _need(seq_of_token, "seq_of_token", torch.int32, (T,))
    _need(positions, "positions", torch.int32, (T,))
    pages, nkv, page_size, dh = k_cache.shape
    if block_table.dim() != 2 or block_table.shape[0] != S:
        raise KernelError(f"block table must be [{S}, max_blocks], got {tuple(block_table.shape)}")
    if nkv != num_kv_heads or dh != head_dim:
        raise KernelError(f"cache of {nkv} heads x {dh} does not match {num_kv_heads} x {head_dim}")
    if block_table.shape[1] * page_size < max_ctx_len:
        raise KernelError(f"block table of {block_table.shape[1]} pages cannot cover a context of {max_ctx_len}")
    if old_lens is not None:
        _need(old_lens, "old_lens", torch.int32, (S,))
    if units is not None:
        _need(units, "attention work list", torch.int32)
        if units.numel() < 4 + 4 * max(unit_slots) or units.data_ptr() % 16:
            raise KernelError(f"attention work list of {units.numel()} words cannot hold {max(unit_slots)} entries (or is not 16-byte aligned)")
    args = (_p(qkv), _p(out), _p(k_cache), _p(v_cache), _i(_dt(qkv)), _p(block_table), _i(block_table.shape[1]),
            _p(q_start), _p(ctx_lens), _p(seq_of_token), _p(positions), _i(T), _i(S),
            _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(page_size), _i(pages), _f(scale),
            _i(0 if window is None else int(window)), _i(max_q_len), _i(max_ctx_len), _p(old_lens), _i(int(singles)),
            _p(units), _i(int(unit_slots[0])), _i(int(unit_slots[1])), _stream(out))
    if implementation is None:
        _check(library().li_paged_attention(*args), "paged_attention")
    else:
        _check(library().li_paged_attention_with(_i(ATTENTION_IMPLEMENTATIONS[implementation]), *args),
               f"paged_attention[{implementation}]")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = up * gate / (1 + exp(-gate)) with gate_up = [gate | up] along the last axis."""
    T, I2 = gate_up.shape
    _need(gate_up, "gate_up")
    _need(out, "swiglu output", gate_up.dtype, (T, I2 // 2))
    _check(library().li_swiglu(_p(gate_up), _p(out), _i(_dt(out)), _i(T), _i(I2 // 2), _stream(out)), "swiglu")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """Index of the first maximum of each row."""
    R, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out, "argmax output", torch.int32, (R,))
    _check(library().li_argmax(_p(logits), _p(out), _i(R), _i(V), _stream(out)), "argmax")


def sample(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor) -> None:
    """One token per row.  ``params`` int32 [R, 6]: temperature (float bits; <= 0
    is argmax), top_k, top_p (float bits), seed low, seed high, output index."""
    R, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(params, "sampling parameters", torch.int32, (R, 6))
    _need(out, "sample output", torch.int32, (R,))
    _check(library().li_sample(_p(logits), _p(params), _p(out), _i(R), _i(V), _stream(out)), "sample")


# --------------------------------------------------------------------------
# LLAISYS_PROFILE=1: device time per kernel function, keyed by phase, reported at exit
# --------------------------------------------------------------------------
# LitInfer's switch of the same name (src/utils/profiler.cpp:47-104) times every operator call on the CPU and prints
# a table of "phase/op  calls  time(ms)  pct(%)" to standard error when the process ends.  Here an operator call is a
# kernel launch, so the time is the device's: a pair of CUDA events around each call, read when the report is made.
# While the switch is on the step function launches every kernel from the host (no captured graphs: a replayed graph
# runs without passing through these functions).

def _env_on(name: str) -> bool:
    import os

    return os.environ.get(name, "").lower() in ("1", "true", "on")


class Profile:
    def __init__(self) -> None:
        self.enabled = _env_on("LLAISYS_PROFILE")
        self.phase = ""
        self._pending = []                                 # (key, start event, stop event)
        self.total_ms = {}
        self.calls = {}
        if self.enabled:
            import atexit

            atexit.register(self.report)

    def reset(self) -> None:
        self._pending.clear()
        self.total_ms.clear()
        self.calls.clear()

    def wrap(self, name, fn):
        import functools

        @functools.wraps(fn)
        def timed(*args, **kwargs):
            if not self.enabled or not torch.cuda.is_available():
                return fn(*args, **kwargs)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            try:
                return fn(*args, **kwargs)
            finally:
                stop.record()
                self._pending.append(((self.phase + "/" + name) if self.phase else name, start, stop))
                if len(self._pending) >= 4096:
                    self.collect()

        return timed

    def collect(self) -> None:
        if self._pending:
            torch.cuda.synchronize()
        for key, start, stop in self._pending:
            self.total_ms[key] = self.total_ms.get(key, 0.0) + start.elapsed_time(stop)
            self.calls[key] = self.calls.get(key, 0) + 1
        self._pending.clear()

    def report(self, out=None) -> None:
        import sys

        out = out or sys.stderr
        self.collect()
        grand = sum(self.total_ms.values())
        print("\n================ LLAISYS PROFILE ================", file=out)
        if grand <= 0.0:
            print("(no profiled operations)\n================================================", file=out)
            return
        print(f"  total op time: {grand:.3f} ms (device time of kernel launches)", file=out)
        print("------------------------------------------------", file=out)
        print("  op                          calls     time(ms)    pct(%)", file=out)
        for key, ms in sorted(self.total_ms.items(), key=lambda kv: -kv[1]):
            print(f"  {key:<28}{self.calls[key]:>8}{ms:>12.3f}{100.0 * ms / grand:>9.2f}", file=out)
        print("================================================", file=out, flush=True)


profile = Profile()
TRACE = _env_on("LLAISYS_TRACE")          # LitInfer's other switch (src/llaisys/models/qwen2.cpp:17-26): a line per call on standard error

_TIMED = ("embedding", "rmsnorm", "add_rmsnorm", "gather_rmsnorm", "residual_add", "linear", "linear_add_scaled", "apply_row_scale",
          "rope_kv_write", "linear_rope_kv", "rope_table", "paged_attention", "swiglu", "argmax", "sample", "gather_rows", "scale_inplace",
          "logit_cap")
if profile.enabled:
    for _name in _TIMED:
        globals()[_name] = profile.wrap(_name, globals()[_name])
