"""The entry point for callers that may not allocate device memory
(litinfer_b200/csrc/no_alloc.h): li_linear_gemv_static, called through its
exported C symbol, against the ordinary weight-streaming kernel and against the
plain float32 product.

Some hosts of this library cannot let it call cudaMalloc: a server that owns
the whole device arena, a latency-critical loop where an allocation would
synchronise the device.  The ordinary kernel
allocates its split-k workspace on first use; this variant keeps partial sums
and arrival counters in fixed __device__ arrays inside the library instead.

Collected last on purpose (the file name sorts after the others): if it fails,
a run that stops at the first failure has already run everything else.  It
passes alone in a fresh process as well as after the other tests, because each
call clears the counters it uses and the arrays are the library's own.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

import kernel_refs as R

pytestmark = pytest.mark.gpu


def _call_static(lib, a, w, bias, out):
    M, Kd = a.shape
    N = w.shape[0]
    fn = lib.li_linear_gemv_static
    fn.restype = ctypes.c_int
    rc = fn(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(bias.data_ptr() if bias is not None else 0),
            ctypes.c_void_p(out.data_ptr()), ctypes.c_int(1 if out.dtype == torch.bfloat16 else 0), ctypes.c_int(M), ctypes.c_int(N),
            ctypes.c_int(Kd), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, (lib.li_last_error() or b"").decode()


# (M, N, K): with and without a split of k (the split is what uses the scratch), one to three token tiles
SHAPES = [(8, 1536, 8960), (32, 1536, 8960), (1, 2048, 1536), (20, 1536, 1536), (64, 389, 96), (3, 32000, 512)]


@pytest.mark.parametrize("shape", SHAPES)
def test_static_scratch_entry_point_matches_the_ordinary_one(shape):
    from litinfer_b200 import kernels as K

    lib = K.library()
    M, N, Kd = shape
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(sum(shape))
    a = torch.randn(M, Kd, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    bias = torch.randn(N, generator=g).to(dev)
    for out_dtype, b in ((torch.bfloat16, None), (torch.float32, bias)):
        ref = torch.empty(M, N, dtype=out_dtype, device=dev)
        K.linear_with("gemv", a, w, b, ref)
        plain = torch.empty(M, N, dtype=torch.float32, device=dev)
        R.linear(a, w, b, plain)                   # the product in float32 on the same bfloat16 operands
        # two calls in a row: the second finds the scratch as the first left it
        for call in range(2):
            out = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
            rc, msg = _call_static(lib, a, w, b, out)
            assert rc == 0, msg
            torch.cuda.synchronize()
            scale = float(ref.float().abs().max())
            tol = 2.0 ** -7 * scale if out_dtype == torch.bfloat16 else 1e-5 * (Kd ** 0.5) * max(scale, 1.0)
            err = float((out.float() - ref.float()).abs().max())
            assert err <= tol, f"call {call}, {shape}, {out_dtype}: max |diff| {err:.3e} > {tol:.3e} against the ordinary kernel"
            err = float((out.float() - plain).abs().max())
            assert err <= tol, f"call {call}, {shape}, {out_dtype}: max |diff| {err:.3e} > {tol:.3e} against the plain product"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from litinfer_b200 import kernels as K

    lib = K.library()
    dev = torch.device("cuda:0")
    M, N, Kd = 64, 1536, 8960                      # 96 tiles x 4 splits x 64 tokens: more partial sums than the built-in scratch holds
    a = torch.zeros(M, Kd, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(N, Kd, dtype=torch.bfloat16, device=dev)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    rc, msg = _call_static(lib, a, w, None, out)
    assert rc != 0 and "built-in scratch" in msg
    rc, msg = _call_static(lib, a[:, :4].contiguous(), w[:, :4].contiguous(), None, out)
    assert rc != 0 and "multiple of 8" in msg
