/* li_linear_gemv_static: the weight-streaming product for few rows, for callers
 * that may not allocate device memory.
 *
 * This entry point has no counterpart in LitInfer; it exists for users of this
 * library only.
 *
 * Who needs it: a host program that owns all device memory itself and forbids
 * cudaMalloc inside libraries (an inference server with a fixed arena, a plugin
 * loaded into another runtime) and code on a latency-critical path where an
 * allocation would synchronise the device.  The ordinary entry
 * point (li_linear) allocates a split-k workspace with cudaMalloc the first time
 * it runs on a device; this one never calls cudaMalloc, cudaFree or any other
 * allocating routine.
 *
 * Its scratch memory (float partial sums of the k-splits and one arrival counter
 * per 16-row tile) lives in two file-scope __device__ arrays of fixed size inside
 * the library: LI_STATIC_PARTIAL_FLOATS floats (1 MiB) and LI_STATIC_TILES
 * counters.  Every GPU that loads the library holds them until the process exits.
 * A product whose splits need more than that is refused with an error: for
 * instance N = 1536, K = 8960 splits k four ways and fits for up to 32 rows of a,
 * but not for 33 to 64.  Products that need no split (for instance N >= 23680)
 * never touch the scratch and have no such limit.
 *
 * The first call on a device looks up the arrays' device addresses
 * (cudaGetSymbolAddress, with that device current).  Make that first call before
 * any stream capture.  The look-up is guarded by a lock, so host threads may make
 * their first calls at the same time; the calls themselves are ordered by the
 * caller (next paragraph).
 *
 * All calls share the arrays, and the arrays keep what the last call left: each
 * call clears the counters it is going to use (an asynchronous memset on the
 * caller's stream) before its kernel runs.  Two calls that overlap on the GPU
 * (different streams, no ordering between them) race on the scratch and give
 * wrong results; order them.
 *
 * out[M, N] = a[M, K] w[N, K]^T (+ bias[N]); a, w bfloat16 row-major, 16-byte
 * aligned; bias float or NULL; out bfloat16 (dtype_out 1) or float (dtype_out 0);
 * 1 <= M <= 64; K a multiple of 8.  Returns 0, or non-zero with the text in
 * li_last_error().
 */
#pragma once

#include <cuda_runtime.h>

#define LI_STATIC_PARTIAL_FLOATS (1u << 18)
#define LI_STATIC_TILES 1024

#ifdef __cplusplus
extern "C" {
#endif

int li_linear_gemv_static(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                          cudaStream_t stream);

#ifdef __cplusplus
}
#endif
