// li_linear: out[M, N] = a[M, K] w[N, K]^T (+ bias[N]), chosen by dtype and size.
//
//   float32            -> CUDA-core kernel (gemm_simt.cu), always: a true 32-bit product
//   bfloat16, M <= 64  -> decode is bound by reading every weight once: wide matrices go to
//                         the tcgen05 kernel with swapped operands (gemv_tcgen05.cu), narrow
//                         ones to the register-fed weight-streaming kernel (gemv_bf16.cu)
//   bfloat16, larger M -> tcgen05 kernel with TMA-fed operands and the accumulator
//                         in tensor memory (gemm_tcgen05.cu), when the sizes meet its
//                         alignment rules (K a multiple of 8 elements = 16 bytes per row)
//   otherwise          -> CUDA-core kernel
#include "common.cuh"

int li_linear_simt(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N, int K,
                   cudaStream_t stream);
int li_linear_gemv_bf16(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                        int epilogue, cudaStream_t stream);
bool li_gemv_bf16_accepts(int M, int N, int K);
int li_linear_tcgen05(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                      int epilogue, cudaStream_t stream);
bool li_tcgen05_accepts(const void* a, const void* w, const void* out, int dtype_out, int M, int N, int K);
int li_linear_gemv_tcgen05(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                           int epilogue, cudaStream_t stream);
bool li_gemv_tcgen05_accepts(const void* a, const void* w, int M, int N, int K);

// epilogue LI_EPILOGUE_SWIGLU: w holds gate and up rows interleaved in groups of 8 (8 gate rows, the
// 8 up rows of the same outputs, ...); out is [M, N / 2] = up * gate / (1 + exp(-gate)).  bfloat16 only.
LI_EXPORT int li_linear(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N, int K,
                        int epilogue, cudaStream_t stream) {
    LI_REQUIRE(M >= 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    LI_REQUIRE(epilogue == LI_EPILOGUE_NONE || epilogue == LI_EPILOGUE_SWIGLU, "linear: unknown epilogue %d", epilogue);
    if (M == 0) return 0;
    if (dtype_in == LI_BF16) {
        const bool aligned = ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0);
        // few rows (decode): wide matrices (at least 96 tiles of 128 rows: gate|up, lm_head) and narrow ones with a long k
        // (down) stream best through TMA and the swapped tcgen05 kernel; narrow and short ones (q|k|v, o) would be cut into
        // splits of two or three k-blocks there, which the register-fed kernel does with less latency
        const bool wide = (N + 127) / 128 >= 96;                   // fills the GPU without a split of k
        const bool long_k = (K + 63) / 64 >= 64 && M <= 32;        // a split of k leaves every CTA enough to stream (measured: down projection)
        if (aligned && M <= 64 && (wide || long_k) && li_gemv_tcgen05_accepts(a, w, M, N, K))
            return li_linear_gemv_tcgen05(a, w, bias, out, dtype_out, M, N, K, epilogue, stream);
        if (aligned && li_gemv_bf16_accepts(M, N, K)) return li_linear_gemv_bf16(a, w, bias, out, dtype_out, M, N, K, epilogue, stream);
        if (li_tcgen05_accepts(a, w, out, dtype_out, M, N, K)) return li_linear_tcgen05(a, w, bias, out, dtype_out, M, N, K, epilogue, stream);
    }
    LI_REQUIRE(epilogue == LI_EPILOGUE_NONE, "linear: the fused swiglu epilogue exists for bfloat16 with K a multiple of 8 only (M=%d N=%d K=%d)", M, N, K);
    return li_linear_simt(a, w, bias, out, dtype_in, dtype_out, M, N, K, stream);
}

// Force one implementation, for tests of each kernel alone: 0 simt, 1 gemv, 2 tcgen05, 3 tcgen05 with swapped operands (few rows).
LI_EXPORT int li_linear_with(int which, const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M,
                             int N, int K, int epilogue, cudaStream_t stream) {
    LI_REQUIRE(M > 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    if (which == 0) {
        LI_REQUIRE(epilogue == LI_EPILOGUE_NONE, "linear: the CUDA-core kernel has no fused epilogue");
        return li_linear_simt(a, w, bias, out, dtype_in, dtype_out, M, N, K, stream);
    }
    LI_REQUIRE(dtype_in == LI_BF16, "linear: implementation %d takes bfloat16 input only", which);
    if (which == 1) {
        LI_REQUIRE(li_gemv_bf16_accepts(M, N, K), "linear: the weight-streaming kernel refuses M=%d N=%d K=%d", M, N, K);
        return li_linear_gemv_bf16(a, w, bias, out, dtype_out, M, N, K, epilogue, stream);
    }
    if (which == 2) {
        LI_REQUIRE(li_tcgen05_accepts(a, w, out, dtype_out, M, N, K), "linear: the tcgen05 kernel refuses M=%d N=%d K=%d (K must be a multiple of 8, pointers 16-byte aligned)", M, N, K);
        return li_linear_tcgen05(a, w, bias, out, dtype_out, M, N, K, epilogue, stream);
    }
    if (which == 3) {
        LI_REQUIRE(li_gemv_tcgen05_accepts(a, w, M, N, K), "linear: the swapped tcgen05 kernel refuses M=%d N=%d K=%d", M, N, K);
        return li_linear_gemv_tcgen05(a, w, bias, out, dtype_out, M, N, K, epilogue, stream);
    }
    return li_fail("linear: unknown implementation %d", which);
}
