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
#include "row_scale.cuh"

int li_linear_simt(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N, int K,
                   cudaStream_t stream);
int li_linear_gemv_bf16(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                        int epilogue, cudaStream_t stream, const RowScale& rs);
int li_linear_gemv_bf16_add_scaled(const void* a, const void* w, const float* bias, int M, int N, int K, const AddScaled& add,
                                   cudaStream_t stream);
int li_gemv_bf16_tiles(int N);
bool li_gemv_bf16_accepts(int M, int N, int K);
int li_linear_tcgen05(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                      int epilogue, cudaStream_t stream);
bool li_tcgen05_accepts(const void* a, const void* w, const void* out, int dtype_out, int M, int N, int K);
int li_linear_gemv_tcgen05(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                           int epilogue, cudaStream_t stream, const RowScale& rs);
int li_linear_gemv_tcgen05_add_scaled(const void* a, const void* w, const float* bias, int M, int N, int K, const AddScaled& add,
                                      cudaStream_t stream);
int li_gemv_tcgen05_tiles(int N);
bool li_gemv_tcgen05_accepts(const void* a, const void* w, int M, int N, int K);

namespace {

// Which of the two kernels for few rows (decode) takes a bfloat16 product: 0 neither, 1 the register-fed one
// (gemv_bf16.cu), 3 the tcgen05 kernel with swapped operands (gemv_tcgen05.cu); numbered as in li_linear_with.
// Wide matrices (at least 96 tiles of 128 rows: gate|up, lm_head) and narrow ones with a long k (down) stream best
// through TMA and the swapped tcgen05 kernel; narrow and short ones (q|k|v, o) would be cut into splits of two or
// three k-blocks there, which the register-fed kernel does with less latency.
int few_rows_kernel(const void* a, const void* w, const void* out, int M, int N, int K) {
    const bool aligned = ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0);
    if (!aligned || M > 64) return 0;
    const bool wide = (N + 127) / 128 >= 96;                   // fills the GPU without a split of k
    const bool long_k = (K + 63) / 64 >= 64;                   // a split of k leaves every CTA enough to stream (measured: down projection)
    if ((wide || long_k) && li_gemv_tcgen05_accepts(a, w, M, N, K)) return 3;
    if (li_gemv_bf16_accepts(M, N, K)) return 1;
    return 0;
}

int linear_impl(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N, int K,
                int epilogue, const RowScale& rs, cudaStream_t stream) {
    LI_REQUIRE(M >= 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    LI_REQUIRE(epilogue == LI_EPILOGUE_NONE || epilogue == LI_EPILOGUE_SWIGLU, "linear: unknown epilogue %d", epilogue);
    if (M == 0) return 0;
    if (dtype_in == LI_BF16) {
        const int few = few_rows_kernel(a, w, out, M, N, K);
        if (few == 3) return li_linear_gemv_tcgen05(a, w, bias, out, dtype_out, M, N, K, epilogue, stream, rs);
        if (few == 1) return li_linear_gemv_bf16(a, w, bias, out, dtype_out, M, N, K, epilogue, stream, rs);
        LI_REQUIRE(rs.ssq == nullptr, "linear: a factor per token exists in the kernels for at most 64 bfloat16 rows only (M=%d N=%d K=%d)", M, N, K);
        if (li_tcgen05_accepts(a, w, out, dtype_out, M, N, K)) return li_linear_tcgen05(a, w, bias, out, dtype_out, M, N, K, epilogue, stream);
    }
    LI_REQUIRE(rs.ssq == nullptr, "linear: a factor per token exists in the kernels for at most 64 bfloat16 rows only (M=%d N=%d K=%d)", M, N, K);
    LI_REQUIRE(epilogue == LI_EPILOGUE_NONE, "linear: the fused swiglu epilogue exists for bfloat16 with K a multiple of 8 only (M=%d N=%d K=%d)", M, N, K);
    return li_linear_simt(a, w, bias, out, dtype_in, dtype_out, M, N, K, stream);
}

}  // namespace

// epilogue LI_EPILOGUE_SWIGLU: w holds gate and up rows interleaved in groups of 8 (8 gate rows, the
// 8 up rows of the same outputs, ...); out is [M, N / 2] = up * gate / (1 + exp(-gate)).  bfloat16 only.
LI_EXPORT int li_linear(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N, int K,
                        int epilogue, cudaStream_t stream) {
    return linear_impl(a, w, bias, out, dtype_in, dtype_out, M, N, K, epilogue, RowScale{}, stream);
}

// The same with every token's row of a w^T multiplied by 1 / sqrt(sum of ssq[token, :] / width + eps) before bias
// and epilogue: the product after an RMSNorm whose weights are already in `a` (row_scale.cuh).
LI_EXPORT int li_linear_scaled_accepts(const void* a, const void* w, const void* out, int dtype_in, int M, int N, int K) {
    return (dtype_in == LI_BF16 && M >= 1 && few_rows_kernel(a, w, out, M, N, K) != 0) ? 1 : 0;
}

LI_EXPORT int li_linear_scaled(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N,
                               int K, int epilogue, const float* ssq, int nparts, int width, float eps, cudaStream_t stream) {
    LI_REQUIRE(ssq != nullptr && nparts >= 1 && width >= 1, "linear (scaled): needs the partial sums of squares");
    LI_REQUIRE(li_linear_scaled_accepts(a, w, out, dtype_in, M, N, K), "linear (scaled): refuses M=%d N=%d K=%d (bfloat16, at most 64 rows)", M, N, K);
    RowScale rs;
    rs.ssq = ssq;
    rs.nparts = nparts;
    rs.width = (float)width;
    rs.eps = eps;
    return linear_impl(a, w, bias, out, dtype_in, dtype_out, M, N, K, epilogue, rs, stream);
}

// x32[M, N] += a w^T (+ bias); hprime = bfloat16(norm_weight * x32); ssq_out[token, part] = sums of the new x32^2
// over the columns of each of the product's tiles.  li_linear_add_scaled_parts says how many parts that is for
// these sizes (0: no kernel takes them, the caller runs product, add and norm separately).
LI_EXPORT int li_linear_add_scaled_parts(const void* a, const void* w, const void* x32, const void* hprime, int dtype_in, int M, int N, int K) {
    if (dtype_in != LI_BF16 || M < 1 || (uintptr_t)x32 % 16 != 0) return 0;
    const int few = few_rows_kernel(a, w, hprime, M, N, K);
    return few == 3 ? li_gemv_tcgen05_tiles(N) : (few == 1 ? li_gemv_bf16_tiles(N) : 0);
}

LI_EXPORT int li_linear_add_scaled(const void* a, const void* w, const float* bias, float* x32, const float* norm_weight, void* hprime,
                                   float* ssq_out, int dtype_in, int M, int N, int K, cudaStream_t stream) {
    const int few = dtype_in == LI_BF16 ? few_rows_kernel(a, w, hprime, M, N, K) : 0;
    LI_REQUIRE(few != 0 && M >= 1, "linear + add: refuses M=%d N=%d K=%d (bfloat16, at most 64 rows)", M, N, K);
    LI_REQUIRE(x32 && norm_weight && hprime && ssq_out, "linear + add: null operand");
    AddScaled add;
    add.x32 = x32;
    add.norm_weight = norm_weight;
    add.hprime = (bf16*)hprime;
    add.ssq_out = ssq_out;
    if (few == 3) return li_linear_gemv_tcgen05_add_scaled(a, w, bias, M, N, K, add, stream);
    return li_linear_gemv_bf16_add_scaled(a, w, bias, M, N, K, add, stream);
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
        return li_linear_gemv_bf16(a, w, bias, out, dtype_out, M, N, K, epilogue, stream, RowScale{});
    }
    if (which == 2) {
        LI_REQUIRE(li_tcgen05_accepts(a, w, out, dtype_out, M, N, K), "linear: the tcgen05 kernel refuses M=%d N=%d K=%d (K must be a multiple of 8, pointers 16-byte aligned)", M, N, K);
        return li_linear_tcgen05(a, w, bias, out, dtype_out, M, N, K, epilogue, stream);
    }
    if (which == 3) {
        LI_REQUIRE(li_gemv_tcgen05_accepts(a, w, M, N, K), "linear: the swapped tcgen05 kernel refuses M=%d N=%d K=%d", M, N, K);
        return li_linear_gemv_tcgen05(a, w, bias, out, dtype_out, M, N, K, epilogue, stream, RowScale{});
    }
    return li_fail("linear: unknown implementation %d", which);
}
