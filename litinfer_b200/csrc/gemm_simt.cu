// out[M, N] = a[M, K] w[N, K]^T (+ bias[N]) on the CUDA cores: the matrix
// product of the true 32-bit path (no tensor-core mode that would round the
// operands), and of sizes the tensor-core kernels refuse.
//
// As LitInfer's linear (src/ops/linear/cpu/linear_cpu.cpp:45-60): both
// operands row-major with K contiguous, accumulation in float, bias added in
// float after the dot product, one rounding.  Each output element is summed by
// one thread over k = 0, 1, 2, ... in that order, whatever M is, so the value
// of a row does not depend on how many other rows are in the batch.
//
// Tile 64 x 64 x 16, 256 threads, 4 x 4 outputs a thread.  Any M, N, K >= 1.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename Tin, typename Tout>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const Tin* __restrict__ A, const Tin* __restrict__ W,
                                                         const float* __restrict__ bias, Tout* __restrict__ C, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid & 15, ty = tid >> 4;          // outputs: rows ty*4.., cols tx*4..
    const int lr = tid >> 2, lk = (tid & 3) * 4;     // loads: row lr, k offset lk..lk+3
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float av[4], wv[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int am = m0 + lr, wn = n0 + lr;
            av[q] = (am < M && k < K) ? to_float(A[(size_t)am * K + k]) : 0.0f;
            wv[q] = (wn < N && k < K) ? to_float(W[(size_t)wn * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            As[lk + q][lr] = av[q];
            Ws[lk + q][lr] = wv[q];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            C[(size_t)m * N + n] = from_float<Tout>(v);
        }
    }
}

}  // namespace

template <typename Tin, typename Tout>
static int launch(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream) {
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
    LI_REQUIRE(grid.y <= 65535, "linear: M=%d is too large for one launch", M);
    gemm_simt_kernel<Tin, Tout><<<grid, 256, 0, stream>>>((const Tin*)a, (const Tin*)w, bias, (Tout*)out, M, N, K);
    return li_check_launch("linear (simt)");
}

int li_linear_simt(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N, int K,
                   cudaStream_t stream) {
    if (dtype_in == LI_F32 && dtype_out == LI_F32) return launch<float, float>(a, w, bias, out, M, N, K, stream);
    if (dtype_in == LI_BF16 && dtype_out == LI_BF16) return launch<bf16, bf16>(a, w, bias, out, M, N, K, stream);
    if (dtype_in == LI_BF16 && dtype_out == LI_F32) return launch<bf16, float>(a, w, bias, out, M, N, K, stream);
    return li_fail("linear: unsupported dtypes in=%d out=%d", dtype_in, dtype_out);
}
