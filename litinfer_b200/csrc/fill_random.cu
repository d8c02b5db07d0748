// Random weights on the device: out[i] = mean + std * n_i with n_i standard normal, a pure function of
// (key, i), so that a tensor's values depend on nothing but its key (made of the seed and the tensor's name
// on the host) and that the host can restate them bit for bit.
//
// Generator: counter-based.  Pair p = i / 2 draws 64 bits z = mix(key + (p + 1) * 0x9E3779B97F4A7C15) with the
// finaliser of splitmix64; u1 = (top 24 bits + 1) / 2^24 in (0, 1], the next 24 bits give the angle
// 2 pi j / 2^24; Box-Muller: r = sqrt(-2 ln u1), elements 2p and 2p + 1 are r cos and r sin of the angle.
// Logarithm, sine and cosine are short series in float32 built from additions, multiplications and
// divisions only, each rounded on its own (never fused), and the square root is the correctly rounded one:
// every step is an IEEE operation with one possible result, so NumPy on a CPU gives the same bits
// (litinfer_b200/weights/random_init.py holds that restatement).  Errors of the series are below 1e-7.
// LitInfer has no random-weights mode (python/llaisys/models/qwen2.py:25-208 loads files only).
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// ln(k / 2^24) for k in [1, 2^24]: k = m 2^e with m in [1, 2); ln m = 2 (t + t^3/3 + ... + t^11/11), t = (m - 1) / (m + 1)
__device__ __forceinline__ float ln_u24(unsigned k) {
    const int e = 31 - __clz(k);
    const float m = __fmul_rn((float)k, __uint_as_float((unsigned)(127 - e) << 23));       // exact: a power of two
    const float t = __fdiv_rn(__fadd_rn(m, -1.0f), __fadd_rn(m, 1.0f));
    const float t2 = __fmul_rn(t, t);
    float s = 1.0f / 11.0f;
    s = __fadd_rn(__fmul_rn(s, t2), 1.0f / 9.0f);
    s = __fadd_rn(__fmul_rn(s, t2), 1.0f / 7.0f);
    s = __fadd_rn(__fmul_rn(s, t2), 1.0f / 5.0f);
    s = __fadd_rn(__fmul_rn(s, t2), 1.0f / 3.0f);
    s = __fadd_rn(__fmul_rn(s, t2), 1.0f);
    const float lnm = __fmul_rn(__fmul_rn(2.0f, t), s);
    return __fadd_rn(__fmul_rn((float)(e - 24), 0.693147180559945309f), lnm);
}

// cos and sin of 2 pi j / 2^24: the top two bits of j pick the quadrant, the rest an angle in [0, pi/2)
__device__ __forceinline__ void sincos_u24(unsigned j, float* sn, float* cs) {
    const unsigned q = j >> 22;
    const float th = __fmul_rn(__fmul_rn((float)(j & 0x3FFFFFu), 1.0f / 4194304.0f), 1.57079632679489662f);
    const float x2 = __fmul_rn(th, th);
    float s = -1.0f / 39916800.0f;
    s = __fadd_rn(__fmul_rn(s, x2), 1.0f / 362880.0f);
    s = __fadd_rn(__fmul_rn(s, x2), -1.0f / 5040.0f);
    s = __fadd_rn(__fmul_rn(s, x2), 1.0f / 120.0f);
    s = __fadd_rn(__fmul_rn(s, x2), -1.0f / 6.0f);
    s = __fadd_rn(__fmul_rn(s, x2), 1.0f);
    s = __fmul_rn(s, th);
    float c = 1.0f / 479001600.0f;
    c = __fadd_rn(__fmul_rn(c, x2), -1.0f / 3628800.0f);
    c = __fadd_rn(__fmul_rn(c, x2), 1.0f / 40320.0f);
    c = __fadd_rn(__fmul_rn(c, x2), -1.0f / 720.0f);
    c = __fadd_rn(__fmul_rn(c, x2), 1.0f / 24.0f);
    c = __fadd_rn(__fmul_rn(c, x2), -0.5f);
    c = __fadd_rn(__fmul_rn(c, x2), 1.0f);
    *cs = q == 0 ? c : (q == 1 ? -s : (q == 2 ? -c : s));
    *sn = q == 0 ? s : (q == 1 ? c : (q == 2 ? -s : -c));
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long long n, unsigned long long key, float mean, float std) {
    const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (2 * p >= n) return;
    const unsigned long long z = mix64(key + (unsigned long long)(p + 1) * 0x9E3779B97F4A7C15ull);
    const unsigned k = (unsigned)(z >> 40) + 1u, j = (unsigned)(z >> 16) & 0xFFFFFFu;
    const float r = __fsqrt_rn(__fmul_rn(-2.0f, ln_u24(k)));
    float sn, cs;
    sincos_u24(j, &sn, &cs);
    out[2 * p] = from_float<T>(__fadd_rn(mean, __fmul_rn(std, __fmul_rn(r, cs))));
    if (2 * p + 1 < n) out[2 * p + 1] = from_float<T>(__fadd_rn(mean, __fmul_rn(std, __fmul_rn(r, sn))));
}

__global__ void fill_randint_kernel(int* __restrict__ out, long long n, unsigned long long key, unsigned range) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned long long z = mix64(key + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull);
    out[i] = (int)((unsigned)(z >> 33) % range);
}

}  // namespace

// out[i] = mean + std * normal(key, i) over n elements of float32 or bfloat16 (rounded to nearest even).
LI_EXPORT int li_fill_normal(void* out, int dtype, long long n, unsigned long long key, float mean, float std, cudaStream_t stream) {
    LI_REQUIRE(n >= 0 && n <= (1LL << 40), "fill_normal: bad size %lld", n);
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "fill_normal: unknown dtype %d", dtype);
    if (n == 0) return 0;
    const long long pairs = (n + 1) / 2;
    const unsigned blocks = (unsigned)((pairs + 255) / 256);
    if (dtype == LI_F32) fill_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, key, mean, std);
    else fill_normal_kernel<bf16><<<blocks, 256, 0, stream>>>((bf16*)out, n, key, mean, std);
    return li_check_launch("fill_normal");
}

// out[i] = an integer in [0, range) from (key, i), for integer tables.
LI_EXPORT int li_fill_randint(int* out, long long n, unsigned long long key, int range, cudaStream_t stream) {
    LI_REQUIRE(n >= 0 && n <= (1LL << 40) && range >= 1, "fill_randint: bad size %lld or range %d", n, range);
    if (n == 0) return 0;
    fill_randint_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(out, n, key, (unsigned)range);
    return li_check_launch("fill_randint");
}
