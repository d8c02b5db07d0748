// Causal grouped-query attention of a ragged batch over the paged cache:
// the general kernel.  It serves the true 32-bit path for every batch shape
// and is the fall-back of the bfloat16 path for head sizes the tensor-core
// kernels refuse.
//
// One warp per (token, query head).  The token at position p of sequence s
// reads keys lo..p of s with lo = max(0, p - window + 1) (window 0: lo = 0),
// one key after the other in ascending order, with the online-softmax
// recurrence of LitInfer's kernel (src/ops/paged_attention/op.cpp:194-234):
//   m' = max(m, s_t); alpha = exp(m - m'); e = exp(s_t - m');
//   l = l alpha + e;  acc = acc alpha + e v_t;  out = acc / l.
// Scores, exponentials, sums and the weighted values are float.  The order of
// the keys and of the lanes' partial sums is fixed, so a token's output does
// not depend on what else is in the batch or on how its sequence was cut.
//
// Cache layout: keys [page][kv_head][offset][head_dim], values transposed
// [page][kv_head][head_dim][offset]; the page of key t of sequence s is
// block_table[s][t / page_size].  Any head_dim up to 512.
#include "common.cuh"

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxPerLane = 16;       // head_dim <= 512

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attention_generic_kernel(const T* __restrict__ qkv, T* __restrict__ out, const T* __restrict__ kcache, const T* __restrict__ vcache,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_of_token,
                         const int* __restrict__ positions, int total, int nh, int nkv, int dh, int page_size, int num_pages,
                         float scale, int window) {
    const int warp = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (warp >= total) return;
    const int t = warp / nh, h = warp - t * nh;
    const int kvh = h / (nh / nkv);
    const int s = seq_of_token[t];
    const int p = positions[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int row = (nh + 2 * nkv) * dh;
    const T* q = qkv + (size_t)t * row + h * dh;
    const int per = (dh + 31) >> 5;

    float qr[kMaxPerLane], acc[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        qr[i] = (i < per && d < dh) ? to_float(q[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const int* bt = block_table + (size_t)s * max_blocks;
    for (int key = lo; key <= p; ++key) {
        const int lb = key / page_size;
        int page = bt[lb];
        if (page < 0 || page >= num_pages) page = 0;      // host-validated; keep the read inside the cache
        const int off = key - lb * page_size;
        const size_t base = (((size_t)page * nkv + kvh) * page_size + off) * dh;
        const size_t vbase = ((size_t)page * nkv + kvh) * dh * page_size + off;
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            const int d = lane + 32 * i;
            if (i < per && d < dh) dot = fmaf(qr[i], to_float(kcache[base + d]), dot);
        }
        const float sc = warp_sum(dot) * scale;
        const float mn = fmaxf(m, sc);
        const float alpha = expf(m - mn);
        const float e = expf(sc - mn);
        l = l * alpha + e;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            const int d = lane + 32 * i;
            if (i < per && d < dh) acc[i] = acc[i] * alpha + e * to_float(vcache[vbase + (size_t)d * page_size]);
        }
        m = mn;
    }
    T* o = out + (size_t)t * nh * dh + h * dh;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        if (i < per && d < dh) o[d] = from_float<T>(acc[i] * inv);
    }
}

}  // namespace

int li_attention_generic(const void* qkv, void* out, const void* kcache, const void* vcache, int dtype, const int* block_table,
                         int max_blocks, const int* seq_of_token, const int* positions, int T, int nh, int nkv, int dh,
                         int page_size, int num_pages, float scale, int window, cudaStream_t stream) {
    LI_REQUIRE(dh <= 32 * kMaxPerLane, "attention: head_dim %d is larger than %d", dh, 32 * kMaxPerLane);
    const long long total = (long long)T * nh;
    LI_REQUIRE(total < (1LL << 31), "attention: too many (token, head) pairs");
    const int blocks = (int)ceil_div_ll(total, kWarpsPerBlock);
    if (dtype == LI_F32)
        attention_generic_kernel<float><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
            (const float*)qkv, (float*)out, (const float*)kcache, (const float*)vcache, block_table, max_blocks, seq_of_token, positions,
            (int)total, nh, nkv, dh, page_size, num_pages, scale, window);
    else if (dtype == LI_BF16)
        attention_generic_kernel<bf16><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
            (const bf16*)qkv, (bf16*)out, (const bf16*)kcache, (const bf16*)vcache, block_table, max_blocks, seq_of_token, positions,
            (int)total, nh, nkv, dh, page_size, num_pages, scale, window);
    else
        return li_fail("attention: unknown dtype %d", dtype);
    return li_check_launch("attention (generic)");
}
