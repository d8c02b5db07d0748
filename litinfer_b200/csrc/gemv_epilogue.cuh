// Epilogues of the weight-streaming products for few rows (gemv_bf16.cu, and the fused decode step that runs the
// same products from shared memory): what happens to the reduced 16 x (8 NT) tile of a product.  ``get(e)`` returns the
// reduced element e = (j * 4 + i) * 32 + lane, which stands for weight row g + 8 (i >> 1) of the tile and token
// j * 8 + 2 t + (i & 1) with g = lane >> 2, t = lane & 3 (the accumulator layout of mma.sync m16n8k16).  ``tid`` is the
// calling thread's index among the ``nthreads`` threads that take part; ``sync`` a barrier among exactly those.
#pragma once

#include "common.cuh"
#include "row_scale.cuh"

// Third epilogue: the product is the fused q|k|v projection and its epilogue is the rotary position
// encoding plus the write of k and v into the paged cache (what rope.cu does as a kernel of its own).
// For that the 16 rows of a tile are rows j .. j + 7 and j + head_dim / 2 .. j + head_dim / 2 + 7 of one
// head: the two halves of a rotation pair end up as the element and its partner 64 places on.
struct RopeArgs {
    const int* positions;
    const float* denom;
    const int* slot_mapping;
    bf16* kcache;
    bf16* vcache;
    int nh, nkv, dh, page_size, num_pages, write;
};

template <int NT, typename Get>
__device__ __forceinline__ void store_rope(Get get, const float* __restrict__ bias, bf16* __restrict__ out, int tile, int M, int N,
                                           const RopeArgs& ra, int tid, int nthreads, const float* rs_sm) {
    const int tiles_per_head = ra.dh >> 4, half = ra.dh >> 1;
    const int head = tile / tiles_per_head, jt = tile - head * tiles_per_head;
    for (int q = tid; q < NT * 64; q += nthreads) {
        const int l = q & 31, i = (q >> 5) & 1, j = q >> 6;
        const int e = (j * 4 + i) * 32 + l;
        const int tok = j * 8 + ((l & 3) << 1) + i;
        if (tok >= M) continue;
        const int jj = jt * 8 + (l >> 2);                       // index of the pair within the head
        const int r0 = head * ra.dh + jj, r1 = r0 + half;
        float x0 = get(e), x1 = get(e + 64);
        if (rs_sm) {
            x0 *= rs_sm[tok];
            x1 *= rs_sm[tok];
        }
        if (bias) {
            x0 += bias[r0];
            x1 += bias[r1];
        }
        float y0 = x0, y1 = x1;
        if (head < ra.nh + ra.nkv) {
            float sn, cs;
            sincosf((float)ra.positions[tok] / ra.denom[jj], &sn, &cs);
            // q and k are rounded to bfloat16 by the projection before they are rotated, as in the unfused path
            x0 = __bfloat162float(__float2bfloat16_rn(x0));
            x1 = __bfloat162float(__float2bfloat16_rn(x1));
            y0 = x0 * cs - x1 * sn;
            y1 = x1 * cs + x0 * sn;
        }
        if (head < ra.nh) {
            out[(size_t)tok * N + r0] = __float2bfloat16_rn(y0);
            out[(size_t)tok * N + r1] = __float2bfloat16_rn(y1);
        } else if (ra.write) {
            const int slot = ra.slot_mapping[tok];
            const int page = slot / ra.page_size, off = slot - page * ra.page_size;
            if (slot < 0 || page >= ra.num_pages) continue;        // validated on the host; never write outside the cache
            if (head < ra.nh + ra.nkv) {
                const int kvh = head - ra.nh;
                bf16* dst = ra.kcache + (((size_t)page * ra.nkv + kvh) * ra.page_size + off) * ra.dh;
                dst[jj] = __float2bfloat16_rn(y0);
                dst[jj + half] = __float2bfloat16_rn(y1);
            } else {
                const int kvh = head - ra.nh - ra.nkv;
                bf16* dst = ra.vcache + ((size_t)page * ra.nkv + kvh) * ra.dh * ra.page_size + off;      // values are cached transposed
                dst[(size_t)jj * ra.page_size] = __float2bfloat16_rn(y0);
                dst[(size_t)(jj + half) * ra.page_size] = __float2bfloat16_rn(y1);
            }
        }
    }
}

// Epilogue of one reduced element.  e = (j * 4 + i) * 32 + lane stands for weight row
// n0 + g + 8 (i >> 1) and token j * 8 + 2 t + (i & 1) with g = lane >> 2, t = lane & 3.
// kSwiglu: the weight rows of a tile are 8 gate rows followed by the 8 up rows of the same
// outputs; the element and its partner 64 places further on give one activation
// up * gate / (1 + exp(-gate)) (src/ops/swiglu/op.cpp:17-23), stored at column n0 / 2 + g.
template <int NT, typename Tout, bool kSwiglu, typename Get>
__device__ __forceinline__ void store_elements(Get get, const float* __restrict__ bias, Tout* __restrict__ out, int n0, int M, int N,
                                               int tid, int nthreads, const float* rs_sm) {
    // rs_sm: a factor per token (the reciprocal root of an RMSNorm whose weights are already in the input), or nullptr
    if (!kSwiglu) {
        for (int e = tid; e < NT * 128; e += nthreads) {
            float v = get(e);
            const int l = e & 31, ji = e >> 5, i = ji & 3, j = ji >> 2;
            const int row = n0 + (l >> 2) + ((i >> 1) << 3), tok = j * 8 + ((l & 3) << 1) + (i & 1);
            if (rs_sm) v *= rs_sm[tok];
            if (row < N && tok < M) out[(size_t)tok * N + row] = from_float<Tout>(bias ? v + bias[row] : v);
        }
    } else {
        const int half_n = N >> 1;
        for (int q = tid; q < NT * 64; q += nthreads) {
            const int l = q & 31, i = (q >> 5) & 1, j = q >> 6;
            const int e = (j * 4 + i) * 32 + l;
            float gate = get(e), up = get(e + 64);
            const int col = (n0 >> 1) + (l >> 2), tok = j * 8 + ((l & 3) << 1) + i;
            if (rs_sm) {
                gate *= rs_sm[tok];
                up *= rs_sm[tok];
            }
            if (col < half_n && tok < M) out[(size_t)tok * half_n + col] = from_float<Tout>(swiglu_of<Tout>(gate, up));
        }
    }
}

// Fourth epilogue (row_scale.cuh): the product is added to the float32 residual stream, this CTA's 16 columns of
// it; the sums also leave as bfloat16(norm_weight * x) for the next product, with their squares added up per token.
// xpre: the stream's old values of this thread's elements, loaded while the weights were streaming.
template <int NT, int XP, typename Get, typename Sync>
__device__ __forceinline__ void store_add_scaled(Get get, const float* __restrict__ bias, const AddScaled& add, const float (&xpre)[XP],
                                                 int tile, int nparts, int M, int N, int tid, int nthreads, float* tile_sm, Sync sync) {
    const int n0 = tile * 16;
#pragma unroll
    for (int q = 0; q < XP; ++q) {
        const int e = tid + q * nthreads;
        if (e < NT * 128) {
            const int l = e & 31, ji = e >> 5, i = ji & 3, j = ji >> 2;
            const int r = (l >> 2) + ((i >> 1) << 3), row = n0 + r, tok = j * 8 + ((l & 3) << 1) + (i & 1);
            float x = 0.0f;
            if (row < N && tok < M) {
                const float v = get(e);
                x = xpre[q] + (bias ? v + bias[row] : v);
                __stcg(add.x32 + (size_t)tok * N + row, x);              // other CTAs own the rest of the line: past L1
                add.hprime[(size_t)tok * N + row] = __float2bfloat16_rn(add.norm_weight[row] * x);
            }
            tile_sm[tok * 16 + r] = x;
        }
    }
    sync();
    for (int tok = tid; tok < M; tok += nthreads) {
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < 16; ++r) s += tile_sm[tok * 16 + r] * tile_sm[tok * 16 + r];
        add.ssq_out[(size_t)tok * nparts + tile] = s;
    }
}

