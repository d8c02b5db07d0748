// One unit of decode attention in bfloat16: the new token of sequence s against the keys [256 split, 256 split + 256)
// of its paged cache, for all query heads of key/value head kvh, by 8 warps (256 threads, ``tid`` 0..255; ``sync`` is a
// barrier among exactly them).  Used by the decode attention kernel (one unit per CTA) and by the fused decode step
// (units handed out to persistent CTAs).  ``wait_for_queries`` is called once by every thread, after the loads of keys
// and values that the step itself does not write have been issued and before anything the step writes is read: the
// kernel waits there for the kernel before it, the fused step for the grid-wide barrier behind the q|k|v product.
// ``sm``: shared scratch of max(2 * 8 * 16 + 8 * G * DH, G * (nsplit + 1)) floats; ``is_last``: a shared int.
#pragma once

#include "attention_mma.cuh"

namespace attn_decode {

using namespace attn;

constexpr int kWarps = 8;

__host__ __device__ inline void split_range(int ctx, int window, int kSplit, int* first, int* last) {
    const int p = ctx - 1;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    *first = lo / kSplit;
    *last = (ctx - 1) / kSplit;
}

// One block of KB keys (16: 8-byte loads; 32: 16-byte loads, half as many requests per byte) from the pages of a
// sequence into the running softmax of a warp.  All loads of the block are issued before the first use.
template <int DH, int KB>
__device__ __forceinline__ void block_step(RowState<DH>& st, const unsigned (&qa)[DH / 16][4], const bf16* __restrict__ kcache,
                                           const bf16* __restrict__ vcache, const int* __restrict__ bt, int key0, int kvh, int nkv,
                                           int page_size, int num_pages, const int (&lo2)[2], const int (&hi2)[2], float scale, int g, int t) {
    if constexpr (KB == 16) {
        int page = bt[key0 / page_size];
        if (page < 0 || page >= num_pages) page = 0;
        const int off = key0 % page_size;
        KFrag<DH> kf;
        VFrag<DH> vf;
        load_k<DH, true>(kf, kcache + (((size_t)page * nkv + kvh) * page_size + off) * DH, g, t);
        load_v<DH, true>(vf, vcache + ((size_t)page * nkv + kvh) * DH * page_size + off, page_size, g, t);
        compute16<DH>(st, qa, kf, vf, key0, lo2, hi2, scale, t);
    } else {
        // keys of this thread's key rows: the group of 8 at 8 (g >> 1); of its value columns: the 8 at 8 t.
        // A group of 8 aligned keys lies in one page (pages hold a multiple of 16); groups wholly past the
        // context may have no page yet: they read page 0 and are masked.
        const int kk = key0 + 8 * (g >> 1), vk = key0 + 8 * t;
        int kpage = kk <= hi2[0] ? bt[kk / page_size] : 0, vpage = vk <= hi2[0] ? bt[vk / page_size] : 0;
        if (kpage < 0 || kpage >= num_pages) kpage = 0;
        if (vpage < 0 || vpage >= num_pages) vpage = 0;
        KFrag32<DH> kf;
        VFrag32<DH> vf;
        load_k32<DH>(kf, kcache + (((size_t)kpage * nkv + kvh) * page_size + kk % page_size) * DH, g, t);
        load_v32<DH>(vf, vcache + ((size_t)vpage * nkv + kvh) * DH * page_size + vk % page_size, page_size, g);
        compute32<DH>(st, qa, kf, vf, key0, lo2, hi2, scale, t);
    }
}

// The two halves of block_step for blocks of 32 keys, so that the loads can be issued before the queries exist.
template <int DH>
__device__ __forceinline__ void block_load32(KFrag32<DH>& kf, VFrag32<DH>& vf, const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                                             const int* __restrict__ bt, int key0, int last_key, int kvh, int nkv, int page_size, int num_pages,
                                             int g, int t) {
    const int kk = key0 + 8 * (g >> 1), vk = key0 + 8 * t;
    int kpage = kk <= last_key ? bt[kk / page_size] : 0, vpage = vk <= last_key ? bt[vk / page_size] : 0;
    if (kpage < 0 || kpage >= num_pages) kpage = 0;
    if (vpage < 0 || vpage >= num_pages) vpage = 0;
    load_k32<DH>(kf, kcache + (((size_t)kpage * nkv + kvh) * page_size + kk % page_size) * DH, g, t);
    load_v32<DH>(vf, vcache + ((size_t)vpage * nkv + kvh) * DH * page_size + vk % page_size, page_size, g);
}

template <int DH, int KB, bool kCut = false, typename Sync, typename Wait>
__device__ __forceinline__ void decode_attention_unit(int split, int kvh, int s, int tid, const bf16* __restrict__ qkv, const bf16* __restrict__ kcache,
                                                      const bf16* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                                                      const int* __restrict__ ctx_lens, const int* __restrict__ old_lens,
                                                      const int* __restrict__ q_start, float* __restrict__ part, unsigned* __restrict__ counters,
                                                      bf16* __restrict__ out, int nh, int nkv, int page_size, int num_pages, float scale, int window,
                                                      int nsplit, float* sm, int* is_last, Sync sync, Wait wait_for_queries, int want = 0) {
    const int ctx = ctx_lens[s];                           // the step's metadata is in place before its first kernel starts
    // A unit covers KB keys per warp and round.  One round (one round trip to memory) where the units of all sequences
    // fit the GPU at once (want = 0).  Else the sequence's own context is cut into `want` units of as many rounds as that
    // takes, each warp walking every eighth block of its unit: the cut depends on the sequence and on `want` alone.
    // (kCut says at compile time whether that can be: the kernel of one round stays as lean as it was)
    const int rounds = (kCut && want > 0) ? max(1, ((ctx + KB * kWarps - 1) / (KB * kWarps) + want - 1) / want) : 1;
    const int kSplit = KB * kWarps * rounds;
    const int p = ctx - 1;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int k_begin = split * kSplit;
    const int k_end = min(ctx, k_begin + kSplit);
    // q_start (a step that also holds portions of prompts): the sequence's token is row q_start[s], and only the
    // sequences of one token are this kernel's; without it sequence s is row s
    const int tok = q_start ? q_start[s] : s;
    const bool mine = !q_start || q_start[s + 1] - tok == 1;
    if (!mine || k_begin >= ctx || k_end <= lo) {
        wait_for_queries();                            // every caller passes here exactly once, whatever it has to do
        return;
    }
    const int G = nh / nkv;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int* bt = block_table + (size_t)s * max_blocks;
    const int my_key0 = k_begin + warp * KB;
    const bool my_block = my_key0 < k_end && my_key0 + KB > lo;           // warp-uniform
    // The kernel before this one (the q|k|v product) writes the keys and values of the step's tokens: of position p
    // only, or, when several sequences of the step are tokens of one request, of the positions from old_lens[s] on.  A
    // warp whose block lies below them asks for its keys and values now, while that kernel is still running, and
    // waits afterwards.
    const int old = old_lens ? old_lens[s] : p;
    [[maybe_unused]] KFrag32<DH> kf_early;
    [[maybe_unused]] VFrag32<DH> vf_early;
    bool early = false;
    if constexpr (KB == 32) {
        early = my_block && my_key0 + KB <= old;
        if (early) block_load32<DH>(kf_early, vf_early, kcache, vcache, bt, my_key0, k_end - 1, kvh, nkv, page_size, num_pages, g, t);
    }
    wait_for_queries();
    // query fragments: rows g and g + 8 are heads kvh * G + g (+ 8)
    const bf16* qrow = qkv + (size_t)tok * (nh + 2 * nkv) * DH + (size_t)kvh * G * DH;
    unsigned qa[DH / 16][4];
    const bf16* q_lo = g < G ? qrow + (size_t)g * DH : nullptr;
    const bf16* q_hi = g + 8 < G ? qrow + (size_t)(g + 8) * DH : nullptr;
    if constexpr (KB == 16) load_q<DH>(qa, q_lo, q_hi, t);
    else load_q32<DH>(qa, q_lo, q_hi, t);
    RowState<DH> st;
    st.init();
    const int lo2[2] = {lo, lo}, hi2[2] = {k_end - 1, k_end - 1};
    if (my_block) {
        if constexpr (KB == 32) {
            if (!early) block_load32<DH>(kf_early, vf_early, kcache, vcache, bt, my_key0, k_end - 1, kvh, nkv, page_size, num_pages, g, t);
            compute32<DH>(st, qa, kf_early, vf_early, my_key0, lo2, hi2, scale, t);
        } else {
            block_step<DH, KB>(st, qa, kcache, vcache, bt, my_key0, kvh, nkv, page_size, num_pages, lo2, hi2, scale, g, t);
        }
    }
    if constexpr (kCut) {
#pragma unroll 1
        for (int rd = 1; rd < rounds; ++rd) {
            const int key0 = k_begin + (rd * kWarps + warp) * KB;
            if (key0 < k_end && key0 + KB > lo)            // warp-uniform
                block_step<DH, KB>(st, qa, kcache, vcache, bt, key0, kvh, nkv, page_size, num_pages, lo2, hi2, scale, g, t);
        }
    }
    const float m0 = st.m[0], m1 = st.m[1];
    const float l0 = quad_sum(st.l[0]), l1 = quad_sum(st.l[1]);
    auto& o = st.o;
    constexpr int NT = DH / 8;

    // merge the warps in fixed order: sm_m[w][16] | sm_l[w][16] | sm_o[w][G][DH]
    float* sm_m = sm;
    float* sm_l = sm + kWarps * 16;
    float* sm_o = sm + 2 * kWarps * 16;
    if (t == 0) {
        sm_m[warp * 16 + g] = m0; sm_m[warp * 16 + g + 8] = m1;
        sm_l[warp * 16 + g] = l0; sm_l[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int col = j * 8 + 2 * t;
        if (g < G) {
            sm_o[((size_t)warp * G + g) * DH + col] = o[j][0];
            sm_o[((size_t)warp * G + g) * DH + col + 1] = o[j][1];
        }
        if (g + 8 < G) {
            sm_o[((size_t)warp * G + g + 8) * DH + col] = o[j][2];
            sm_o[((size_t)warp * G + g + 8) * DH + col + 1] = o[j][3];
        }
    }
    sync();
    // partial layout per (sequence, head, split): DH floats of O, then m, l
    for (int e = tid; e < G * DH; e += kWarps * 32) {
        const int r = e / DH, d = e - r * DH;
        float M = sm_m[r];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
        float O = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float f = expf(sm_m[w * 16 + r] - M);
            O += sm_o[((size_t)w * G + r) * DH + d] * f;
            L += sm_l[w * 16 + r] * f;
        }
        float* dst = part + (((size_t)s * nh + kvh * G + r) * nsplit + split) * (DH + 2);
        dst[d] = O;
        if (d == 0) {
            dst[DH] = M;
            dst[DH + 1] = L;
        }
    }
    // the CTA that finishes last for this (sequence, kv head) merges the splits, in split order
    int first, last;
    split_range(ctx, window, kSplit, &first, &last);
    __threadfence();
    sync();
    if (tid == 0) {
        const unsigned prev = atomicAdd(&counters[s * nkv + kvh], 1u);
        *is_last = (prev == (unsigned)(last - first));
    }
    sync();
    if (!*is_last) return;
    __threadfence();
    // factors exp(m_split - M) and the denominators first (one round of loads), then the sums
    // over splits with eight loads in flight at a time
    const int nact = last - first + 1;
    float* f_sm = sm;                                  // [G][nact] factors; reuses the warp-merge buffer
    float* l_sm = sm + (size_t)G * nact;               // [G] denominators
    sync();
    for (int r = warp; r < G; r += kWarps) {
        // one warp per head: maxima and denominators of up to 32 splits per round of loads
        const float* base = part + ((size_t)s * nh + kvh * G + r) * nsplit * (DH + 2);
        float M = -INFINITY;
        for (int sp = first + lane; sp <= last; sp += 32) M = fmaxf(M, __ldcg(base + (size_t)sp * (DH + 2) + DH));
        M = warp_max(M);
        float L = 0.0f;
        for (int sp0 = first; sp0 <= last; sp0 += 32) {        // ascending split order within each lane
            const int sp = sp0 + lane;
            if (sp <= last) {
                const float m = __ldcg(base + (size_t)sp * (DH + 2) + DH), l = __ldcg(base + (size_t)sp * (DH + 2) + DH + 1);
                const float f = expf(m - M);
                f_sm[r * nact + sp - first] = f;
                L += l * f;
            }
        }
        L = warp_sum(L);
        if (lane == 0) l_sm[r] = L;
    }
    sync();
    // the weighted sums: up to four outputs a thread at once, eight splits each, all their loads in flight together
    constexpr int E = 4;
    for (int e0 = tid; e0 < G * DH; e0 += E * kWarps * 32) {
        const float* src[E];
        const float* fac[E];
        float O[E];
#pragma unroll
        for (int q = 0; q < E; ++q) {
            const int e = e0 + q * kWarps * 32;
            const int r = e < G * DH ? e / DH : 0, d = e < G * DH ? e - r * DH : 0;
            src[q] = part + ((size_t)s * nh + kvh * G + r) * nsplit * (DH + 2) + d;
            fac[q] = f_sm + r * nact;
            O[q] = 0.0f;
        }
        for (int i = 0; i < nact; i += 8) {
            float v[E][8];
#pragma unroll
            for (int q = 0; q < E; ++q)
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    v[q][u] = (i + u < nact && e0 + q * kWarps * 32 < G * DH) ? __ldcg(src[q] + (size_t)(first + i + u) * (DH + 2)) : 0.0f;
#pragma unroll
            for (int q = 0; q < E; ++q)
#pragma unroll
                for (int u = 0; u < 8; ++u) O[q] += (i + u < nact) ? v[q][u] * fac[q][i + u] : 0.0f;
        }
#pragma unroll
        for (int q = 0; q < E; ++q) {
            const int e = e0 + q * kWarps * 32;
            if (e < G * DH) {
                const int r = e / DH, d = e - r * DH;
                const float L = l_sm[r];
                out[((size_t)tok * nh + kvh * G + r) * DH + d] = __float2bfloat16_rn(L > 0.0f ? O[q] / L : 0.0f);
            }
        }
    }
    if (tid == 0) counters[s * nkv + kvh] = 0;          // ready for the next launch on this stream
}

}  // namespace attn_decode
