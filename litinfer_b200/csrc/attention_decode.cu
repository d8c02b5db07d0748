// Decode attention in bfloat16: one new token per sequence over its paged
// cache, grouped-query.
//
// Two kernels share one inner step.  Few sequences: grid (split, kv head,
// sequence); a CTA of 8 warps covers 256 keys at fixed absolute positions
// [256 s, 256 s + 256), each warp 32 of them (all its loads are in flight at
// once: one round trip to memory).  Many sequences (sequences x kv heads >= 120):
// one CTA per (sequence, kv head) whose warps walk every 8th block of 32 keys;
// nothing to merge across CTAs.  Either way a warp works for all query heads of
// one key/value head at once (they share every K and V byte read; heads are the
// 16 rows of a tensor-core tile).  Per block a warp computes S = Q K^T and
// O += P V with mma.sync m16n8k16 (bfloat16 in, float accumulate), softmax
// online in float as in LitInfer's kernel (src/ops/paged_attention/op.cpp:194-234).
// All operands go from global memory straight into fragment registers with
// 16-byte loads (8-byte loads and blocks of 16 keys for head_dim 256, where
// registers are short):
//   * the sum over head_dim does not depend on its order, so the 8 consecutive
//     elements a thread loads from a q row and from a key row are used as the
//     element pairs the fragment layout asks for in two k-steps, the same way
//     on both sides;
//   * values are cached transposed, [page][kv_head][head_dim][slot], so that for
//     one output column the 8 consecutive keys a thread needs are contiguous;
//     the score tiles are computed with their key columns permuted to match.
// Warps are merged through shared memory, CTAs through a float workspace by the
// CTA that finishes last (a counter per sequence and kv head), both in fixed
// order: which keys a warp or a CTA takes depends on absolute key positions
// only, so a sequence's result does not depend on the batch it is in, as long
// as the same kernel runs (the choice depends on the number of sequences).
// Window: keys below p - window + 1 are masked, blocks wholly below it skipped.
//
// Requires head_dim in {16, 32, ..., 128, 256}, at most 16 query heads per
// key/value head, page_size a multiple of 16.
#include "attention_mma.cuh"

namespace {

constexpr int kWholeFrom = 120;        // (sequences x kv heads) from which a CTA takes a whole context
constexpr int kWarps = 8;

struct Workspace {
    float* buf = nullptr;
    size_t floats = 0;
    unsigned* counters = nullptr;
};
constexpr size_t kCounters = 1u << 20;
Workspace g_ws[16];

using namespace attn;

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

template <int DH, int KB>
__global__ void __launch_bounds__(kWarps * 32, 1)
decode_attention_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ ctx_lens,
                        const int* __restrict__ old_lens, const int* __restrict__ q_start, float* __restrict__ part,
                        unsigned* __restrict__ counters, bf16* __restrict__ out, int nh, int nkv, int page_size, int num_pages,
                        float scale, int window, int nsplit) {
    extern __shared__ float sm[];
    __shared__ int is_last;
    pdl_launch_dependents();
    constexpr int kSplit = KB * kWarps;                // one block of KB keys per warp: one round trip to memory
    const int split = blockIdx.x, kvh = blockIdx.y, s = blockIdx.z;
    const int ctx = ctx_lens[s];                       // the step's metadata is in place before its first kernel starts
    const int p = ctx - 1;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int k_begin = split * kSplit;
    const int k_end = min(ctx, k_begin + kSplit);
    // q_start (a step that also holds portions of prompts): the sequence's token is row q_start[s], and only the
    // sequences of one token are this kernel's; without it sequence s is row s
    const int tok = q_start ? q_start[s] : s;
    const bool mine = !q_start || q_start[s + 1] - tok == 1;
    if (!mine || k_begin >= ctx || k_end <= lo) {
        pdl_wait();                                    // a CTA leaves only after the kernel before it has finished: the chain of dependent kernels stays ordered
        return;
    }
    const int G = nh / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
    pdl_wait();
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
    __syncthreads();
    // partial layout per (sequence, head, split): DH floats of O, then m, l
    for (int e = threadIdx.x; e < G * DH; e += kWarps * 32) {
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
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(&counters[s * nkv + kvh], 1u);
        is_last = (prev == (unsigned)(last - first));
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // factors exp(m_split - M) and the denominators first (one round of loads), then the sums
    // over splits with eight loads in flight at a time
    const int nact = last - first + 1;
    float* f_sm = sm;                                  // [G][nact] factors; reuses the warp-merge buffer
    float* l_sm = sm + (size_t)G * nact;               // [G] denominators
    __syncthreads();
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
    __syncthreads();
    // the weighted sums: up to four outputs a thread at once, eight splits each, all their loads in flight together
    constexpr int E = 4;
    for (int e0 = threadIdx.x; e0 < G * DH; e0 += E * kWarps * 32) {
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
    if (threadIdx.x == 0) counters[s * nkv + kvh] = 0;          // ready for the next launch on this stream
}

// Many sequences at once: with one CTA per (sequence, kv head) the GPU is already full, and splitting the
// context over CTAs would only add partial results to write, merge and wait for.  Each of the CTA's warps
// walks every WARPS-th block of 16 keys with a running softmax; the warps are merged through shared memory in
// warp order at the end.  The assignment of blocks to warps depends on the sequence alone.
template <int DH, int WARPS, int KB>
__global__ void __launch_bounds__(WARPS * 32, 1)
decode_attention_whole_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                              const int* __restrict__ block_table, int max_blocks, const int* __restrict__ ctx_lens,
                              const int* __restrict__ q_start, bf16* __restrict__ out, int nh, int nkv, int page_size, int num_pages,
                              float scale, int window) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int kvh = blockIdx.x, s = blockIdx.y;
    const int tok = q_start ? q_start[s] : s;          // as in the kernel above
    if (q_start && q_start[s + 1] - tok != 1) return;
    const int ctx = ctx_lens[s];
    const int p = ctx - 1;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int G = nh / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const bf16* qrow = qkv + (size_t)tok * (nh + 2 * nkv) * DH + (size_t)kvh * G * DH;
    unsigned qa[DH / 16][4];
    const bf16* q_lo = g < G ? qrow + (size_t)g * DH : nullptr;
    const bf16* q_hi = g + 8 < G ? qrow + (size_t)(g + 8) * DH : nullptr;
    if constexpr (KB == 16) load_q<DH>(qa, q_lo, q_hi, t);
    else load_q32<DH>(qa, q_lo, q_hi, t);
    RowState<DH> st;
    st.init();
    const int lo2[2] = {lo, lo}, hi2[2] = {p, p};
    const int* bt = block_table + (size_t)s * max_blocks;
    const int b_first = lo / KB, b_last = p / KB;
#pragma unroll 1
    for (int b = b_first + warp; b <= b_last; b += WARPS)
        block_step<DH, KB>(st, qa, kcache, vcache, bt, b * KB, kvh, nkv, page_size, num_pages, lo2, hi2, scale, g, t);
    const float m0 = st.m[0], m1 = st.m[1];
    const float l0 = quad_sum(st.l[0]), l1 = quad_sum(st.l[1]);
    float* sm_m = sm;
    float* sm_l = sm + WARPS * 16;
    float* sm_o = sm + 2 * WARPS * 16;
    if (t == 0) {
        sm_m[warp * 16 + g] = m0; sm_m[warp * 16 + g + 8] = m1;
        sm_l[warp * 16 + g] = l0; sm_l[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int j = 0; j < DH / 8; ++j) {
        const int col = j * 8 + 2 * t;
        if (g < G) {
            sm_o[((size_t)warp * G + g) * DH + col] = st.o[j][0];
            sm_o[((size_t)warp * G + g) * DH + col + 1] = st.o[j][1];
        }
        if (g + 8 < G) {
            sm_o[((size_t)warp * G + g + 8) * DH + col] = st.o[j][2];
            sm_o[((size_t)warp * G + g + 8) * DH + col + 1] = st.o[j][3];
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < G * DH; e += WARPS * 32) {
        const int r = e / DH, d = e - r * DH;
        float M = sm_m[r];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
        float O = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = (sm_m[w * 16 + r] == -INFINITY) ? 0.0f : expf(sm_m[w * 16 + r] - M);
            O += sm_o[((size_t)w * G + r) * DH + d] * f;
            L += sm_l[w * 16 + r] * f;
        }
        out[((size_t)tok * nh + kvh * G + r) * DH + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
    }
}

int ensure_workspace(size_t floats, float** buf, unsigned** counters) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return li_fail("attention (decode): cudaGetDevice: %s", cudaGetErrorString(e));
    LI_REQUIRE(dev >= 0 && dev < 16, "attention (decode): device index %d out of range", dev);
    Workspace& w = g_ws[dev];
    if (w.floats < floats) {
        // grows on demand; the first call of a given size must come before stream capture.  The buffer that was
        // outgrown is kept until the process ends: a captured graph may still hold its address.
        size_t want = floats < (8u << 20) ? (8u << 20) : floats + floats / 2;
        float* nb = nullptr;
        e = cudaMalloc(&nb, want * sizeof(float));
        if (e != cudaSuccess) {
            return li_fail("attention (decode): cannot allocate %zu bytes of workspace: %s (a first call of this size inside a stream capture cannot allocate)",
                           want * sizeof(float), cudaGetErrorString(e));
        }
        w.buf = nb;
        w.floats = want;
    }
    if (!w.counters) {
        e = cudaMalloc(&w.counters, kCounters * sizeof(unsigned));
        if (e == cudaSuccess) e = cudaMemset(w.counters, 0, kCounters * sizeof(unsigned));
        if (e != cudaSuccess) return li_fail("attention (decode): cannot allocate the split counters: %s", cudaGetErrorString(e));
    }
    *buf = w.buf;
    *counters = w.counters;
    return 0;
}

template <int DH>
int launch(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
           const int* ctx_lens, const int* old_lens, const int* q_start, int S, int nh, int nkv, int page_size, int num_pages, float scale,
           int window, int max_ctx_len, cudaStream_t stream) {
    const int G = nh / nkv;
    LI_REQUIRE(S <= 65535 && nkv <= 65535, "attention (decode): batch %d or kv heads %d too large for one launch", S, nkv);
    if ((long long)S * nkv >= kWholeFrom) {
        // one CTA per (sequence, kv head) fills the GPU: no split of the context
        constexpr int W = 8, KB = DH <= 128 ? 32 : 16;
        const size_t wsmem = (2 * W * 16 + (size_t)W * G * DH) * sizeof(float);
        if (wsmem <= 200 * 1024) {
            static bool raised = false;
            if (!raised && wsmem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(decode_attention_whole_kernel<DH, W, KB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
                if (e != cudaSuccess) return li_fail("attention (decode): cannot raise shared memory: %s", cudaGetErrorString(e));
                raised = true;
            }
            li_launch_pdl(decode_attention_whole_kernel<DH, W, KB>, dim3(nkv, S), dim3(W * 32), wsmem, stream, (const bf16*)qkv, (const bf16*)kcache,
                          (const bf16*)vcache, block_table, max_blocks, ctx_lens, q_start, (bf16*)out, nh, nkv, page_size, num_pages, scale, window);
            return li_check_launch("attention (decode, whole context)");
        }
    }
    constexpr int KBS = DH <= 128 ? 32 : 16;
    constexpr int kSplit = KBS * kWarps;
    const int nsplit = ceil_div(max_ctx_len > 0 ? max_ctx_len : 1, kSplit);
    float* part = nullptr;
    unsigned* counters = nullptr;
    if (int rc = ensure_workspace((size_t)S * nh * nsplit * (DH + 2), &part, &counters)) return rc;
    LI_REQUIRE((size_t)S * nkv <= kCounters, "attention (decode): batch %d x %d kv heads exceeds the split counters", S, nkv);
    size_t smem_floats = 2 * kWarps * 16 + (size_t)kWarps * G * DH;
    if (smem_floats < (size_t)G * (nsplit + 1)) smem_floats = (size_t)G * (nsplit + 1);      // the final merge reuses the buffer
    const size_t smem = smem_floats * sizeof(float);
    static bool attr_set = false;
    if (!attr_set && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<DH, KBS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return li_fail("attention (decode): cannot raise shared memory: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    LI_REQUIRE(smem <= 200 * 1024, "attention (decode): shared memory %zu too large", smem);
    LI_REQUIRE(S <= 65535 && nkv <= 65535, "attention (decode): batch %d or kv heads %d too large for one launch", S, nkv);
    dim3 grid(nsplit, nkv, S);
    li_launch_pdl(decode_attention_kernel<DH, KBS>, dim3(grid), dim3(kWarps * 32), smem, stream, (const bf16*)qkv, (const bf16*)kcache, (const bf16*)vcache,
                                                                      block_table, max_blocks, ctx_lens, old_lens, q_start, part, counters, (bf16*)out,
                                                                      nh, nkv, page_size, num_pages, scale, window, nsplit);
    return li_check_launch("attention (decode)");
}

}  // namespace

bool li_attention_decode_accepts(int nh, int nkv, int dh, int page_size) {
    const bool dh_ok = (dh % 16 == 0 && dh >= 16 && dh <= 128) || dh == 256;
    return dh_ok && nh % nkv == 0 && nh / nkv <= 16 && page_size % 16 == 0;
}

int li_attention_decode(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                        const int* ctx_lens, const int* old_lens, const int* q_start, int S, int nh, int nkv, int dh, int page_size, int num_pages,
                        float scale, int window, int max_ctx_len, cudaStream_t stream) {
#define LI_CASE(D)                                                                                                             \
    case D:                                                                                                                    \
        return launch<D>(qkv, out, kcache, vcache, block_table, max_blocks, ctx_lens, old_lens, q_start, S, nh, nkv, page_size, num_pages, scale, \
                         window, max_ctx_len, stream);
    switch (dh) {
        LI_CASE(16) LI_CASE(32) LI_CASE(48) LI_CASE(64) LI_CASE(80) LI_CASE(96) LI_CASE(112) LI_CASE(128) LI_CASE(256)
        default:
            return li_fail("attention (decode): head_dim %d is not supported by this kernel", dh);
    }
#undef LI_CASE
}
