// Prefill attention in bfloat16: portions of prompts (any length, with or
// without history in the cache) over the paged cache, causal, grouped-query.
// Single tokens in the same batch are portions of length one.
//
// Grid (query head, tile of 64 tokens, sequence); a CTA has 4 warps, each owns
// 16 consecutive tokens of the portion for one head.  The keys and values the
// CTA needs are brought into shared memory in tiles of 64 keys with cp.async,
// two tiles in flight (the next one loads while the current one is used), and
// every warp takes its tensor-core fragments (mma.sync m16n8k16, bfloat16 in,
// float accumulate) from there with 16-byte loads:
//   * S = Q K^T sums over head_dim in any order: the 8 consecutive elements a
//     thread reads from a key row (and from its query row, read once from global
//     memory) serve two k-steps, the same permutation on both sides;
//   * O += P V sums over keys in any order: values are cached transposed
//     ([head_dim][slot]), a tile is stored as [head_dim][64 keys], the 8
//     consecutive keys a thread reads for an output column serve two k-steps,
//     and the score tiles carry their key columns in the matching order
//     (thread t of a quad owns keys 8t..8t+7 and 32+8t..32+8t+7 of the 64).
// Shared-memory rows are XOR-swizzled in 16-byte chunks so that the eight rows a
// load touches fall into different banks.  Softmax online in float as in
// LitInfer's kernel (src/ops/paged_attention/op.cpp:194-234).  The keys and
// values of the portion itself are already in the cache (the rope kernel ran
// before), so history and new tokens are read the same way, through the block
// table.  Token i of a portion of n tokens in a context of c sits at position
// p = c - n + i and sees keys max(0, p - window + 1) .. p.
//
// Requires head_dim in {16, 32, ..., 128, 256} and page_size a multiple of 16.
#include "attention_mma.cuh"

namespace {

using namespace attn;

constexpr int kWarps = 4;
constexpr int kTile = kWarps * 16;      // query rows per CTA
constexpr int kKeys = 64;               // keys per shared-memory tile

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// position of 16-byte chunk c of a row whose swizzle key is `key` (0..7), in a row of `chunks` chunks:
// XOR on the low three bits, inside complete groups of eight chunks only
__device__ __forceinline__ int swz(int c, int key, int chunks) { return ((c | 7) < chunks) ? (c ^ key) : c; }

// swizzle key of key row r of a tile.  A fragment load touches the rows base + {0, 1, 8, 9, 16, 17, 24, 25}: they get
// eight different keys, and the two rows that share a quarter-warp (r, r + 1) differ in bit 2, so that their four
// chunks each cover all eight 16-byte bank groups together.
__device__ __forceinline__ int k_row_key(int r) { return ((r & 1) << 2) | ((r >> 3) & 3); }

// the same for a row of the transposed value tile (one output column): a load touches columns 8 j + {0..7}
__device__ __forceinline__ int v_row_key(int col) { return ((col & 1) << 2) | ((col >> 1) & 3); }

// key (0..63 within the tile) behind column n of score tile tau: tiles 2s and 2s+1 feed k-step s of P V,
// where thread t of a quad holds keys K_s(t) .. K_s(t) + 3, K_s(t) = 8 t + 4 (s & 1) + 32 (s >> 1)
__device__ __forceinline__ int tile_key(int tau, int n) {
    const int s = tau >> 1, h = tau & 1;
    return 8 * (n >> 1) + 4 * (s & 1) + 32 * (s >> 1) + 2 * h + (n & 1);
}

template <int DH>
__global__ void __launch_bounds__(kWarps * 32, 2)
prefill_attention_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ out, const bf16* __restrict__ kcache,
                         const bf16* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                         const int* __restrict__ q_start, const int* __restrict__ ctx_lens, int nh, int nkv, int page_size,
                         int num_pages, float scale, int window, int skip_single) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int KCH = DH / 8;                     // 16-byte chunks in a key row
    constexpr int kKBytes = kKeys * DH * 2, kVBytes = DH * kKeys * 2;
    constexpr int F = DH / 32, R = (DH % 32) / 16;  // 32-wide groups of head_dim (16-byte fragment loads), 16-wide tail (8-byte loads)
    constexpr int KS = DH / 16, NT = DH / 8;

    const int s = blockIdx.z, h = blockIdx.x;
    const int tok0 = q_start[s], n = q_start[s + 1] - tok0;
    // the last tiles of a portion see the most keys: they are started first
    const int cta_i0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * kTile;       // CTAs start in the order x, y, z: all heads of the heaviest tile first
    if (cta_i0 >= n || (skip_single && n == 1)) return;          // skip_single: sequences of one token are another kernel's
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ctx = ctx_lens[s];
    const int kvh = h / (nh / nkv);
    const int row_elems = (nh + 2 * nkv) * DH;
    const int i0 = cta_i0 + warp * 16;                     // first token of this warp within the portion
    const bool warp_active = i0 < n;
    const int r_lo = i0 + g, r_hi = i0 + g + 8;

    // query fragments, permuted like the key fragments: group f gives k-steps 2f (elements 0-3 of the thread's 8) and 2f+1
    unsigned qa[KS][4];
    {
        const bf16* q0 = (warp_active && r_lo < n) ? qkv + (size_t)(tok0 + r_lo) * row_elems + (size_t)h * DH : nullptr;
        const bf16* q1 = (warp_active && r_hi < n) ? qkv + (size_t)(tok0 + r_hi) * row_elems + (size_t)h * DH : nullptr;
#pragma unroll
        for (int f = 0; f < F; ++f) {
            const uint4 a = q0 ? *reinterpret_cast<const uint4*>(q0 + f * 32 + t * 8) : make_uint4(0, 0, 0, 0);
            const uint4 b = q1 ? *reinterpret_cast<const uint4*>(q1 + f * 32 + t * 8) : make_uint4(0, 0, 0, 0);
            qa[2 * f][0] = a.x; qa[2 * f][1] = b.x; qa[2 * f][2] = a.y; qa[2 * f][3] = b.y;
            qa[2 * f + 1][0] = a.z; qa[2 * f + 1][1] = b.z; qa[2 * f + 1][2] = a.w; qa[2 * f + 1][3] = b.w;
        }
        if (R) {
            const uint2 a = q0 ? ld8(q0 + F * 32 + t * 4) : make_uint2(0, 0);
            const uint2 b = q1 ? ld8(q1 + F * 32 + t * 4) : make_uint2(0, 0);
            qa[KS - 1][0] = a.x; qa[KS - 1][1] = b.x; qa[KS - 1][2] = a.y; qa[KS - 1][3] = b.y;
        }
    }
    RowState<DH> st;
    st.init();
    int lo[2], hi[2];
    hi[0] = (warp_active && r_lo < n) ? ctx - n + r_lo : -1;
    hi[1] = (warp_active && r_hi < n) ? ctx - n + r_hi : -1;
    lo[0] = (window > 0 && hi[0] - window + 1 > 0) ? hi[0] - window + 1 : 0;
    lo[1] = (window > 0 && hi[1] - window + 1 > 0) ? hi[1] - window + 1 : 0;
    // what the CTA as a whole reads, and this warp's share of it
    const int cta_rows = min(kTile, n - cta_i0);
    const int cta_p_first = ctx - n + cta_i0, cta_p_last = cta_p_first + cta_rows - 1;
    const int cta_key_lo = (window > 0 && cta_p_first - window + 1 > 0) ? cta_p_first - window + 1 : 0;
    const int warp_p_first = ctx - n + i0;
    const int warp_p_last = warp_p_first + min(16, n - i0) - 1;
    const int warp_key_lo = (window > 0 && warp_p_first - window + 1 > 0) ? warp_p_first - window + 1 : 0;
    const int warp_lo_max = (window > 0 && warp_p_last - window + 1 > 0) ? warp_p_last - window + 1 : 0;     // the largest lower bound among the warp's rows
    const float scale_log2 = scale * 1.4426950408889634f;

    const int* bt = block_table + (size_t)s * max_blocks;
    auto page_of = [&](int key) {
        int idx = key / page_size;
        if (idx >= max_blocks) idx = max_blocks - 1;
        const int page = bt[idx];
        return (page < 0 || page >= num_pages) ? 0 : page;
    };
    auto load_tile = [&](int stage, int k0) {
        unsigned char* ks = smem + (size_t)stage * (kKBytes + kVBytes);
        unsigned char* vs = ks + kKBytes;
        // keys: 64 rows of DH elements
        for (int idx = threadIdx.x; idx < kKeys * KCH; idx += kWarps * 32) {
            const int r = idx / KCH, c = idx - r * KCH;
            const int key = k0 + r;
            const int page = page_of(key), off = key % page_size;
            cp_async16(ks + (size_t)r * (DH * 2) + swz(c, k_row_key(r), KCH) * 16,
                       kcache + (((size_t)page * nkv + kvh) * page_size + off) * DH + c * 8);
        }
        // values, transposed: DH rows of 64 keys; every 16 keys of a column are 32 contiguous bytes of a page
        for (int idx = threadIdx.x; idx < DH * 8; idx += kWarps * 32) {
            const int col = idx >> 3, c = idx & 7;
            const int key = k0 + (c >> 1) * 16;
            const int page = page_of(key), off = key % page_size;
            cp_async16(vs + (size_t)col * (kKeys * 2) + ((c ^ v_row_key(col)) * 16),
                       vcache + (((size_t)page * nkv + kvh) * DH + col) * page_size + off + (c & 1) * 8);
        }
    };

    const int k_first = (cta_key_lo / kKeys) * kKeys;
    load_tile(0, k_first);
    cp_async_commit();
    int stage = 0;
#pragma unroll 1
    for (int k0 = k_first; k0 <= cta_p_last; k0 += kKeys, stage ^= 1) {
        const bool more = k0 + kKeys <= cta_p_last;
        if (more) {
            load_tile(stage ^ 1, k0 + kKeys);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (warp_active && k0 <= warp_p_last && k0 + kKeys > warp_key_lo) {
            const unsigned char* ks = smem + (size_t)stage * (kKBytes + kVBytes);
            const unsigned char* vs = ks + kKBytes;
            // scores: 8 tiles of 8 keys
            float sc[8][4];
#pragma unroll
            for (int tau = 0; tau < 8; ++tau) {
                sc[tau][0] = sc[tau][1] = sc[tau][2] = sc[tau][3] = 0.0f;
                const int r = tile_key(tau, g);
                const unsigned char* krow = ks + (size_t)r * (DH * 2);
                const int key = k_row_key(r);
#pragma unroll
                for (int f = 0; f < F; ++f) {
                    const uint4 b = *reinterpret_cast<const uint4*>(krow + swz(f * 4 + t, key, KCH) * 16);
                    mma_bf16(sc[tau], qa[2 * f][0], qa[2 * f][1], qa[2 * f][2], qa[2 * f][3], b.x, b.y);
                    mma_bf16(sc[tau], qa[2 * f + 1][0], qa[2 * f + 1][1], qa[2 * f + 1][2], qa[2 * f + 1][3], b.z, b.w);
                }
                if (R) {
                    const uint2 b = *reinterpret_cast<const uint2*>(krow + swz(F * 4 + (t >> 1), key, KCH) * 16 + (t & 1) * 8);
                    mma_bf16(sc[tau], qa[KS - 1][0], qa[KS - 1][1], qa[KS - 1][2], qa[KS - 1][3], b.x, b.y);
                }
            }
            // mask (only tiles that touch the diagonal or the window's edge need one), online softmax over the 64
            // keys in base 2: exp(x scale - m) = 2^(x c - m'), c = scale log2(e), m' kept in the scaled units.
            // Rows g (index 0: c0, c1) and g + 8 (index 1: c2, c3).
            const bool interior = (k0 + kKeys - 1 <= warp_p_first) && (k0 >= warp_lo_max);
            float alpha[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float mx = -INFINITY;
                if (interior) {
#pragma unroll
                    for (int tau = 0; tau < 8; ++tau) mx = fmaxf(mx, fmaxf(sc[tau][2 * r], sc[tau][2 * r + 1]));
                } else {
#pragma unroll
                    for (int tau = 0; tau < 8; ++tau) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int key = k0 + tile_key(tau, 2 * t + e);
                            float& v = sc[tau][2 * r + e];
                            v = (key >= lo[r] && key <= hi[r]) ? v : -INFINITY;
                            mx = fmaxf(mx, v);
                        }
                    }
                }
                mx = quad_max(mx) * scale_log2;                  // scale > 0: the maximum commutes with the scaling
                const float mn = fmaxf(st.m[r], mx);
                const float ms = (mn == -INFINITY) ? 0.0f : mn;
                alpha[r] = fast_exp2(st.m[r] - ms);
                float sum = 0.0f;
#pragma unroll
                for (int tau = 0; tau < 8; ++tau) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        float& v = sc[tau][2 * r + e];
                        v = fast_exp2(fmaf(v, scale_log2, -ms));
                        sum += v;
                    }
                }
                st.l[r] = st.l[r] * alpha[r] + sum;
                st.m[r] = mn;
            }
            // P as A fragments of the four k-steps
            unsigned pa[4][4];
#pragma unroll
            for (int ks4 = 0; ks4 < 4; ++ks4) {
                pa[ks4][0] = pack_bf16(sc[2 * ks4][0], sc[2 * ks4][1]);
                pa[ks4][1] = pack_bf16(sc[2 * ks4][2], sc[2 * ks4][3]);
                pa[ks4][2] = pack_bf16(sc[2 * ks4 + 1][0], sc[2 * ks4 + 1][1]);
                pa[ks4][3] = pack_bf16(sc[2 * ks4 + 1][2], sc[2 * ks4 + 1][3]);
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int col = j * 8 + g;
                const unsigned char* vrow = vs + (size_t)col * (kKeys * 2);
                const uint4 v0 = *reinterpret_cast<const uint4*>(vrow + ((t ^ v_row_key(col)) * 16));          // keys 8t .. 8t+7
                const uint4 v1 = *reinterpret_cast<const uint4*>(vrow + (((t + 4) ^ v_row_key(col)) * 16));    // keys 32+8t .. 32+8t+7
                st.o[j][0] *= alpha[0]; st.o[j][1] *= alpha[0]; st.o[j][2] *= alpha[1]; st.o[j][3] *= alpha[1];
                mma_bf16(st.o[j], pa[0][0], pa[0][1], pa[0][2], pa[0][3], v0.x, v0.y);
                mma_bf16(st.o[j], pa[1][0], pa[1][1], pa[1][2], pa[1][3], v0.z, v0.w);
                mma_bf16(st.o[j], pa[2][0], pa[2][1], pa[2][2], pa[2][3], v1.x, v1.y);
                mma_bf16(st.o[j], pa[3][0], pa[3][1], pa[3][2], pa[3][3], v1.z, v1.w);
            }
        }
        __syncthreads();          // the stage is overwritten by the load the next iteration issues
    }
    if (!warp_active) return;
    const float l0 = quad_sum(st.l[0]), l1 = quad_sum(st.l[1]);
    const float inv0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, inv1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
    bf16* o_lo = out + (size_t)(tok0 + r_lo) * nh * DH + (size_t)h * DH;
    bf16* o_hi = out + (size_t)(tok0 + r_hi) * nh * DH + (size_t)h * DH;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int col = j * 8 + 2 * t;
        if (r_lo < n) *reinterpret_cast<unsigned*>(o_lo + col) = pack_bf16(st.o[j][0] * inv0, st.o[j][1] * inv0);
        if (r_hi < n) *reinterpret_cast<unsigned*>(o_hi + col) = pack_bf16(st.o[j][2] * inv1, st.o[j][3] * inv1);
    }
}

template <int DH>
int launch(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
           const int* q_start, const int* ctx_lens, int S, int nh, int nkv, int page_size, int num_pages, float scale, int window,
           int max_q_len, int skip_single, cudaStream_t stream) {
    LI_REQUIRE(S <= 65535 && ceil_div(max_q_len > 0 ? max_q_len : 1, kTile) <= 65535, "attention (prefill): batch %d or portions of %d tokens too large for one launch", S, max_q_len);
    constexpr size_t smem = 2 * (size_t)(kKeys * DH * 2 + DH * kKeys * 2);
    static bool raised = false;
    if (!raised && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return li_fail("attention (prefill): cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    dim3 grid(nh, ceil_div(max_q_len > 0 ? max_q_len : 1, kTile), S);
    prefill_attention_kernel<DH><<<grid, kWarps * 32, smem, stream>>>((const bf16*)qkv, (bf16*)out, (const bf16*)kcache,
                                                                      (const bf16*)vcache, block_table, max_blocks, q_start, ctx_lens,
                                                                      nh, nkv, page_size, num_pages, scale, window, skip_single);
    return li_check_launch("attention (prefill)");
}

}  // namespace

bool li_attention_prefill_accepts(int nh, int nkv, int dh, int page_size) {
    const bool dh_ok = (dh % 16 == 0 && dh >= 16 && dh <= 128) || dh == 256;
    return dh_ok && nh % nkv == 0 && page_size % 16 == 0;
}

int li_attention_prefill(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                         const int* q_start, const int* ctx_lens, int T, int S, int nh, int nkv, int dh, int page_size,
                         int num_pages, float scale, int window, int max_q_len, int skip_single, cudaStream_t stream) {
    (void)T;
    LI_REQUIRE(scale > 0.0f, "attention (prefill): the scale must be positive, got %g", (double)scale);
#define LI_CASE(D)                                                                                                                  \
    case D:                                                                                                                         \
        return launch<D>(qkv, out, kcache, vcache, block_table, max_blocks, q_start, ctx_lens, S, nh, nkv, page_size, num_pages, scale, \
                         window, max_q_len, skip_single, stream);
    switch (dh) {
        LI_CASE(16) LI_CASE(32) LI_CASE(48) LI_CASE(64) LI_CASE(80) LI_CASE(96) LI_CASE(112) LI_CASE(128) LI_CASE(256)
        default:
            return li_fail("attention (prefill): head_dim %d is not supported by this kernel", dh);
    }
#undef LI_CASE
}
