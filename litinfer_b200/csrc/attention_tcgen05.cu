// Prefill attention on the fifth-generation tensor cores: long portions of prompts over the paged cache,
// causal, grouped-query, bfloat16.
//
// Grid (query head, tile of 128 tokens, sequence).  A CTA of eleven warps works on 128 consecutive tokens of a
// portion for one head, against tiles of 128 keys:
//   warp 0     brings K of each tile into shared memory with TMA, up to three tiles ahead, page by page through the
//              block table, a lane per block of 16 keys: a block is 16 rows of the K operand ([keys, head_dim],
//              128-byte swizzle);
//   warp 10    the same for V: a block of values (cached transposed, [head_dim, 16 slots]) is the V operand of
//              one k-step ([head_dim, 16 keys], 32-byte swizzle);
//   warp 1     one thread issues the products with tcgen05.mma, accumulators in tensor memory:
//              S = Q K^T (128 x 128, two buffers) and O += P V (128 x head_dim), with Q and P as operands FROM
//              tensor memory: shared memory, whose bandwidth bounded the kernel when Q and P were read from it
//              as well, then carries K and V only;
//   warps 2-9  two threads per token, each with half of a tile's keys: they put the token's row of Q into tensor
//              memory once; per tile they read their part of the row of S, apply scale and mask, keep the
//              maximum (exchanged between the two) and sum of the online softmax in float
//              (src/ops/paged_attention/op.cpp:194-234), and write P as bfloat16 over the first half of that S
//              buffer.  O stays in tensor memory; it is scaled down only when a row's maximum has grown by more
//              than 2^8 (see kLazy).  S of tile j + 1 is issued before P V of tile j.
// Keys and values of the portion itself are already in the cache (the rope kernel ran before).  Token i of a
// portion of n tokens in a context of c sits at position p = c - n + i and sees keys max(0, p - window + 1) .. p.
// Keys of a tile that lie past the context are read from whatever page the table names (page 0 if none) and get
// probability zero; the cache holds finite numbers only.
//
// Every wait on a barrier is bounded; a wait that runs out raises the status word of the tcgen05 kernels and the
// CTA leaves, freeing its tensor memory.
//
// Requires head_dim 64 or 128 and page_size a multiple of 16.
#define LI_PDL_KIND 4
#include "tcgen05.cuh"

namespace tc {
int make_map_ex(CUtensorMap* map, const void* base, unsigned long long rows, unsigned long long cols, unsigned box_cols, unsigned box_rows,
                int swizzle_bytes);
}

namespace {

using namespace tc;

constexpr int kRows = 128;          // tokens per CTA
constexpr int kKeys = 128;          // keys per tile
constexpr int kThreads = 352;        // warp 0 loads keys (and the queries), warp 1 issues the products, warps 2-9 softmax, warp 10 loads values
constexpr int kBuffers = 3;
constexpr int kPartTiles = 2;        // fewest key tiles a CTA takes when a tile of tokens is shared out
constexpr int kMultiprocessors = 148;

template <int DH>
struct __align__(1024) Smem {
    unsigned char k[kBuffers][kKeys * DH * 2];       // DH / 64 panels of [128 keys][64] (128-byte swizzle)
    unsigned char v[kBuffers][kKeys * DH * 2];       // 8 blocks of [DH rows][16 keys] (32-byte swizzle)
    unsigned long long q_full, p_full[2], pv_full[2];      // P written / P V done, by tile parity
    unsigned long long s_full[2], mx_full[2];
    float mx[2][2][kRows];                           // [tile parity][half of the keys][row]: maxima, exchanged between a row's two threads
    int is_last;                                     // of the CTAs that share a tile of tokens, this one finished last
    int failed;                                      // a softmax thread gave up waiting
    unsigned long long k_full[kBuffers], k_empty[kBuffers], v_full[kBuffers], v_empty[kBuffers];
    unsigned tmem_base;
};

// bytes of dynamic shared memory beyond the structure, for its alignment: all that a CTA may have, up to a kilobyte
template <int DH>
__host__ __device__ constexpr size_t smem_pad() {
    return sizeof(Smem<DH>) + 1024 <= 232448 ? 1024 : 232448 - sizeof(Smem<DH>);
}

template <int DH>
__global__ void __launch_bounds__(kThreads, 1)
prefill_attention_tc_kernel(const bf16* __restrict__ qkv, long long row_elems, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, const int* __restrict__ block_table,
                            int max_blocks, const int* __restrict__ q_start, const int* __restrict__ ctx_lens, int nh, int nkv,
                            int page_size, int num_pages, float scale, int window, int skip_single, int* __restrict__ error_flag, int trace,
                            const int* __restrict__ units, float* __restrict__ partial, unsigned* __restrict__ counters) {
    extern __shared__ unsigned char smem_raw[];
    Smem<DH>& sm = *reinterpret_cast<Smem<DH>*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // the tiles want 1024-byte alignment; with head_dim 128 there is not a whole kilobyte to spare for it
    if ((size_t)(reinterpret_cast<unsigned char*>(&sm) - smem_raw) > smem_pad<DH>()) {
        if (threadIdx.x == 0) atomicExch(error_flag, 14);
        return;
    }
    constexpr int kPanels = DH / 64;
    constexpr unsigned kTmemCols = 512;              // S of two tiles: 128 columns each; O: up to 128; Q: up to 64
    // What this CTA works on.  With a work list (`units`, made on the host with the step's other metadata: two counts, two
    // unused words, then per entry sequence, tile of tokens, part | parts << 8, unused; heaviest first, the parts of a tile
    // next to each other) blockIdx.y is an entry; entries past the count (the first: portions of two tokens and more,
    // the second: all) are not there.  Without one the grid is (head, tile of tokens, sequence), the last tiles (which see
    // the most keys) first, all heads of a tile together, so that the long CTAs do not start late.
    const int h = blockIdx.x;
    int s, tile, part = 0, parts_asked = 1, first_entry = 0;
    if (units) {
        const int u = blockIdx.y;
        if (u >= units[skip_single ? 0 : 1]) return;
        const int4 e = *reinterpret_cast<const int4*>(units + 4 + 4 * u);
        s = e.x, tile = e.y, part = e.z & 0xff, parts_asked = partial ? (e.z >> 8) : 1, first_entry = u - part;
    } else {
        s = blockIdx.z, tile = (int)gridDim.y - 1 - (int)blockIdx.y;
    }
    const int tok0 = q_start[s], n = q_start[s + 1] - tok0;
    const int cta_i0 = tile * kRows;
    if (cta_i0 >= n || (skip_single && n == 1)) return;          // skip_single: sequences of one token are another kernel's
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ctx = ctx_lens[s];
    const int kvh = h / (nh / nkv);
    const int cta_rows = min(kRows, n - cta_i0);
    const int p_first = ctx - n + cta_i0, p_last = p_first + cta_rows - 1;
    const int key_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    // The key tiles of this tile of tokens.  When the step has so few tiles of tokens that multiprocessors would stand idle,
    // the work list shares them out among several CTAs (entries with parts > 1), at least kPartTiles each, and the last
    // CTA to finish adds the partial results up.  The workspace has room for one partial result per multiprocessor.
    const int tiles_all = p_last / kKeys - key_lo / kKeys + 1;
    int parts = min(parts_asked, (tiles_all + kPartTiles - 1) / kPartTiles);
    if ((first_entry + parts_asked) * nh > kMultiprocessors) parts = 1;
    if (part >= parts) return;
    const int kt_first = key_lo / kKeys + (int)((long long)part * tiles_all / parts);
    const int ntiles = key_lo / kKeys + (int)((long long)(part + 1) * tiles_all / parts) - kt_first;
    // the page of each 16-key block of a tile, for the lanes of the loading warps; the first tile's as early as possible
    // (the table and the lengths were written before the step's first kernel started, so they may be read before pdl_wait)
    const int* bt = block_table + (size_t)s * max_blocks;
    auto look_up = [&](int j, int& page, int& off) {
        const int key = (kt_first + j) * kKeys + (lane & 7) * 16;
        const int idx = key / page_size;
        page = (j < ntiles && key < ctx && idx < max_blocks) ? bt[idx] : 0;
        if (page < 0 || page >= num_pages) page = 0;
        off = key - idx * page_size;
    };
    int page = 0, off = 0;
    if (warp == 0 || warp == 10) look_up(0, page, off);

    if (threadIdx.x == 0) {
        sm.failed = 0;
        mbar_init(&sm.q_full, 256);
        mbar_init(&sm.s_full[0], 1);
        mbar_init(&sm.s_full[1], 1);
        mbar_init(&sm.p_full[0], 256);
        mbar_init(&sm.p_full[1], 256);
        mbar_init(&sm.mx_full[0], 256);
        mbar_init(&sm.mx_full[1], 256);
        mbar_init(&sm.pv_full[0], 1);
        mbar_init(&sm.pv_full[1], 1);
        for (int b = 0; b < kBuffers; ++b) {
            mbar_init(&sm.k_full[b], 1);
            mbar_init(&sm.k_empty[b], 1);
            mbar_init(&sm.v_full[b], 1);
            mbar_init(&sm.v_empty[b], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Tensor memory is taken only once the kernel before this one has finished: a CTA that waits for that kernel must not
    // hold what a CTA of it may still ask for (gemm_tcgen05.cu has the story).
    pdl_launch_dependents();
    pdl_wait();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // S of tile j at tmem_s + 128 (j & 1), and P of tile j over its first 64 columns (two bfloat16 a column)
    const unsigned tmem_s = sm.tmem_base, tmem_pv = sm.tmem_base + 256, tmem_q = sm.tmem_base + 384;
    // Debugging aid (LITINFER_B200_ATTN_TRACE): the first CTA leaves the clock at which each role passed each point of each
    // of its first 16 key tiles in the mapped status area, [role][point][tile] from word 16 on.
    const bool tracing = trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    auto stamp = [&](int role, int point, int j) {
        if (tracing && j < 16) error_flag[16 + (role * 8 + point) * 16 + j] = (int)clock64();
    };

    if (warp == 0 || warp == 10) {
        // The loading warps: warp 0 the keys, warp 10 the values.  A tile of 128 keys is eight
        // blocks of 16 keys, each in one page; lane b looks block b's page up (for the next tile while this one's copies are
        // issued) and issues that block's copies, so that the lookups and the issue of a tile's 8 or 16 copies run side by
        // side instead of one after another in a single thread.  Lane 0 waits for the buffer and announces the bytes.
        const bool keys = warp == 0;
        bool ok = true;
        // keys of a tile as soon as the product S two tiles back has read its buffer, values once P V has
        for (int j = 0; j < ntiles; ++j) {
            const int b = j % kBuffers;
            const unsigned free_parity = ((j / kBuffers) & 1) ^ 1;
            int next_page, next_off;
            look_up(j + 1, next_page, next_off);
            if (lane == 0) {
                stamp(keys ? 0 : 4, 0, j);
                ok = mbar_wait(keys ? &sm.k_empty[b] : &sm.v_empty[b], free_parity);
                if (ok) mbar_expect_tx(keys ? &sm.k_full[b] : &sm.v_full[b], kKeys * DH * 2);
                stamp(keys ? 0 : 4, 1, j);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < kKeys / 16) {
                if (keys) {
#pragma unroll
                    for (int pn = 0; pn < kPanels; ++pn)
                        tma_load_2d(sm.k[b] + pn * (kKeys * 128) + lane * 2048, &map_k, pn * 64, (page * nkv + kvh) * page_size + off, &sm.k_full[b]);
                } else {
                    tma_load_2d(sm.v[b] + lane * (DH * 32), &map_v, off, (page * nkv + kvh) * DH, &sm.v_full[b]);
                }
            }
            if (lane == 0) stamp(keys ? 0 : 4, 2, j);
            page = next_page;
            off = next_off;
        }
        if (!ok && lane == 0) atomicExch(error_flag, 11);
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr unsigned idesc_s = umma_idesc(kRows, kKeys), idesc_pv = umma_idesc(kRows, DH);
            bool ok = mbar_wait(&sm.q_full, 0);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // S of tile j + 1 is issued before P V of tile j: the tensor cores work on it while the softmax of tile j runs
            auto issue_s = [&](int j) {
                const int b = j % kBuffers;
                stamp(1, 0, j);
                if (!mbar_wait(&sm.k_full[b], (j / kBuffers) & 1)) return false;
                stamp(1, 1, j);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int k = 0; k < DH / 16; ++k) {
                    const unsigned long long db = umma_desc(sm.k[b] + (k >> 2) * (kKeys * 128)) + (unsigned long long)((k & 3) * 2);
                    umma_bf16_ta(tmem_s + 128 * (j & 1), tmem_q + 8 * k, db, idesc_s, k ? 1u : 0u);
                }
                umma_commit(&sm.s_full[j & 1]);
                umma_commit(&sm.k_empty[b]);
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; j < ntiles && ok; ++j) {
                const int b = j % kBuffers;
                if (j + 1 < ntiles) {
                    ok = issue_s(j + 1);
                    if (!ok) break;
                }
                stamp(1, 2, j);
                ok = mbar_wait(&sm.v_full[b], (j / kBuffers) & 1);
                if (!ok) break;
                stamp(1, 3, j);
                ok = mbar_wait(&sm.p_full[j & 1], (j >> 1) & 1);
                if (!ok) break;
                stamp(1, 4, j);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k) {
                    const unsigned long long db = umma_desc_sw32(sm.v[b] + k * (DH * 32));
                    umma_bf16_ta(tmem_pv, tmem_s + 128 * (j & 1) + 8 * k, db, idesc_pv, (j | k) ? 1u : 0u);     // the output accumulates over the tiles
                }
                umma_commit(&sm.pv_full[j & 1]);
                umma_commit(&sm.v_empty[b]);
                stamp(1, 5, j);
            }
            if (!ok) atomicExch(error_flag, 12);
        }
    } else {
        // Two threads a token (warps w and w + 4 reach the same lanes of tensor memory): each takes half of a tile's
        // keys and half of the output columns; they exchange their maxima through shared memory.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;                       // this thread's token within the tile = its lane of tensor memory
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        constexpr int HK = kKeys / 2, HD = DH / 2;
        const bool valid = cta_i0 + r < n;
        const int p = valid ? p_first + r : -1;                  // its position; no key is visible to an unused row
        const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
        const float scale_log2 = scale * 1.4426950408889634f;
        // m: the maximum the exponentials are taken against.  It follows the true maximum lazily: only when that has grown by
        // more than kLazy (in powers of two) is the output so far, which accumulates in tensor memory, scaled down to the
        // new one.  Until then the probabilities may reach 2^kLazy, which costs bfloat16 and the float sums nothing, and
        // the quotient at the end is the same.
        constexpr float kLazy = 8.0f;
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        // The token's row of Q into tensor memory, the operand layout of the product S = Q K^T: two bfloat16 a column, this
        // thread the 64 dimensions from 64 * half on (with head_dim 64 the first thread of the row has them all).
        if (half * 64 < DH) {                                    // the same for the whole warp
            unsigned qw[32];
            if (valid) {
                const uint4* src = reinterpret_cast<const uint4*>(qkv + (size_t)(tok0 + cta_i0 + r) * row_elems + (size_t)h * DH + half * 64);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 t4 = __ldg(src + i);
                    qw[4 * i] = t4.x, qw[4 * i + 1] = t4.y, qw[4 * i + 2] = t4.z, qw[4 * i + 3] = t4.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) qw[i] = 0u;
            }
            tmem_st_32x32(tmem_q + lane_addr + half * 32, qw);
            tmem_st_wait();
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&sm.q_full);
        for (int j = 0; j < ntiles && ok; ++j) {
            const int key0 = (kt_first + j) * kKeys + half * HK;
            if (lane == 0 && quarter == 0) stamp(2 + half, 0, j);
            ok = mbar_wait(&sm.s_full[j & 1], (j >> 1) & 1);
            if (!ok) break;
            if (lane == 0 && quarter == 0) stamp(2 + half, 1, j);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // this thread's 64 scores of the tile, read once and kept for both passes; a key the row does not see reads -inf
            float v[HK];
            tmem_ld_32x64(tmem_s + 128 * (j & 1) + lane_addr + half * HK, v);
            const bool whole = key0 >= lo && key0 + HK - 1 <= p;
            if (!whole) {
#pragma unroll
                for (int i = 0; i < HK; ++i)
                    if (key0 + i < lo || key0 + i > p) v[i] = -INFINITY;
            }
            // the row's maximum over the tile: this half's, then the other thread's through shared memory
            float mine = -INFINITY;
#pragma unroll
            for (int i = 0; i < HK; ++i) mine = fmaxf(mine, v[i]);
            sm.mx[j & 1][half][r] = mine;
            if (lane == 0 && quarter == 0) stamp(2 + half, 2, j);
            mbar_arrive(&sm.mx_full[j & 1]);
            ok = mbar_wait(&sm.mx_full[j & 1], (j >> 1) & 1);
            if (!ok) break;
            if (lane == 0 && quarter == 0) stamp(2 + half, 3, j);
            const float mx = fmaxf(mine, sm.mx[j & 1][half ^ 1][r]);
            const float m_true = fmaxf(m, mx * scale_log2);          // scale > 0: the order is the same
            const bool grow = m_true > m + kLazy;                    // also the first visible key of a row (m = -inf)
            const float m_new = grow ? m_true : m;
            const float ms = (m_new == -INFINITY) ? 0.0f : m_new;
            if (lane == 0 && quarter == 0) stamp(2 + half, 4, j);
            if (j > 0) {
                if (__any_sync(0xffffffffu, grow)) {                 // whole warps: the accesses to tensor memory are warp-wide
                    // the output so far is complete once P V of the tile before is
                    ok = mbar_wait(&sm.pv_full[(j - 1) & 1], ((j - 1) >> 1) & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const float alpha = grow ? fast_exp2(m - ms) : 1.0f;
#pragma unroll
                    for (int c = 0; c < HD / 32; ++c) {
                        float w[32];
                        tmem_ld_32x32(tmem_pv + lane_addr + half * HD + c * 32, w);
#pragma unroll
                        for (int i = 0; i < 32; ++i) w[i] *= alpha;
                        tmem_st_32x32(tmem_pv + lane_addr + half * HD + c * 32, w);
                    }
                    tmem_st_wait();
                    l *= alpha;
                }
            }
            m = m_new;
            if (lane == 0 && quarter == 0) stamp(2 + half, 5, j);
            // second pass: probabilities (2^-inf = 0 for the keys not seen), rounded to bfloat16, over the first half of this
            // tile's S, in the operand layout of the product P V: both threads of the row have their scores in registers
            // by now (the exchange above), and the S that will overwrite them is issued after that product.
            // The special-function unit delivers 16 exponentials a clock, and a tile has 16,384: where all of this thread's
            // keys are seen (no -inf among the scores) every fourth one is computed by a polynomial instead.
            float sum = 0.0f;
            const float neg_ms = -ms;
            unsigned pk[HK / 2];
            auto second_pass = [&](auto fourth) {
#pragma unroll
                for (int i = 0; i < HK / 2; ++i) {
                    const float x0 = fmaf(v[2 * i], scale_log2, neg_ms), x1 = fmaf(v[2 * i + 1], scale_log2, neg_ms);
                    const float e0 = fast_exp2(x0), e1 = (i & 1) ? fourth(x1) : fast_exp2(x1);
                    sum += e0 + e1;
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(e0, e1);
                    pk[i] = *reinterpret_cast<unsigned*>(&t2);
                }
            };
            if (whole) second_pass([](float x) { return poly_exp2(x); });
            else second_pass([](float x) { return fast_exp2(x); });
            l += sum;
            tmem_st_32x32(tmem_s + 128 * (j & 1) + lane_addr + half * (HK / 2), pk);
            tmem_st_wait();
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&sm.p_full[j & 1]);
            if (lane == 0 && quarter == 0) stamp(2 + half, 6, j);
        }
        // the output of the last product
        float o[HD];
        if (ok) ok = mbar_wait(&sm.pv_full[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                float v[32];
                tmem_ld_32x32(tmem_pv + lane_addr + half * HD + c * 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) o[c * 32 + i] = v[i];
            }
        }
        // the row's denominator: the sums of its two threads (both ran with the same maxima)
        if (ok) {
            const int jx = ntiles;                               // one more use of the exchange buffers
            sm.mx[jx & 1][half][r] = l;
            mbar_arrive(&sm.mx_full[jx & 1]);
            ok = mbar_wait(&sm.mx_full[jx & 1], (jx >> 1) & 1);
            if (ok) l = sm.mx[jx & 1][0][r] + sm.mx[jx & 1][1][r];
        }
        bool store = valid;
        if (parts > 1) {                                          // the same for the whole CTA; every softmax thread takes part, failed or not
            // Shared tile of tokens: this CTA's output (unnormalised, against its maximum m), m and the sum l go to the
            // workspace, [column][row] so that a warp writes consecutive words.  The CTA that arrives last adds all parts
            // up in their order, whichever it is itself, so the result does not depend on the order of arrival.
            constexpr int kPartFloats = kRows * (DH + 2);
            const size_t unit = (size_t)first_entry * nh + h;      // the tile's first entry stands for it
            if (ok) {
                float* mine = partial + ((size_t)(first_entry + part) * nh + h) * kPartFloats;
#pragma unroll
                for (int d = 0; d < HD; ++d) mine[(half * HD + d) * kRows + r] = o[d];
                if (half == 0) {
                    mine[DH * kRows + r] = m;
                    mine[(DH + 1) * kRows + r] = l;
                }
                __threadfence();
            } else {
                sm.failed = 1;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (warp == 2 && lane == 0) sm.is_last = (!sm.failed && atomicAdd(&counters[unit], 1u) == (unsigned)(parts - 1)) ? 1 : 0;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (sm.failed) ok = false;
            if (ok && sm.is_last) {
                __threadfence();
                const float* first = partial + unit * kPartFloats;
                const size_t stride = (size_t)nh * kPartFloats;     // from one part of the tile to the next
                float m_all = -INFINITY;
                for (int q = 0; q < parts; ++q) m_all = fmaxf(m_all, __ldcg(first + q * stride + DH * kRows + r));
                const float ref = (m_all == -INFINITY) ? 0.0f : m_all;
#pragma unroll
                for (int d = 0; d < HD; ++d) o[d] = 0.0f;
                l = 0.0f;
                for (int q = 0; q < parts; ++q) {
                    const float* theirs = first + q * stride;
                    const float w = exp2f(__ldcg(theirs + DH * kRows + r) - ref);
                    l += __ldcg(theirs + (DH + 1) * kRows + r) * w;
#pragma unroll
                    for (int d = 0; d < HD; ++d) o[d] += __ldcg(theirs + (half * HD + d) * kRows + r) * w;
                }
                if (warp == 2 && lane == 0) counters[unit] = 0;           // ready for the next launch
            } else {
                store = false;                                    // the last CTA writes the tokens' output
            }
        }
        if (!ok) {
            if (lane == 0) atomicExch(error_flag, 13);
        } else if (store) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            bf16* dst = out + ((size_t)(tok0 + cta_i0 + r) * nh + h) * DH + half * HD;
#pragma unroll
            for (int d = 0; d < HD; d += 8) {
                unsigned pk[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(o[d + 2 * i] * inv, o[d + 2 * i + 1] * inv);
                    pk[i] = *reinterpret_cast<unsigned*>(&t2);
                }
                *reinterpret_cast<uint4*>(dst + d) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        }
    }
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(sm.tmem_base), "r"(kTmemCols) : "memory");
    }
}

// Workspace of the CTAs that share a tile of tokens: their partial outputs and a counter per tile and head.  One per process,
// of a fixed size (as many partial outputs of head_dim 128 as there are multiprocessors: 10 MB), allocated at the first launch
// that wants it; launches that use it are in stream order (the library runs a model's step on one stream).
struct SplitSpace {
    float* partial = nullptr;
    unsigned* counters = nullptr;
    // false if there is none and none can be made now (a stream capture is under way): the launch then shares nothing out
    bool ready(cudaStream_t stream, int* rc) {
        *rc = 0;
        if (partial) return true;
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) {
            cudaGetLastError();
            return false;
        }
        const size_t bytes = (size_t)kMultiprocessors * kRows * (128 + 2) * sizeof(float);
        cudaError_t e = cudaMalloc((void**)&partial, bytes);
        if (e == cudaSuccess) e = cudaMalloc((void**)&counters, kMultiprocessors * sizeof(unsigned));
        if (e == cudaSuccess) e = cudaMemset(counters, 0, kMultiprocessors * sizeof(unsigned));
        if (e != cudaSuccess) {
            *rc = li_fail("attention (tcgen05): cannot allocate %zu bytes of workspace: %s", bytes, cudaGetErrorString(e));
            partial = nullptr;
            return false;
        }
        return true;
    }
};

SplitSpace& split_space() {
    static SplitSpace space;
    return space;
}

template <int DH>
int launch(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks, const int* q_start,
           const int* ctx_lens, int T, int S, int nh, int nkv, int page_size, int num_pages, float scale, int window, int max_q_len,
           int skip_single, const int* units, int unit_slots, cudaStream_t stream) {
    EncodeTiledFn encode = nullptr;
    int *err_host = nullptr, *err_dev = nullptr;
    if (int rc = setup(&encode, &err_host, &err_dev)) return rc;
    if (*err_host != 0)
        return li_fail("attention (tcgen05): an earlier launch gave up waiting on a barrier (status %d); the results since then are invalid", *err_host);
    CUtensorMap map_k, map_v;
    const long long row_elems = (long long)(nh + 2 * nkv) * DH;
    if (int rc = make_map_ex(&map_k, kcache, (unsigned long long)num_pages * nkv * page_size, DH, 64, 16, 128)) return rc;
    if (int rc = make_map_ex(&map_v, vcache, (unsigned long long)num_pages * nkv * DH, (unsigned long long)page_size, 16, DH, 32)) return rc;
    const size_t smem = sizeof(Smem<DH>) + smem_pad<DH>();
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return li_fail("attention (tcgen05): cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    LI_REQUIRE(S <= 65535 && ceil_div(max_q_len, kRows) <= 65535, "attention (tcgen05): batch %d or portions of %d tokens too large for one launch", S, max_q_len);
    // With a work list the grid is (head, entry); a step with few tiles of tokens (a portion of a prompt behind a long
    // context) would leave multiprocessors idle while each CTA walks many key tiles, so its list shares the key tiles of
    // a tile of tokens out among as many CTAs as still run all at once.  (Measured: with more CTAs than multiprocessors
    // the fixed cost of the extra CTAs outweighs the shorter walks, 29 -> 38 us for 2,048 tokens x 12 heads.)
    SplitSpace& space = split_space();
    float* partial = nullptr;
    if (units) {
        LI_REQUIRE(unit_slots >= 0 && unit_slots <= 65535, "attention (tcgen05): a work list of %d entries", unit_slots);
        if (unit_slots == 0) return 0;
        int rc = 0;
        if (space.ready(stream, &rc)) partial = space.partial;
        if (rc) return rc;
    }
    const dim3 grid = units ? dim3(nh, unit_slots, 1) : dim3(nh, ceil_div(max_q_len, kRows), S);
    static const int trace = getenv("LITINFER_B200_ATTN_TRACE") ? 1 : 0;
    li_launch_pdl(prefill_attention_tc_kernel<DH>, grid, dim3(kThreads), smem, stream, (const bf16*)qkv, row_elems, map_k, map_v, (bf16*)out, block_table, max_blocks,
                  q_start, ctx_lens, nh, nkv, page_size, num_pages, scale, window, skip_single, err_dev, trace, units, partial,
                  space.counters);
    return li_check_launch("attention (tcgen05)");
}

}  // namespace

bool li_attention_tcgen05_accepts(const void* qkv, const void* kcache, const void* vcache, int nh, int nkv, int dh, int page_size) {
    const bool aligned = ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)kcache % 16 == 0) && ((uintptr_t)vcache % 16 == 0);
    return aligned && (dh == 64 || dh == 128) && nh % nkv == 0 && page_size % 16 == 0 && page_size <= 256;
}

int li_attention_tcgen05(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                         const int* q_start, const int* ctx_lens, int T, int S, int nh, int nkv, int dh, int page_size, int num_pages,
                         float scale, int window, int max_q_len, int skip_single, const int* units, int unit_slots, cudaStream_t stream) {
    LI_REQUIRE(li_attention_tcgen05_accepts(qkv, kcache, vcache, nh, nkv, dh, page_size),
               "attention (tcgen05): refuses heads=%d/%d head_dim=%d page=%d (head_dim 64 or 128, pages a multiple of 16)", nh, nkv, dh, page_size);
    LI_REQUIRE(scale > 0.0f, "attention (tcgen05): the scale must be positive");
    if (dh == 64)
        return launch<64>(qkv, out, kcache, vcache, block_table, max_blocks, q_start, ctx_lens, T, S, nh, nkv, page_size, num_pages, scale,
                          window, max_q_len, skip_single, units, unit_slots, stream);
    return launch<128>(qkv, out, kcache, vcache, block_table, max_blocks, q_start, ctx_lens, T, S, nh, nkv, page_size, num_pages, scale,
                       window, max_q_len, skip_single, units, unit_slots, stream);
}
