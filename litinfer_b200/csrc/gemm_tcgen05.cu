// out[M, N] = a[M, K] w[N, K]^T (+ bias) in bfloat16 on the fifth-generation
// tensor cores: tcgen05.mma with both operands staged in shared memory by TMA
// and the float accumulator in tensor memory.  The prefill path of every
// projection (q|k|v, o, gate|up, down, lm_head).
//
// One CTA computes a BM x BN tile: 128 x 128 with a ring of 6 stages, 256 x 128
// with 4, or 256 x 256 (two accumulators of 128 lanes x 256 columns: all of
// tensor memory) with 3 stages.  A multiprocessor takes in operand bytes from
// L2 at a limited rate (about 55 GB/s measured here, 8 TB/s over the GPU); a
// 128 x 128 tile needs 32 KB per 256 tensor-core cycles and is bound by that,
// a 256 x 256 tile needs 64 KB per 1024 cycles.  The large tile is used where it
// still fills the GPU (wide products: gate|up, lm_head of many rows; with a
// split of k: down), the middle one for narrow products with a short k
// (q|k|v, o).  Roles, by warp:
//   warp 0   producer: one lane issues the TMA loads of a BM x 64 tile of a and
//            a BN x 64 tile of w per k-block (64 bfloat16 = one 128-byte swizzle
//            row) into a ring of stages, each guarded by a full/empty mbarrier pair;
//   warp 1   allocates tensor memory; one lane issues four tcgen05.mma (M 128,
//            N BN, K 16) per k-block and 128 rows of a, commits the stage's
//            empty barrier, and at the end the accumulator's barrier;
//   warps 2-5 epilogue: tcgen05.ld of their quarter of the 128 lanes, bias in
//            float, one rounding, stores to global memory.
// Both operands are K-major ([rows, K] row-major), which is how activations and
// LitInfer-style [out, in] weights (src/ops/linear/cpu/linear_cpu.cpp:45-60)
// lie in memory; TMA zero-fills rows and columns beyond the tensor, so any M,
// N and any K that is a multiple of 8 (16-byte rows) work.
//
// Every wait on an mbarrier is bounded.  A wait that runs out raises a flag in
// mapped host memory (li_tcgen05_status() reads it), the CTA waits, again
// bounded, for the copies it has in flight, frees its tensor memory and returns.
#define LI_PDL_KIND 1
#include "gemm_epilogue.cuh"
#include "rope_epilogue.cuh"
#include "tcgen05.cuh"

bool li_tcgen05_persistent_wanted(int M, int N, int K);
bool li_tcgen05_accepts(const void* a, const void* w, const void* out, int dtype_out, int M, int N, int K);

namespace {

using namespace tc;

constexpr int kThreads = 192;

int g_forced_ksplit = 0;         // > 0: split k this many ways whatever the shape (tests and measurements)

// kPair: two CTAs of a cluster (multiprocessors of one pair) work as one on a tile of 2 BM x BN with tcgen05.mma
// cta_group::2: each brings its own BM rows of a and half of the BN rows of w, the tensor cores of both read both halves
// of w, and each keeps the accumulator of its own rows.  A CTA then takes in a quarter less per flop (BM = BN = 256).
template <int BM, int BN, bool kPair = false>
struct Tile {
    static constexpr int kRowsB = kPair ? BN / 2 : BN;
    static constexpr int kBytesA = BM * BK * 2, kBytesB = kRowsB * BK * 2;
    static constexpr int kStages = (kBytesA + kBytesB) <= 24576 ? 8 : (kBytesA + kBytesB) <= 32768 ? 6 : ((kBytesA + kBytesB) <= 49152 ? 4 : 3);
    static constexpr unsigned kAccCols = (BM / 128) * BN;       // tensor-memory columns: one accumulator per 128 rows
    static constexpr unsigned kCols = kAccCols <= 32 ? 32 : kAccCols <= 64 ? 64 : kAccCols <= 128 ? 128 : kAccCols <= 256 ? 256 : 512;   // allocated: a power of two
};

template <int BM, int BN, bool kPair = false>
struct __align__(1024) SharedStorage {
    unsigned char a[Tile<BM, BN, kPair>::kStages][Tile<BM, BN, kPair>::kBytesA];
    unsigned char b[Tile<BM, BN, kPair>::kStages][Tile<BM, BN, kPair>::kBytesB];
    unsigned long long full[Tile<BM, BN, kPair>::kStages];
    unsigned long long empty[Tile<BM, BN, kPair>::kStages];
    unsigned long long accum;
    unsigned long long peer_alloc;       // a pair: the second CTA has its tensor memory
    unsigned tmem_base;
    int failed;
    int is_last;
};

// One head (128 columns at `col0` of the accumulator row of token `row`) of the q|k|v product: bias, rotation of q and k
// by the step's table, q into the output row, k into the paged cache, v into it transposed (rope_epilogue.cuh).
// Called by whole warps (the loads from tensor memory are warp-wide); `valid`: this thread's row is a row of the product.
// Two threads share a row (the warps w and w + 4 reach the same lanes of tensor memory): `part` 0 takes the first half of
// the head's rotation pairs (or of a value head's columns), `part` 1 the second.
// `cs`: this row's 64 (cos, sin) pairs, in the step's table or staged in shared memory by the caller (rope_stage_table).
__device__ __forceinline__ void rope_store_head(unsigned tmem_row, int col_in_tile, int row, bool valid, int head, const float* __restrict__ bias,
                                                bf16* __restrict__ out, int N, const RopeEpilogue& re, int part, const float2* cs) {
    const int slot = valid ? re.slot_mapping[row] : -1;
    const int page = slot / re.page_size, off = slot - page * re.page_size;
    const bool cache_ok = valid && re.write && slot >= 0 && page < re.num_pages;       // validated on the host; never write outside the cache
    if (head < re.nh + re.nkv) {                                   // the same for the whole warp
        const bool is_q = head < re.nh;
        const bool store = is_q ? valid : cache_ok;
        bf16* dst = !store ? nullptr
                    : (is_q ? out + (size_t)row * N + (size_t)head * 128
                            : re.kcache + (((size_t)page * re.nkv + (head - re.nh)) * re.page_size + off) * 128);
        {
            const int c = part;
            float lo[32], hi[32];
            tc::tmem_ld_32x32(tmem_row + (unsigned)(col_in_tile + c * 32), lo);
            tc::tmem_ld_32x32(tmem_row + (unsigned)(col_in_tile + c * 32 + 64), hi);
            unsigned plo[16], phi[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float y[4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = c * 32 + i + e;
                    float a = lo[i + e], b = hi[i + e];
                    if (bias) {
                        a += bias[head * 128 + j];
                        b += bias[head * 128 + j + 64];
                    }
                    // q and k are rounded to bfloat16 by the projection before they are rotated, as in the unfused path
                    a = __bfloat162float(__float2bfloat16_rn(a));
                    b = __bfloat162float(__float2bfloat16_rn(b));
                    const float2 t2 = cs[j];
                    y[e] = a * t2.x - b * t2.y;
                    y[2 + e] = b * t2.x + a * t2.y;
                }
                __nv_bfloat162 l2 = __floats2bfloat162_rn(y[0], y[1]), h2 = __floats2bfloat162_rn(y[2], y[3]);
                plo[i >> 1] = *reinterpret_cast<unsigned*>(&l2);
                phi[i >> 1] = *reinterpret_cast<unsigned*>(&h2);
            }
            if (store) {
                uint4* dl = reinterpret_cast<uint4*>(dst + c * 32);
                uint4* dh = reinterpret_cast<uint4*>(dst + c * 32 + 64);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    dl[q] = make_uint4(plo[4 * q], plo[4 * q + 1], plo[4 * q + 2], plo[4 * q + 3]);
                    dh[q] = make_uint4(phi[4 * q], phi[4 * q + 1], phi[4 * q + 2], phi[4 * q + 3]);
                }
            }
        }
    } else {
        bf16* dst = cache_ok ? re.vcache + ((size_t)page * re.nkv + (head - re.nh - re.nkv)) * 128 * re.page_size + off : nullptr;
#pragma unroll 1
        for (int c = 2 * part; c < 2 * part + 2; ++c) {
            float v[32];
            tc::tmem_ld_32x32(tmem_row + (unsigned)(col_in_tile + c * 32), v);
            if (cache_ok) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int d = c * 32 + i;
                    dst[(size_t)d * re.page_size] = __float2bfloat16_rn(bias ? v[i] + bias[head * 128 + d] : v[i]);
                }
            }
        }
    }
}

// The step's table of cosines and sines for the tile's 128 rows, from global memory (64 pairs = 512 bytes a row) into shared
// memory with coalesced loads, a row every 65 pairs so that the lanes of a warp, a row each, read different banks.  Read
// row by row straight from global memory, every load of a warp touched 32 lines: the load/store unit then bounded the
// epilogue (26 us for q|k|v of 2,048 tokens at hidden 1536, of which the tensor pipe works 6).
constexpr int kRopeRowPairs = 65;
__device__ __forceinline__ void rope_stage_table(float2* cs_sm, const float* __restrict__ cos_sin, int m0, int M, int tid) {
    // 256 threads, 16 loads of two pairs each, all in flight at once (a loop of single loads cost their latency 32 times)
    const float4* src = reinterpret_cast<const float4*>(cos_sin);
    float4 t4[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const int i = tid + k * 256, r = i >> 5;                 // pair 2 (i & 31) of row r
        t4[k] = (m0 + r < M) ? __ldg(src + (size_t)(m0 + r) * 32 + (i & 31)) : make_float4(1.0f, 0.0f, 1.0f, 0.0f);
    }
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const int i = tid + k * 256, r = i >> 5, j = 2 * (i & 31);
        cs_sm[r * kRopeRowPairs + j] = make_float2(t4[k].x, t4[k].y);
        cs_sm[r * kRopeRowPairs + j + 1] = make_float2(t4[k].z, t4[k].w);
    }
}

// threads of a CTA: producer warp, issuing warp, four epilogue warps; eight with the rotary epilogue, the longest one for
// its product (a k of `hidden` only, and per row a table read, a rotation and scattered stores): two threads share a row
template <bool kRope>
__host__ __device__ constexpr int threads_of() { return kRope ? 320 : kThreads; }

template <int BM, int BN, typename Tout, bool kSwiglu, bool kPair = false, bool kRope = false>
__global__ void __launch_bounds__(threads_of<kRope>(), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, Tout* __restrict__ out, int M, int N, int K, int* __restrict__ error_flag,
                    float* __restrict__ partial, unsigned* __restrict__ counters, int ksplit, const RopeEpilogue rope) {
    extern __shared__ unsigned char smem_raw[];
    using SS = SharedStorage<BM, BN, kPair>;
    constexpr int kStages = Tile<BM, BN, kPair>::kStages;
    constexpr int kStageBytesA = Tile<BM, BN, kPair>::kBytesA, kStageBytesB = Tile<BM, BN, kPair>::kBytesB;
    constexpr unsigned kCols = Tile<BM, BN, kPair>::kCols;
    const unsigned pair_rank = kPair ? cluster_cta_rank() : 0u;
    SS& sm = *reinterpret_cast<SS*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // a pair is two neighbours along x (the hardware pairs CTAs of consecutive rank): they share the tile's columns and
    // take consecutive tiles of rows
    const int m0 = kPair ? ((int)blockIdx.y * 2 + (int)(blockIdx.x & 1)) * BM : (int)blockIdx.y * BM;
    const int n0 = kPair ? (int)(blockIdx.x >> 1) * BN : (int)blockIdx.x * BN;
    const int nkb_total = (K + BK - 1) / BK;
    const int split = blockIdx.z;
    const int kb_first = (int)((long long)split * nkb_total / ksplit);
    const int nkb = (int)((long long)(split + 1) * nkb_total / ksplit) - kb_first;       // this CTA's k-blocks

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        mbar_init(&sm.accum, 1);
        mbar_init(&sm.peer_alloc, 1);
        sm.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();          // the other CTA's barriers are set up before anything arrives on them
    // Tensor memory is taken only once the kernel before this one has finished (warp 1, below): a CTA that waits for
    // that kernel must not hold what a CTA of it may still ask for.  With the accumulators taken first and every launch a
    // dependent one, steps of thousands of tokens of a 7B-shaped model stopped in tcgen05.alloc about two runs in five.
    // The warps that read the accumulator meet warp 1 at a named barrier once it has the address.
    constexpr int kAllocMeet = 32 + (threads_of<kRope>() - 64);
    auto take_tensor_memory = [&]() {
        pdl_wait();
        if constexpr (kPair) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kCols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kCols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };
    auto meet_tensor_memory = [&]() {
        asm volatile("bar.sync 3, %0;" ::"n"(kAllocMeet) : "memory");
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        return sm.tmem_base;
    };
    // programmatic dependent launch: everything up to here overlapped the end of the kernel before this one; what reads
    // its results (the producer) or writes over memory it may still read (the epilogue) waits for it
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            // the weight tiles of the first stages at once (weights do not depend on the kernel before this one); the
            // tiles of a once that kernel has finished
            const int first = nkb < kStages ? nkb : kStages;
            for (int kb = 0; kb < first; ++kb) {
                if constexpr (kPair) {
                    if (pair_rank == 0) mbar_expect_tx(&sm.full[kb], 2 * (kStageBytesA + kStageBytesB));
                    tma_load_2d_pair(sm.b[kb], &map_w, (kb_first + kb) * BK, n0 + (int)pair_rank * (BN / 2), &sm.full[kb]);
                } else {
                    mbar_expect_tx(&sm.full[kb], kStageBytesA + kStageBytesB);
                    tma_load_2d(sm.b[kb], &map_w, (kb_first + kb) * BK, n0, &sm.full[kb]);
                }
            }
            pdl_wait();
            for (int kb = 0; kb < first; ++kb) {
                if constexpr (kPair) tma_load_2d_pair(sm.a[kb], &map_a, (kb_first + kb) * BK, m0, &sm.full[kb]);
                else tma_load_2d(sm.a[kb], &map_a, (kb_first + kb) * BK, m0, &sm.full[kb]);
            }
            int issued = first;
            for (int kb = first; kb < nkb && ok; ++kb) {
                const int s = kb % kStages;
                const unsigned phase = (kb / kStages) & 1;
                ok = mbar_wait(&sm.empty[s], phase ^ 1);
                if (!ok) break;
                if constexpr (kPair) {
                    // both CTAs' tiles are counted on the first CTA's barrier, which expects the bytes of both
                    if (pair_rank == 0) mbar_expect_tx(&sm.full[s], 2 * (kStageBytesA + kStageBytesB));
                    tma_load_2d_pair(sm.a[s], &map_a, (kb_first + kb) * BK, m0, &sm.full[s]);
                    tma_load_2d_pair(sm.b[s], &map_w, (kb_first + kb) * BK, n0 + (int)pair_rank * (BN / 2), &sm.full[s]);
                } else {
                    mbar_expect_tx(&sm.full[s], kStageBytesA + kStageBytesB);
                    tma_load_2d(sm.a[s], &map_a, (kb_first + kb) * BK, m0, &sm.full[s]);
                    tma_load_2d(sm.b[s], &map_w, (kb_first + kb) * BK, n0, &sm.full[s]);
                }
                issued = kb + 1;
            }
            if (!ok) {
                sm.failed = 1;
                atomicExch(error_flag, 1);
                // the copies already issued must land before the CTA may leave (in a pair only the first CTA can tell)
                if (!kPair || pair_rank == 0)
                    for (int kb = (issued > kStages ? issued - kStages : 0); kb < issued; ++kb)
                        mbar_wait(&sm.full[kb % kStages], (kb / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        take_tensor_memory();
        const unsigned tmem_acc = meet_tensor_memory();
        if constexpr (kPair) {
            if (lane == 0 && pair_rank == 1) mbar_arrive_remote(&sm.peer_alloc, 0);
        }
        if (lane == 0 && pair_rank == 0) {                 // in a pair the first CTA issues the products of both
            const unsigned idesc = umma_idesc(kPair ? 256 : 128, BN);
            bool ok = true;
            if constexpr (kPair) ok = mbar_wait(&sm.peer_alloc, 0);       // the products write the second CTA's tensor memory too
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % kStages;
                const unsigned phase = (kb / kStages) & 1;
                ok = mbar_wait(&sm.full[s], phase);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned long long da = umma_desc(sm.a[s]), db = umma_desc(sm.b[s]);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
#pragma unroll
                    for (int half = 0; half < BM / 128; ++half) {     // rows 128 half .. of the a tile: 128 rows x 128 bytes further on
                        if constexpr (kPair)
                            umma_bf16_pair(tmem_acc + (unsigned)(half * BN), da + (unsigned long long)(k * 2 + half * (128 * 128 / 16)),
                                           db + (unsigned long long)(k * 2), idesc, (kb | k) ? 1u : 0u);
                        else
                            umma_bf16(tmem_acc + (unsigned)(half * BN), da + (unsigned long long)(k * 2 + half * (128 * 128 / 16)),
                                      db + (unsigned long long)(k * 2), idesc, (kb | k) ? 1u : 0u);
                    }
                if constexpr (kPair) umma_commit_pair(&sm.empty[s]);
                else umma_commit(&sm.empty[s]);
            }
            if (ok) {
                if constexpr (kPair) umma_commit_pair(&sm.accum);
                else umma_commit(&sm.accum);
            } else {
                sm.failed = 1;
                atomicExch(error_flag, 2);
            }
        }
    } else {
        // epilogue: warp w may read the tensor-memory lanes 32 (w % 4) .. 32 (w % 4) + 31
        const int quarter = warp & 3;
        const unsigned tmem_acc = meet_tensor_memory();
        const bool ok = mbar_wait(&sm.accum, 0);
        if (!ok) {
            if (lane == 0) atomicExch(error_flag, 3);
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            pdl_wait();
            // one 32-column piece of a row: bias or SwiGLU, one rounding, store
            auto emit = [&](int row, int c, float (&v)[32]) { gemm_store_piece<Tout, kSwiglu>(row, n0 + c, v, bias, out, M, N); };
            const size_t tile_id = (size_t)blockIdx.y * gridDim.x + blockIdx.x, tiles = (size_t)gridDim.x * gridDim.y;
            if constexpr (kRope) {
                // the q|k|v product of a prefill step: a tile of 128 or 256 columns is one or two heads of 128; never split along k
                static_assert(!kRope || (BM == 128 && BN % 128 == 0 && sizeof(Tout) == 2 && !kSwiglu), "the rope epilogue is for tiles of whole heads of 128 in bfloat16");
                const int row = m0 + quarter * 32 + lane;
                // the accumulator is complete, so every product has read its operands and every copy has landed: the
                // stages of the a operand are free to hold the table
                static_assert(sizeof(sm.a) >= 128 * kRopeRowPairs * sizeof(float2), "the rotary table of a tile fits the a stages");
                // (a tile of one head gains nothing from the detour: 17.6 -> 18.6 us for 544 tokens; it reads the table in place)
                constexpr bool kStaged = BN >= 256;
                float2* cs_sm = reinterpret_cast<float2*>(&sm.a[0][0]);
                if constexpr (kStaged) {
                    rope_stage_table(cs_sm, rope.cos_sin, m0, M, threadIdx.x - 64);      // the eight epilogue warps
                    asm volatile("bar.sync 2, 256;" ::: "memory");
                }
                const float2* cs_row = kStaged ? cs_sm + (quarter * 32 + lane) * kRopeRowPairs
                                               : reinterpret_cast<const float2*>(rope.cos_sin) + (size_t)(row < M ? row : 0) * 64;
#pragma unroll 1
                for (int hl = 0; hl < BN / 128; ++hl) {
                    const int head = n0 / 128 + hl;
                    if (head * 128 < N)                            // the same for the whole CTA
                        rope_store_head(tmem_acc + ((unsigned)(quarter * 32) << 16), hl * 128, row, row < M, head, bias, reinterpret_cast<bf16*>(out), N, rope,
                                        (warp - 2) >> 2, cs_row);
                }
            } else if (ksplit == 1) {
#pragma unroll 1
                for (int hc = 0; hc < (BM / 128) * (BN / 32); ++hc) {
                    const int half = hc / (BN / 32), c = (hc - half * (BN / 32)) * 32;
                    float v[32];
                    tmem_ld_32x32(tmem_acc + ((unsigned)(quarter * 32) << 16) + (unsigned)(half * BN + c), v);
                    emit(m0 + half * 128 + quarter * 32 + lane, c, v);
                }
            } else {
                // k is split over several CTAs: each leaves its float tile in the workspace; the one that
                // arrives last (a counter per tile) adds the tiles in split order and finishes
#pragma unroll 1
                for (int hc = 0; hc < (BM / 128) * (BN / 32); ++hc) {
                    const int half = hc / (BN / 32), c = (hc - half * (BN / 32)) * 32;
                    float v[32];
                    tmem_ld_32x32(tmem_acc + ((unsigned)(quarter * 32) << 16) + (unsigned)(half * BN + c), v);
                    if (nkb == 0) {                       // more splits than k-blocks: this one adds nothing (its accumulator was never written)
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                    }
                    // layout [split][tile][piece hc][column i][128 rows]: the 32 lanes of a warp write 32 consecutive floats
                    float* dst = partial + ((((size_t)split * tiles + tile_id) * ((BM / 128) * (BN / 32)) + hc) * 32) * 128 + quarter * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 32; ++i) dst[(size_t)i * 128] = v[i];
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const unsigned prev = atomicAdd(&counters[tile_id], 1u);
                    sm.is_last = (prev == (unsigned)(ksplit - 1)) ? 1 : 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (sm.is_last) {
                    __threadfence();
#pragma unroll 1
                    for (int hc = 0; hc < (BM / 128) * (BN / 32); ++hc) {
                        const int half = hc / (BN / 32), c = (hc - half * (BN / 32)) * 32;
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                        for (int sp = 0; sp < ksplit; ++sp) {
                            const float* src = partial + ((((size_t)sp * tiles + tile_id) * ((BM / 128) * (BN / 32)) + hc) * 32) * 128 + quarter * 32 + lane;
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += __ldcg(src + (size_t)i * 128);
                        }
                        emit(m0 + half * 128 + quarter * 32 + lane, c, v);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (warp == 2 && lane == 0) counters[tile_id] = 0;          // ready for the next launch
                }
            }
        }
    }
    __syncwarp();                    // the lanes that had no role wait for the one that had
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();          // neither CTA frees tensor memory or leaves while the other may still use it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (kPair) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(sm.tmem_base), "r"(kCols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(sm.tmem_base), "r"(kCols) : "memory");
    }
}

// ---- host side -----------------------------------------------------------

struct SplitWorkspace {
    float* partial = nullptr;
    size_t floats = 0;
    unsigned* counters = nullptr;
};
SplitWorkspace g_split_ws[16];
constexpr int kSplitCounters = 1 << 16;

// Workspace of the k-splits (prefill only: it may grow, so the first call of a size must not be under stream capture).
// A buffer that was outgrown is kept until the process ends: a captured graph may still hold its address.
int split_workspace(size_t floats, SplitWorkspace** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return li_fail("linear (tcgen05): cudaGetDevice: %s", cudaGetErrorString(e));
    LI_REQUIRE(dev >= 0 && dev < 16, "linear (tcgen05): device index %d out of range", dev);
    SplitWorkspace& w = g_split_ws[dev];
    if (!w.counters) {
        e = cudaMalloc(&w.counters, kSplitCounters * sizeof(unsigned));
        if (e == cudaSuccess) e = cudaMemset(w.counters, 0, kSplitCounters * sizeof(unsigned));
        if (e != cudaSuccess) return li_fail("linear (tcgen05): cannot allocate the tile counters: %s", cudaGetErrorString(e));
    }
    if (w.floats < floats) {
        float* nb = nullptr;
        size_t want = floats < (4u << 20) ? (4u << 20) : floats + floats / 2;
        e = cudaMalloc(&nb, want * sizeof(float));
        if (e != cudaSuccess) return li_fail("linear (tcgen05): cannot allocate %zu bytes for the k-splits: %s", want * sizeof(float), cudaGetErrorString(e));
        w.partial = nb;
        w.floats = want;
    }
    *out = &w;
    return 0;
}

template <int BM, int BN, typename Tout, bool kSwiglu, bool kPair = false, bool kRope = false>
int launch_tile(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream, int ksplit = 1,
                const RopeEpilogue& rope = RopeEpilogue{}) {
    EncodeTiledFn encode = nullptr;
    int *g_error_host = nullptr, *g_error_dev = nullptr;
    if (int rc = setup(&encode, &g_error_host, &g_error_dev)) return rc;
    if (*g_error_host != 0)
        return li_fail("linear (tcgen05): an earlier launch gave up waiting on a barrier (status %d); the results since then are invalid", *g_error_host);
    CUtensorMap map_a, map_w;
    if (int rc = make_map(&map_a, a, M, K, BM)) return rc;
    if (int rc = make_map(&map_w, w, N, K, Tile<BM, BN, kPair>::kRowsB)) return rc;
    const size_t smem = sizeof(SharedStorage<BM, BN, kPair>) + 1024;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BM, BN, Tout, kSwiglu, kPair, kRope>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return li_fail("linear (tcgen05): cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM), ksplit);
    if (kPair) {                                           // pairs along x; a tile of rows past the matrix reads zeros and stores nothing
        grid.x *= 2;
        grid.y = (grid.y + 1) / 2;
    }
    LI_REQUIRE(grid.y <= 65535, "linear (tcgen05): M=%d is too large for one launch", M);
    SplitWorkspace none, *ws = &none;
    if (ksplit > 1) {
        LI_REQUIRE((size_t)grid.x * grid.y <= (size_t)kSplitCounters, "linear (tcgen05): too many tiles for a split of k");
        if (int rc = split_workspace((size_t)ksplit * grid.x * grid.y * BM * BN, &ws)) return rc;
    }
    li_launch_pdl(gemm_tcgen05_kernel<BM, BN, Tout, kSwiglu, kPair, kRope>, grid, dim3(threads_of<kRope>()), smem, stream, dim3(kPair ? 2 : 1, 1, 1), map_a, map_w,
                  bias, (Tout*)out, M, N, K, g_error_dev, ws->partial, ws->counters, ksplit, rope);
    return li_check_launch("linear (tcgen05)");
}

// 256 x 256 tiles where they still fill most of the GPU (measured: better from about 120 CTAs on), else 128 x 128.
// tile: 0 chooses, 1 forces the small tile, 2 the large one (for tests and measurements).
template <typename Tout, bool kSwiglu>
int launch(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream, int tile) {
    const long long big_ctas = (long long)ceil_div(M, 256) * ceil_div(N, 256);
    const int nkb = ceil_div(K, BK);
    // few large tiles and a long k: split k so that the large tiles fill the GPU
    int ksplit = 1;
    if (big_ctas < 120 && big_ctas >= 24) {
        ksplit = (int)(148 / big_ctas);
        if (ksplit > nkb / 32) ksplit = nkb / 32;          // measured: worth it from about 32 k-blocks a split (down projection), not for k = 1536
        if (ksplit < 1) ksplit = 1;
    }
    if (g_forced_ksplit > 0) ksplit = g_forced_ksplit;
    // narrow products (q|k|v, o, down of a long step): pairs of CTAs on 256 x 256 (128 rows each, one accumulator) fill the GPU
    // in one wave without a split of k and its merge (measured at 2,048 rows: down 56 us against 73 us with the split,
    // q|k|v 17 us against 19 us on 256 x 128 tiles)
    const long long pair_rows = (ceil_div(M, 128) + 1) & ~1;
    const long long pair_ctas = pair_rows * ceil_div(N, 256), pair_ctas_192 = pair_rows * ceil_div(N, 192);
    // 192 columns a tile instead of 256 where that fills the waves of 148 CTAs clearly better (N = 1536: 8 column tiles
    // instead of 6; measured at 2,048 rows: down 52 us against 55 us, o 16 us against 18 us)
    auto wave_fill = [](long long ctas) { return (double)ctas / (double)(((ctas + 147) / 148) * 148); };
    const bool narrow = N % 192 == 0 && wave_fill(pair_ctas_192) > 1.1 * wave_fill(pair_ctas);
    const bool pairs = tile == 0 && big_ctas < 120 && g_forced_ksplit == 0 && pair_ctas >= 74 && M > 128;     // up to 128 rows the second CTA of a pair would have none
    if (tile == 7 || (pairs && narrow))
        return launch_tile<128, 192, Tout, kSwiglu, true>(a, w, bias, out, M, N, K, stream, g_forced_ksplit > 0 ? g_forced_ksplit : 1);
    if (tile == 5 || pairs)
        return launch_tile<128, 256, Tout, kSwiglu, true>(a, w, bias, out, M, N, K, stream, g_forced_ksplit > 0 ? g_forced_ksplit : 1);
    // half as many of them and a long k (down of about 1,000 rows): the same tiles with k split two or three ways
    // (measured at 1,024 rows: 39 us against 69 us on 256 x 256 tiles with four splits)
    if (tile == 0 && big_ctas < 120 && g_forced_ksplit == 0 && pair_ctas >= 40 && pair_ctas < 74 && nkb >= 64)
        return launch_tile<128, 256, Tout, kSwiglu, true>(a, w, bias, out, M, N, K, stream, (int)(148 / pair_ctas));
    if (tile == 8) return launch_tile<128, 64, Tout, kSwiglu>(a, w, bias, out, M, N, K, stream, g_forced_ksplit > 0 ? g_forced_ksplit : 1);
    if (tile == 9) return launch_tile<128, 32, Tout, kSwiglu>(a, w, bias, out, M, N, K, stream, g_forced_ksplit > 0 ? g_forced_ksplit : 1);
    const bool big = tile == 2 || tile == 4 || (tile == 0 && (big_ctas >= 120 || ksplit > 1));
    if (big && tile == 4) return launch_tile<256, 256, Tout, kSwiglu, true>(a, w, bias, out, M, N, K, stream, ksplit);
    if (big) return launch_tile<256, 256, Tout, kSwiglu>(a, w, bias, out, M, N, K, stream, ksplit);
    // few tiles of rows (a step of up to about 500 tokens) and a narrow product: the weights are the traffic, and 128 x 128
    // tiles are too few CTAs to stream them (q|k|v at 128 rows: 16).  Narrower column tiles, and a split of k where there
    // is room left, bring the count near one wave (measured at 128 / 256 / 512 rows, 40 launches in a graph: q|k|v 11.1 ->
    // 8.7, 11.4 -> 9.4, 11.7 -> 10.2 us; o 11.8 -> 8.0, 11.8 -> 9.5, 12.1 -> 10.7 us; down 25.3 -> 18.0, 25.5 -> 21.9 us
    // and unchanged from 384 rows on, where 128 x 128 tiles with four splits stay ahead)
    if (tile == 0 && g_forced_ksplit == 0) {
        const long long rows = ceil_div(M, 128);
        if (nkb < 32) {
            for (int bn = 32; bn <= 64; bn *= 2) {
                const long long ctas = rows * ceil_div(N, bn);
                if (ctas > 148) continue;
                int ks = (int)(148 / ctas);
                if (ks > nkb / 8) ks = nkb / 8;
                if (ks < 1) ks = 1;
                if (bn == 32) return launch_tile<128, 32, Tout, kSwiglu>(a, w, bias, out, M, N, K, stream, ks);
                return launch_tile<128, 64, Tout, kSwiglu>(a, w, bias, out, M, N, K, stream, ks);
            }
        } else if (rows <= 2) {
            const long long ctas = rows * ceil_div(N, 64);
            if (ctas * 2 <= 148) {
                int ks = (int)(148 / ctas);
                if (ks > nkb / 16) ks = nkb / 16;
                if (ks < 1) ks = 1;
                return launch_tile<128, 64, Tout, kSwiglu>(a, w, bias, out, M, N, K, stream, ks);
            }
        }
    }
    // narrow products with a short k (q|k|v, o): 256 x 128 tiles take in a quarter less per flop than 128 x 128, and
    // there are still enough of them to occupy most of the GPU; with no more than 128 rows their second half would be empty
    const long long mid_ctas = (long long)ceil_div(M, 256) * ceil_div(N, 128);
    if (tile == 3 || (tile == 0 && mid_ctas >= 74 && M > 128))
        return launch_tile<256, 128, Tout, kSwiglu>(a, w, bias, out, M, N, K, stream, g_forced_ksplit > 0 ? g_forced_ksplit : 1);
    // few small tiles and a long k (down of a short step): split k so that they fill the GPU, at least 16 k-blocks a split
    int small_split = 1;
    const long long small_ctas = (long long)ceil_div(M, 128) * ceil_div(N, 128);
    if (small_ctas < 74 && nkb >= 32) {
        small_split = (int)(148 / small_ctas);
        if (small_split > nkb / 16) small_split = nkb / 16;
        if (small_split < 1) small_split = 1;
    }
    return launch_tile<128, 128, Tout, kSwiglu>(a, w, bias, out, M, N, K, stream, g_forced_ksplit > 0 ? g_forced_ksplit : small_split);
}

int g_forced_tile = 0;

// whether `launch` takes paired tiles (one accumulator a CTA) for this shape by itself
bool pair_tiles_chosen(int M, int N, int K) {
    const long long big_ctas = (long long)ceil_div(M, 256) * ceil_div(N, 256);
    const long long pair_ctas = (long long)((ceil_div(M, 128) + 1) & ~1) * ceil_div(N, 256);
    (void)K;
    return g_forced_tile == 0 && g_forced_ksplit == 0 && big_ctas < 120 && pair_ctas >= 74 && M > 128;
}

}  // namespace

// The q|k|v product with rotary encoding and the cache writes as its epilogue (rope_epilogue.cuh): where the shape takes
// the paired tiles anyway, and on single 128 x 128 tiles (a head each) for steps too short for those: there the two
// kernels that would rotate and write the cache cost more than the narrower column tiles of the plain product gain.
int g_rope_single_tiles = 1;      // 0: the rope epilogue only on paired tiles (measurements)
LI_EXPORT void li_tcgen05_rope_single_tiles(int on) { g_rope_single_tiles = on; }

bool li_tcgen05_rope_wanted(const void* a, const void* w, const void* out, int M, int N, int K) {
    if (!li_tcgen05_accepts(a, w, out, LI_BF16, M, N, K) || N % 128 != 0 || li_tcgen05_persistent_wanted(M, N, K)) return false;
    return g_forced_tile == 0 && g_forced_ksplit == 0 && (g_rope_single_tiles || pair_tiles_chosen(M, N, K));
}

int li_linear_tcgen05_rope(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, const RopeEpilogue& rope,
                           cudaStream_t stream) {
    LI_REQUIRE(li_tcgen05_rope_wanted(a, w, out, M, N, K), "linear + rope (tcgen05): refuses M=%d N=%d K=%d", M, N, K);
    LI_REQUIRE(N == (rope.nh + 2 * rope.nkv) * 128 && rope.cos_sin && rope.slot_mapping && rope.kcache && rope.vcache,
               "linear + rope (tcgen05): N=%d does not match %d + 2 x %d heads of 128, or a null operand", N, rope.nh, rope.nkv);
    if (pair_tiles_chosen(M, N, K)) return launch_tile<128, 256, bf16, false, true, true>(a, w, bias, out, M, N, K, stream, 1, rope);
    return launch_tile<128, 128, bf16, false, false, true>(a, w, bias, out, M, N, K, stream, 1, rope);
}

// 0: tile size by shape; 1: 128 x 128 always; 2: 256 x 256 always, one CTA a tile; 3: 256 x 128 always; 4: pairs of CTAs on
// 512 x 256 (two accumulators each); 5: pairs of CTAs on 256 x 256 (one accumulator each); 6: the persistent kernel
// (gemm_tcgen05_persistent.cu); 7: pairs of CTAs on 256 x 192; 8: 128 x 64; 9: 128 x 32.  For tests and measurements.
LI_EXPORT void li_tcgen05_force_tile(int tile) { g_forced_tile = tile; }

// 0: splits of k by shape; n > 0: n splits always.  For tests and measurements.
LI_EXPORT void li_tcgen05_force_ksplit(int n) { g_forced_ksplit = n; }

bool li_tcgen05_accepts(const void* a, const void* w, const void* out, int dtype_out, int M, int N, int K) {
    return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0 && ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
           (dtype_out == LI_BF16 || dtype_out == LI_F32);
}

bool li_tcgen05_persistent_wanted(int M, int N, int K);
int li_linear_tcgen05_persistent(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K, int epilogue,
                                 cudaStream_t stream);

int li_linear_tcgen05(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                      int epilogue, cudaStream_t stream) {
    // wide products with a short k (gate|up): the persistent kernel, whose epilogue overlaps the next tile's products
    if (g_forced_tile == 6 || (g_forced_tile == 0 && g_forced_ksplit == 0 && li_tcgen05_persistent_wanted(M, N, K)))
        return li_linear_tcgen05_persistent(a, w, bias, out, dtype_out, M, N, K, epilogue, stream);
    if (epilogue == LI_EPILOGUE_SWIGLU) {
        LI_REQUIRE(N % 16 == 0 && bias == nullptr && dtype_out == LI_BF16,
                   "linear (tcgen05): the swiglu epilogue needs N a multiple of 16, no bias and bfloat16 output");
        return launch<bf16, true>(a, w, bias, out, M, N, K, stream, g_forced_tile);
    }
    if (dtype_out == LI_BF16) return launch<bf16, false>(a, w, bias, out, M, N, K, stream, g_forced_tile);
    if (dtype_out == LI_F32) return launch<float, false>(a, w, bias, out, M, N, K, stream, g_forced_tile);
    return li_fail("linear (tcgen05): unsupported output dtype %d", dtype_out);
}
