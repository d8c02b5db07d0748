// out[M, N] = a[M, K] w[N, K]^T (+ bias) in bfloat16 for few rows of a (M <= 64:
// decode), with the roles of the operands swapped on the fifth-generation
// tensor cores: 128 weight rows are the M side of tcgen05.mma, the tokens its N
// side (16, 32 or 64 columns of tensor memory).  The kernel is bound by reading
// every weight once; TMA streams 16 KB weight tiles through a ring of shared
// memory stages with no registers involved, which keeps more bytes in flight per
// multiprocessor than loads into registers can.
//
// Grid (tiles of 128 weight rows, splits of k).  Warp 0: producer (TMA), warp 1:
// tensor-memory allocation and MMA issue, warps 2-5: epilogue.  The weight tiles of
// the first stages are requested before griddepcontrol.wait (weights do not depend
// on the kernel before), the activation tiles after it.  With several splits each
// CTA writes its float partial tile to a workspace and the one that arrives last
// (a counter per tile) adds them in split order; the number of splits depends on N
// and K only, so a token's result does not depend on the batch it is in.
// Epilogue: bias, or the SwiGLU of gate and up rows interleaved in groups of 8
// (up * gate / (1 + exp(-gate)), src/ops/swiglu/op.cpp:17-23).
//
// K a multiple of 8; waits bounded as in the other tcgen05 kernel.
#define LI_PDL_KIND 2
#include "row_scale.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BR = 128;                  // weight rows per CTA
constexpr int kStages = 6;
constexpr int kThreads = 192;
constexpr int kTargetCtas = 148;
constexpr size_t kWorkspaceFloats = 4u << 20;
constexpr int kMaxTiles = 1 << 16;

template <int BT>
struct __align__(1024) Smem {
    unsigned char w[kStages][BR * BK * 2];
    unsigned char x[kStages][BT * BK * 2];
    unsigned long long full[kStages];
    unsigned long long empty[kStages];
    unsigned long long accum;
    unsigned tmem_base;
    int is_last;
    float factor[64];                // per token: the reciprocal root of the norm before this product
    float squares[4][64];            // per epilogue warp and token: sums of squares of the new residual values
};

struct Workspace {
    float* partial = nullptr;
    unsigned* counters = nullptr;
};
Workspace g_ws[16];

template <int N>
__device__ __forceinline__ void tmem_ld(unsigned taddr, float (&v)[N]);

template <>
__device__ __forceinline__ void tmem_ld<16>(unsigned taddr, float (&v)[16]) {
    unsigned r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

template <>
__device__ __forceinline__ void tmem_ld<32>(unsigned taddr, float (&v)[32]) { tmem_ld_32x32(taddr, v); }

template <>
__device__ __forceinline__ void tmem_ld<64>(unsigned taddr, float (&v)[64]) {
    float a[32], b[32];
    tmem_ld_32x32(taddr, a);
    tmem_ld_32x32(taddr + 32, b);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = a[i];
        v[32 + i] = b[i];
    }
}

enum { kEpiNone = 0, kEpiSwiglu = 1, kEpiAddScaled = 2 };

template <int BT, typename Tout, int kEpi>
__global__ void __launch_bounds__(kThreads)
gemv_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const float* __restrict__ bias, Tout* __restrict__ out, float* __restrict__ partial,
                    unsigned* __restrict__ counters, int M, int N, int K, int ksplit, int* __restrict__ error_flag, const RowScale rs,
                    const AddScaled add) {
    constexpr bool kSwiglu = kEpi == kEpiSwiglu, kAdd = kEpi == kEpiAddScaled;
    extern __shared__ unsigned char smem_raw[];
    Smem<BT>& sm = *reinterpret_cast<Smem<BT>*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int n0 = tile * BR;
    const int nkb_total = (K + BK - 1) / BK;
    const int kb0 = (int)((long long)split * nkb_total / ksplit), kb1 = (int)((long long)(split + 1) * nkb_total / ksplit);
    const int nkb = kb1 - kb0;
    constexpr unsigned kStageBytes = BR * BK * 2 + BT * BK * 2;
    constexpr unsigned kCols = BT < 32 ? 32 : BT;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        mbar_init(&sm.accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // (The other tcgen05 kernels take their tensor memory only after the kernel before them has finished, see
    // gemm_tcgen05.cu.  This one takes its 32 or 64 of the 512 columns at once: with the allocation behind the wait a decode
    // step of batch 8 went from 1.311 to 1.337 ms, and a CTA that holds so little while it waits leaves room for any other
    // kernel's CTAs; in all runs that stopped, this kernel launched plainly made no difference.)
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_acc = sm.tmem_base;
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // weights of the first stages at once; the activations once the kernel before has finished
            const int first = nkb < kStages ? nkb : kStages;
            for (int i = 0; i < first; ++i) {
                mbar_expect_tx(&sm.full[i], kStageBytes);
                tma_load_2d(sm.w[i], &map_w, (kb0 + i) * BK, n0, &sm.full[i]);
            }
            pdl_wait();
            for (int i = 0; i < first; ++i) tma_load_2d(sm.x[i], &map_x, (kb0 + i) * BK, 0, &sm.full[i]);
            bool ok = true;
            int issued = first;
            for (int i = first; i < nkb; ++i) {
                const int s = i % kStages;
                ok = mbar_wait(&sm.empty[s], ((i / kStages) & 1) ^ 1);
                if (!ok) break;
                mbar_expect_tx(&sm.full[s], kStageBytes);
                tma_load_2d(sm.w[s], &map_w, (kb0 + i) * BK, n0, &sm.full[s]);
                tma_load_2d(sm.x[s], &map_x, (kb0 + i) * BK, 0, &sm.full[s]);
                issued = i + 1;
            }
            if (!ok) {
                atomicExch(error_flag, 31);
                for (int i = (issued > kStages ? issued - kStages : 0); i < issued; ++i) mbar_wait(&sm.full[i % kStages], (i / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = umma_idesc(BR, BT);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % kStages;
                ok = mbar_wait(&sm.full[s], (i / kStages) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned long long da = umma_desc(sm.w[s]), db = umma_desc(sm.x[s]);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    umma_bf16(tmem_acc, da + (unsigned long long)(k * 2), db + (unsigned long long)(k * 2), idesc, (i | k) ? 1u : 0u);
                umma_commit(&sm.empty[s]);
            }
            if (ok) umma_commit(&sm.accum);
            else atomicExch(error_flag, 32);
        }
    } else {
        pdl_wait();
        const int quarter = warp & 3;
        const int r_in_tile = quarter * 32 + lane;
        const int row = n0 + r_in_tile;
        // while the weights stream: the tokens' factors from the partial sums of squares, and the old values of
        // the residual stream that the product will be added to (row_scale.cuh)
        if (rs.ssq) {
            // a warp takes every fourth token, eight tokens' loads in flight at once
            row_scales_of_warp<8>(rs, M, warp - 2, 4, lane, sm.factor);
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        float xold[kAdd ? BT : 1];
        if constexpr (kAdd) {
#pragma unroll
            for (int j = 0; j < BT; ++j) xold[j] = (j < M && row < N) ? __ldcg(add.x32 + (size_t)j * N + row) : 0.0f;
        }
        const bool ok = mbar_wait(&sm.accum, 0);
        if (!ok) {
            if (lane == 0) atomicExch(error_flag, 33);
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float v[BT];
            tmem_ld<BT>(tmem_acc + ((unsigned)(quarter * 32) << 16), v);
            bool write = true;
            if (ksplit > 1) {
                const size_t tiles = gridDim.x;
                float* mine = partial + (((size_t)split * tiles + tile) * BT) * BR + r_in_tile;
#pragma unroll
                for (int j = 0; j < BT; ++j)
                    if (j < M) mine[(size_t)j * BR] = v[j];
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const unsigned prev = atomicAdd(&counters[tile], 1u);
                    sm.is_last = (prev == (unsigned)(ksplit - 1));
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                write = sm.is_last != 0;
                if (write) {
                    __threadfence();
#pragma unroll
                    for (int j = 0; j < BT; ++j) v[j] = 0.0f;
                    // several splits' loads in flight at once (64 values a thread), added in split order
                    constexpr int SU = 64 / BT;
                    for (int s0 = 0; s0 < ksplit; s0 += SU) {
                        float p[SU][BT];
#pragma unroll
                        for (int u = 0; u < SU; ++u) {
                            const float* src = partial + (((size_t)(s0 + u) * tiles + tile) * BT) * BR + r_in_tile;
#pragma unroll
                            for (int j = 0; j < BT; ++j) p[u][j] = (s0 + u < ksplit && j < M) ? __ldcg(src + (size_t)j * BR) : 0.0f;
                        }
#pragma unroll
                        for (int u = 0; u < SU; ++u)
#pragma unroll
                            for (int j = 0; j < BT; ++j) v[j] += p[u][j];
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (warp == 2 && lane == 0) counters[tile] = 0;          // ready for the next launch on this stream
                }
            }
            if (write && rs.ssq) {
#pragma unroll
                for (int j = 0; j < BT; ++j)
                    if (j < M) v[j] *= sm.factor[j];
            }
            if (write) {
                if constexpr (kAdd) {
                    // into the residual stream, and on to the next product as bfloat16(norm_weight * x) with the sums of x^2
                    const float b = (bias && row < N) ? bias[row] : 0.0f;
                    const float nw = row < N ? add.norm_weight[row] : 0.0f;
#pragma unroll
                    for (int j = 0; j < BT; ++j) {
                        if (j < M) {                                       // uniform
                            const float x = row < N ? xold[j] + (v[j] + b) : 0.0f;
                            if (row < N) {
                                __stcg(add.x32 + (size_t)j * N + row, x);
                                add.hprime[(size_t)j * N + row] = __float2bfloat16_rn(nw * x);
                            }
                            const float sq = warp_sum(x * x);
                            if (lane == 0) sm.squares[quarter][j] = sq;
                        }
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const int tid = (int)threadIdx.x - 64;
                    if (tid < M)
                        add.ssq_out[(size_t)tid * gridDim.x + tile] = ((sm.squares[0][tid] + sm.squares[1][tid]) + sm.squares[2][tid]) + sm.squares[3][tid];
                } else if constexpr (!kSwiglu) {
                    const float b = (bias && row < N) ? bias[row] : 0.0f;
#pragma unroll
                    for (int j = 0; j < BT; ++j)
                        if (j < M && row < N) out[(size_t)j * N + row] = from_float<Tout>(v[j] + b);
                } else {
                    // rows come as 8 gate, 8 up, ...: lanes 0-7 and 16-23 hold gates, the lane 8 further on the matching up
                    const int half_n = N >> 1;
                    const int col = (row >> 4) * 8 + (row & 7);
#pragma unroll
                    for (int j = 0; j < BT; ++j) {
                        const float up = __shfl_down_sync(0xffffffffu, v[j], 8);
                        if (j < M && (lane & 8) == 0 && row + 8 < N) {
                            const float gate = v[j];
                            out[(size_t)j * half_n + col] = from_float<Tout>(swiglu_of<Tout>(gate, up));
                        }
                    }
                }
            }
        }
    }
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(kCols) : "memory");
    }
}

int ensure_workspace(Workspace** ws) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return li_fail("linear (tcgen05 gemv): cudaGetDevice: %s", cudaGetErrorString(e));
    LI_REQUIRE(dev >= 0 && dev < 16, "linear (tcgen05 gemv): device index %d out of range", dev);
    Workspace& w = g_ws[dev];
    if (!w.partial) {
        // first call on this device; must happen outside stream capture
        e = cudaMalloc(&w.partial, kWorkspaceFloats * sizeof(float));
        if (e != cudaSuccess) return li_fail("linear (tcgen05 gemv): cannot allocate the split-k workspace: %s", cudaGetErrorString(e));
        e = cudaMalloc(&w.counters, kMaxTiles * sizeof(unsigned));
        if (e == cudaSuccess) e = cudaMemset(w.counters, 0, kMaxTiles * sizeof(unsigned));
        if (e != cudaSuccess) return li_fail("linear (tcgen05 gemv): cannot allocate the tile counters: %s", cudaGetErrorString(e));
    }
    *ws = &w;
    return 0;
}

int g_forced_ksplit = 0;          // > 0: this many splits of k whatever the shape (measurements)

// Splits of k: a function of N, K and the token tile (16, 32 or 64 columns), never of the number of tokens itself.
int choose_ksplit(int N, int K, int bt) {
    const int tiles = ceil_div(N, BR), nkb = ceil_div(K, BK);
    int ks;
    if (g_forced_ksplit > 0) {
        ks = g_forced_ksplit < nkb ? g_forced_ksplit : nkb;
    } else {
        ks = kTargetCtas / tiles;
        if (ks < 1) ks = 1;
        if (bt == 64 && ks > 8) ks = 8;                               // 32 KB of partial sums a split: the merge by one CTA grows with them (measured)
        const int by_work = nkb / 2 > 0 ? nkb / 2 : 1;                // at least two k-blocks a CTA
        if (ks > by_work) ks = by_work;
    }
    while (ks > 1 && (size_t)ks * tiles * 64 * BR > kWorkspaceFloats) --ks;      // the partial sums fit the workspace: sized for 64 tokens whatever M is
    return ks;
}

template <int BT, typename Tout, int kEpi>
int launch(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream, const RowScale& rs,
           const AddScaled& add) {
    EncodeTiledFn encode = nullptr;
    int *err_host = nullptr, *err_dev = nullptr;
    if (int rc = setup(&encode, &err_host, &err_dev)) return rc;
    if (*err_host != 0)
        return li_fail("linear (tcgen05 gemv): an earlier launch gave up waiting on a barrier (status %d); the results since then are invalid", *err_host);
    Workspace* ws = nullptr;
    if (int rc = ensure_workspace(&ws)) return rc;
    const int tiles = ceil_div(N, BR);
    const int ksplit = choose_ksplit(N, K, BT);
    LI_REQUIRE(tiles <= kMaxTiles, "linear (tcgen05 gemv): N=%d has too many tiles", N);
    LI_REQUIRE(ksplit == 1 || (size_t)ksplit * tiles * BT * BR <= kWorkspaceFloats, "linear (tcgen05 gemv): %d splits of %d tiles do not fit the workspace",
               ksplit, tiles);
    CUtensorMap map_w, map_x;
    if (int rc = make_map(&map_w, w, N, K, BR)) return rc;
    if (int rc = make_map(&map_x, a, M, K, BT)) return rc;
    const size_t smem = sizeof(Smem<BT>) + 1024;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(gemv_tcgen05_kernel<BT, Tout, kEpi>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return li_fail("linear (tcgen05 gemv): cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    li_launch_pdl(gemv_tcgen05_kernel<BT, Tout, kEpi>, dim3(tiles, ksplit), dim3(kThreads), smem, stream, map_w, map_x, bias, (Tout*)out,
                  ws->partial, ws->counters, M, N, K, ksplit, err_dev, rs, add);
    return li_check_launch("linear (tcgen05 gemv)");
}

template <typename Tout, int kEpi>
int launch_bt(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream, const RowScale& rs,
              const AddScaled& add = AddScaled{}) {
    if (M <= 16) return launch<16, Tout, kEpi>(a, w, bias, out, M, N, K, stream, rs, add);
    if (M <= 32) return launch<32, Tout, kEpi>(a, w, bias, out, M, N, K, stream, rs, add);
    return launch<64, Tout, kEpi>(a, w, bias, out, M, N, K, stream, rs, add);
}

}  // namespace

// 0: splits of k by shape; n > 0: n splits always.  For measurements.
LI_EXPORT void li_gemv_tcgen05_force_ksplit(int n) { g_forced_ksplit = n; }

bool li_gemv_tcgen05_accepts(const void* a, const void* w, int M, int N, int K) {
    return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0 && ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0);
}

int li_linear_gemv_tcgen05(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                           int epilogue, cudaStream_t stream, const RowScale& rs) {
    LI_REQUIRE(li_gemv_tcgen05_accepts(a, w, M, N, K), "linear (tcgen05 gemv): refuses M=%d N=%d K=%d (M <= 64, K a multiple of 8, 16-byte aligned operands)", M, N, K);
    if (epilogue == LI_EPILOGUE_SWIGLU) {
        LI_REQUIRE(N % 16 == 0 && bias == nullptr && dtype_out == LI_BF16,
                   "linear (tcgen05 gemv): the swiglu epilogue needs N a multiple of 16, no bias and bfloat16 output");
        return launch_bt<bf16, kEpiSwiglu>(a, w, bias, out, M, N, K, stream, rs);
    }
    if (dtype_out == LI_BF16) return launch_bt<bf16, kEpiNone>(a, w, bias, out, M, N, K, stream, rs);
    if (dtype_out == LI_F32) return launch_bt<float, kEpiNone>(a, w, bias, out, M, N, K, stream, rs);
    return li_fail("linear (tcgen05 gemv): unsupported output dtype %d", dtype_out);
}

// x32 += a w^T (+ bias), hprime = bfloat16(norm_weight * x32), ssq_out[token, tile] = sums of squares (row_scale.cuh).
int li_gemv_tcgen05_tiles(int N) { return ceil_div(N, BR); }

int li_linear_gemv_tcgen05_add_scaled(const void* a, const void* w, const float* bias, int M, int N, int K, const AddScaled& add,
                                      cudaStream_t stream) {
    LI_REQUIRE(li_gemv_tcgen05_accepts(a, w, M, N, K), "linear + add (tcgen05 gemv): refuses M=%d N=%d K=%d", M, N, K);
    return launch_bt<bf16, kEpiAddScaled>(a, w, bias, add.hprime, M, N, K, stream, RowScale{}, add);
}
