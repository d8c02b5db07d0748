// out[M, N] = a[M, K] w[N, K]^T for wide products with a short k (gate|up of a prefill step): a persistent form of the
// tcgen05 GEMM in which the epilogue of one tile runs while the tensor cores work on the next.
//
// With k = 1536 a tile's main loop is only 24 k-blocks long; filling the pipeline and, above all, the epilogue (SwiGLU and
// the stores of a 256 x 256 tile) then cost as much as the products, and a kernel that does one tile per CTA cannot
// overlap them.  Here one pair of CTAs per pair of multiprocessors (a cluster of two, tcgen05.mma cta_group::2) walks over
// tiles of 256 x 256: each CTA brings its own 128 rows of a and half of the 256 rows of w per k-block (32 KB a stage, six
// stages) and keeps the accumulator of its rows, 256 columns of tensor memory.  The other 256 columns hold the tile before:
// the four epilogue warps of each CTA read it, apply bias or SwiGLU and store, while the first CTA's issuer already
// multiplies the next tile; the producers run ahead through the ring of stages without regard to tile boundaries.
// Tiles are taken in the order (row pair fastest, then columns), so that the pairs at work at one time share few tiles of w.
//
// Barriers: full / empty per stage as in gemm_tcgen05.cu (both CTAs' loads are counted on the first CTA's full barrier; the
// commit that frees a stage arrives in both); acc_full per accumulator (commit to both CTAs); acc_empty per accumulator in
// the first CTA, on which the epilogue warps of both CTAs arrive.  Every wait is bounded; a wait that runs out raises the
// status word of the tcgen05 kernels, and every role leaves its loops and meets the others at the final barriers.
#define LI_PDL_KIND 1
#include "gemm_epilogue.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int kRows = 128;          // rows of a per CTA
constexpr int BN = 256;             // columns of a tile
constexpr int kStages = 6;
constexpr int kThreads = 192;
constexpr int kBytesA = kRows * BK * 2, kBytesB = (BN / 2) * BK * 2;

__host__ __device__ constexpr int cdiv(int a, int b) { return (a + b - 1) / b; }

struct __align__(1024) Smem {
    unsigned char a[kStages][kBytesA];
    unsigned char b[kStages][kBytesB];
    unsigned long long full[kStages];
    unsigned long long empty[kStages];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned tmem_base;
};

template <typename Tout, bool kSwiglu>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                               const float* __restrict__ bias, Tout* __restrict__ out, int M, int N, int K, int* __restrict__ error_flag) {
    extern __shared__ unsigned char smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_cta_rank();
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int row_pairs = (cdiv(M, kRows) + 1) >> 1, col_tiles = cdiv(N, BN);
    const int total = row_pairs * col_tiles;
    const int nkb = cdiv(K, BK);
    constexpr unsigned kCols = 512;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.acc_full[b], 1);
            mbar_init(&sm.acc_empty[b], 8);          // four epilogue warps in each of the two CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Tensor memory is taken only once the kernel before this one has finished: a CTA that waits for that kernel must not
    // hold what a CTA of it may still ask for (gemm_tcgen05.cu has the story).  Nothing here could start before that anyway.
    pdl_launch_dependents();
    pdl_wait();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                               // the other CTA's barriers are set up before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_acc = sm.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            int it = 0;                               // k-blocks loaded so far, over all tiles
            for (int t = pair; t < total && ok; t += npairs) {
                const int m0 = ((t % row_pairs) * 2 + (int)rank) * kRows, n0 = (t / row_pairs) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % kStages;
                    ok = mbar_wait(&sm.empty[s], ((it / kStages) & 1) ^ 1);
                    if (!ok) break;
                    if (rank == 0) mbar_expect_tx(&sm.full[s], 2 * (kBytesA + kBytesB));
                    tma_load_2d_pair(sm.a[s], &map_a, kb * BK, m0, &sm.full[s]);
                    tma_load_2d_pair(sm.b[s], &map_w, kb * BK, n0 + (int)rank * (BN / 2), &sm.full[s]);
                }
            }
            if (!ok) atomicExch(error_flag, 21);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {                 // the first CTA issues the products of both
            constexpr unsigned idesc = umma_idesc(2 * kRows, BN);
            bool ok = true;
            int it = 0, ti = 0;
            for (int t = pair; t < total && ok; t += npairs, ++ti) {
                const unsigned acc = tmem_acc + (unsigned)((ti & 1) * BN);
                ok = mbar_wait(&sm.acc_empty[ti & 1], ((ti >> 1) & 1) ^ 1);     // both epilogues are done with this accumulator
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % kStages;
                    ok = mbar_wait(&sm.full[s], (it / kStages) & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned long long da = umma_desc(sm.a[s]), db = umma_desc(sm.b[s]);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_bf16_pair(acc, da + (unsigned long long)(k * 2), db + (unsigned long long)(k * 2), idesc, (kb | k) ? 1u : 0u);
                    umma_commit_pair(&sm.empty[s]);
                }
                if (ok) umma_commit_pair(&sm.acc_full[ti & 1]);
            }
            if (!ok) atomicExch(error_flag, 22);
        }
    } else {
        // epilogue: warp w may read the tensor-memory lanes 32 (w % 4) .. 32 (w % 4) + 31
        const int quarter = warp & 3;
        bool ok = true;
        int ti = 0;
        for (int t = pair; t < total && ok; t += npairs, ++ti) {
            const int m0 = ((t % row_pairs) * 2 + (int)rank) * kRows, n0 = (t / row_pairs) * BN;
            ok = mbar_wait(&sm.acc_full[ti & 1], (ti >> 1) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned acc = tmem_acc + ((unsigned)(quarter * 32) << 16) + (unsigned)((ti & 1) * BN);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                float v[32];
                tmem_ld_32x32(acc + (unsigned)c, v);
                gemm_store_piece<Tout, kSwiglu>(m0 + quarter * 32 + lane, n0 + c, v, bias, out, M, N);
            }
            // this warp has read its lanes of the accumulator: one arrival on the first CTA's barrier
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(&sm.acc_empty[ti & 1], 0);
        }
        if (!ok && lane == 0) atomicExch(error_flag, 23);
    }
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                               // neither CTA frees tensor memory or leaves while the other may still use it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(kCols) : "memory");
    }
}

template <typename Tout, bool kSwiglu>
int launch(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream) {
    EncodeTiledFn encode = nullptr;
    int *err_host = nullptr, *err_dev = nullptr;
    if (int rc = setup(&encode, &err_host, &err_dev)) return rc;
    if (*err_host != 0)
        return li_fail("linear (tcgen05, persistent): an earlier launch gave up waiting on a barrier (status %d); the results since then are invalid", *err_host);
    CUtensorMap map_a, map_w;
    if (int rc = make_map(&map_a, a, M, K, kRows)) return rc;
    if (int rc = make_map(&map_w, w, N, K, BN / 2)) return rc;
    const size_t smem = sizeof(Smem) + 1024;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<Tout, kSwiglu>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return li_fail("linear (tcgen05, persistent): cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms < 2) return li_fail("linear (tcgen05, persistent): cannot read the number of multiprocessors: %s", cudaGetErrorString(e));
    }
    const int total = ((ceil_div(M, kRows) + 1) / 2) * ceil_div(N, BN);
    int pairs = sms / 2;
    if (pairs > total) pairs = total;
    li_launch_pdl(gemm_tcgen05_persistent_kernel<Tout, kSwiglu>, dim3(2 * pairs), dim3(kThreads), smem, stream, dim3(2, 1, 1), map_a, map_w, bias,
                  (Tout*)out, M, N, K, err_dev);
    return li_check_launch("linear (tcgen05, persistent)");
}

}  // namespace

// Worth it when a pair of multiprocessors gets more than one tile and k is short enough for the epilogue to matter
// (measured: gate|up of 512 rows, 140 tiles: 29 us against 33 us; of 2,048 rows: 94 us against 138 us).
bool li_tcgen05_persistent_wanted(int M, int N, int K) {
    const long long total = (long long)((ceil_div(M, kRows) + 1) / 2) * ceil_div(N, BN);
    return total >= 120 && ceil_div(K, BK) <= 64;
}

int li_linear_tcgen05_persistent(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K, int epilogue,
                                 cudaStream_t stream) {
    if (epilogue == LI_EPILOGUE_SWIGLU) {
        LI_REQUIRE(N % 16 == 0 && bias == nullptr && dtype_out == LI_BF16,
                   "linear (tcgen05, persistent): the swiglu epilogue needs N a multiple of 16, no bias and bfloat16 output");
        return launch<bf16, true>(a, w, bias, out, M, N, K, stream);
    }
    if (dtype_out == LI_BF16) return launch<bf16, false>(a, w, bias, out, M, N, K, stream);
    if (dtype_out == LI_F32) return launch<float, false>(a, w, bias, out, M, N, K, stream);
    return li_fail("linear (tcgen05, persistent): unsupported output dtype %d", dtype_out);
}
