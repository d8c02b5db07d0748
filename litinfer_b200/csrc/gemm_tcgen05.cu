// out[M, N] = a[M, K] w[N, K]^T (+ bias) in bfloat16 on the fifth-generation
// tensor cores: tcgen05.mma with both operands staged in shared memory by TMA
// and the float accumulator in tensor memory.  The prefill path of every
// projection (q|k|v, o, gate|up, down, lm_head).
//
// One CTA computes a 128 x BN tile (BN = 128).  Roles, by warp:
//   warp 0   producer: one lane issues the TMA loads of a 128 x 64 tile of a and
//            a BN x 64 tile of w per k-block (64 bfloat16 = one 128-byte swizzle
//            row) into a ring of stages, each guarded by a full/empty mbarrier pair;
//   warp 1   allocates BN columns of tensor memory; one lane issues four
//            tcgen05.mma (M 128, N BN, K 16) per k-block, commits the stage's
//            empty barrier, and at the end the accumulator's barrier;
//   warps 2-5 epilogue: tcgen05.ld of their quarter of the 128 lanes, bias in
//            float, one rounding, stores to global memory.
// Both operands are K-major ([rows, K] row-major), which is how activations and
// LitInfer-style [out, in] weights (src/ops/linear/cpu/linear_cpu.cpp:45-60)
// lie in memory; TMA zero-fills rows and columns beyond the tensor, so any M,
// N and any K that is a multiple of 8 (16-byte rows) work.  No cluster
// multicast is used.
//
// Every wait on an mbarrier is bounded.  A wait that runs out raises a flag in
// mapped host memory (li_tcgen05_status() reads it), the CTA waits, again
// bounded, for the copies it has in flight, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>

namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int kStages = 6;
constexpr int kStageBytesA = BM * BK * 2, kStageBytesB = BN * BK * 2;
constexpr int kThreads = 192;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;      // two seconds: far beyond any legitimate wait

struct __align__(1024) SharedStorage {
    unsigned char a[kStages][kStageBytesA];
    unsigned char b[kStages][kStageBytesB];
    unsigned long long full[kStages];
    unsigned long long empty[kStages];
    unsigned long long accum;
    unsigned tmem_base;
    int failed;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Bounded wait for the phase with the given parity; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    const unsigned addr = smem_u32(bar);
    unsigned long long t0 = 0;
    for (unsigned spin = 0;; ++spin) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spin & 255u) == 255u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) return false;
        }
        if (spin > (1u << 30)) return false;
    }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor: K-major tile of rows x 64 bfloat16 written by TMA
// with the 128-byte swizzle; 8-row groups are 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc(const void* tile) {
    const unsigned addr = smem_u32(tile);
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);         // start address
    d |= (unsigned long long)0 << 16;                           // leading byte offset: unused with this swizzle
    d |= (unsigned long long)(1024 >> 4) << 32;                 // stride byte offset
    d |= (unsigned long long)1 << 46;                           // descriptor version of this architecture
    d |= (unsigned long long)2 << 61;                           // 128-byte swizzle
    return d;
}

// Instruction descriptor of kind::f16: bfloat16 a and b, float accumulator, both K-major.
__host__ __device__ constexpr unsigned umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

template <typename Tout, bool kSwiglu>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, Tout* __restrict__ out, int M, int N, int K, int* __restrict__ error_flag) {
    extern __shared__ unsigned char smem_raw[];
    SharedStorage& sm = *reinterpret_cast<SharedStorage*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nkb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        mbar_init(&sm.accum, 1);
        sm.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"((unsigned)BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_acc = sm.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % kStages;
                const unsigned phase = (kb / kStages) & 1;
                ok = mbar_wait(&sm.empty[s], phase ^ 1);
                if (!ok) break;
                mbar_expect_tx(&sm.full[s], kStageBytesA + kStageBytesB);
                tma_load_2d(sm.a[s], &map_a, kb * BK, m0, &sm.full[s]);
                tma_load_2d(sm.b[s], &map_w, kb * BK, n0, &sm.full[s]);
                issued = kb + 1;
            }
            if (!ok) {
                sm.failed = 1;
                atomicExch(error_flag, 1);
                // the copies already issued must land before the CTA may leave
                for (int kb = (issued > kStages ? issued - kStages : 0); kb < issued; ++kb)
                    mbar_wait(&sm.full[kb % kStages], (kb / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = umma_idesc(BM, BN);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % kStages;
                const unsigned phase = (kb / kStages) & 1;
                ok = mbar_wait(&sm.full[s], phase);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned long long da = umma_desc(sm.a[s]), db = umma_desc(sm.b[s]);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    umma_bf16(tmem_acc, da + (unsigned long long)(k * 2), db + (unsigned long long)(k * 2), idesc, (kb | k) ? 1u : 0u);
                umma_commit(&sm.empty[s]);
            }
            if (ok) {
                umma_commit(&sm.accum);
            } else {
                sm.failed = 1;
                atomicExch(error_flag, 2);
            }
        }
    } else {
        // epilogue: warp w may read the tensor-memory lanes 32 (w % 4) .. 32 (w % 4) + 31
        const int quarter = warp & 3;
        const bool ok = mbar_wait(&sm.accum, 0);
        if (!ok) {
            if (lane == 0) atomicExch(error_flag, 3);
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                float v[32];
                tmem_ld_32x32(tmem_acc + ((unsigned)(quarter * 32) << 16) + (unsigned)c, v);
                const int col0 = n0 + c;
                if (kSwiglu) {
                    // columns come as 8 gate, 8 up, 8 gate, 8 up: 16 activations up * gate / (1 + exp(-gate))
                    if (row < M && col0 < N) {
                        const int half_n = N >> 1;
                        Tout* dst = out + (size_t)row * half_n + (col0 >> 1);
                        float a16[16];
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float gate = v[16 * h + i], up = v[16 * h + 8 + i];
                                a16[8 * h + i] = up * (gate / (1.0f + expf(-gate)));
                            }
                        if (col0 + 32 <= N && (((uintptr_t)dst) & 15) == 0 && sizeof(Tout) == 2) {
                            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                uint4 pk;
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(a16[8 * i + 0], a16[8 * i + 1]);
                                __nv_bfloat162 h1 = __floats2bfloat162_rn(a16[8 * i + 2], a16[8 * i + 3]);
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(a16[8 * i + 4], a16[8 * i + 5]);
                                __nv_bfloat162 h3 = __floats2bfloat162_rn(a16[8 * i + 6], a16[8 * i + 7]);
                                pk.x = *reinterpret_cast<unsigned*>(&h0);
                                pk.y = *reinterpret_cast<unsigned*>(&h1);
                                pk.z = *reinterpret_cast<unsigned*>(&h2);
                                pk.w = *reinterpret_cast<unsigned*>(&h3);
                                d4[i] = pk;
                            }
                        } else {
                            for (int i = 0; i < 16; ++i) {
                                const int src_col = col0 + 16 * (i >> 3) + (i & 7);      // the gate column of activation i
                                if (src_col + 8 < N) dst[i] = from_float<Tout>(a16[i]);
                            }
                        }
                    }
                } else if (row < M && col0 < N) {
                    Tout* dst = out + (size_t)row * N + col0;
                    if (col0 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
                        if (bias) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += bias[col0 + i];
                        }
                        if (sizeof(Tout) == 2) {
                            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                uint4 pk;
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * i + 0], v[8 * i + 1]);
                                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
                                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
                                pk.x = *reinterpret_cast<unsigned*>(&h0);
                                pk.y = *reinterpret_cast<unsigned*>(&h1);
                                pk.z = *reinterpret_cast<unsigned*>(&h2);
                                pk.w = *reinterpret_cast<unsigned*>(&h3);
                                d4[i] = pk;
                            }
                        } else {
                            float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
                            for (int i = 0; i < 8; ++i) d4[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                        }
                    } else {
                        for (int i = 0; i < 32 && col0 + i < N; ++i) dst[i] = from_float<Tout>(bias ? v[i] + bias[col0 + i] : v[i]);
                    }
                }
            }
        }
    }
    __syncwarp();                    // the lanes that had no role wait for the one that had
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((unsigned)BN) : "memory");
    }
}

// ---- host side -----------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode = nullptr;
int* g_error_host = nullptr;       // mapped pinned memory: the kernel writes, the host reads without a sync
int* g_error_dev = nullptr;
bool g_attr_set[3] = {false, false, false};

int setup() {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return li_fail("linear (tcgen05): the driver has no cuTensorMapEncodeTiled: %s", cudaGetErrorString(e));
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    if (!g_error_host) {
        cudaError_t e = cudaHostAlloc((void**)&g_error_host, sizeof(int), cudaHostAllocMapped);
        if (e != cudaSuccess) return li_fail("linear (tcgen05): cannot allocate the status word: %s", cudaGetErrorString(e));
        *g_error_host = 0;
        e = cudaHostGetDevicePointer((void**)&g_error_dev, g_error_host, 0);
        if (e != cudaSuccess) return li_fail("linear (tcgen05): cannot map the status word: %s", cudaGetErrorString(e));
    }
    return 0;
}

int make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return li_fail("linear (tcgen05): cuTensorMapEncodeTiled failed with %d for a [%d, %d] tensor", (int)r, rows, cols);
    return 0;
}

template <typename Tout, bool kSwiglu>
int launch(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream, int which) {
    if (int rc = setup()) return rc;
    if (*g_error_host != 0)
        return li_fail("linear (tcgen05): an earlier launch gave up waiting on a barrier (status %d); the results since then are invalid", *g_error_host);
    CUtensorMap map_a, map_w;
    if (int rc = make_map(&map_a, a, M, K, BM)) return rc;
    if (int rc = make_map(&map_w, w, N, K, BN)) return rc;
    const size_t smem = sizeof(SharedStorage) + 1024;
    if (!g_attr_set[which]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<Tout, kSwiglu>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return li_fail("linear (tcgen05): cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
        g_attr_set[which] = true;
    }
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
    LI_REQUIRE(grid.y <= 65535, "linear (tcgen05): M=%d is too large for one launch", M);
    gemm_tcgen05_kernel<Tout, kSwiglu><<<grid, kThreads, smem, stream>>>(map_a, map_w, bias, (Tout*)out, M, N, K, g_error_dev);
    return li_check_launch("linear (tcgen05)");
}

}  // namespace

bool li_tcgen05_accepts(const void* a, const void* w, const void* out, int dtype_out, int M, int N, int K) {
    return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0 && ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
           (dtype_out == LI_BF16 || dtype_out == LI_F32);
}

int li_linear_tcgen05(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                      int epilogue, cudaStream_t stream) {
    if (epilogue == LI_EPILOGUE_SWIGLU) {
        LI_REQUIRE(N % 16 == 0 && bias == nullptr && dtype_out == LI_BF16,
                   "linear (tcgen05): the swiglu epilogue needs N a multiple of 16, no bias and bfloat16 output");
        return launch<bf16, true>(a, w, bias, out, M, N, K, stream, 2);
    }
    if (dtype_out == LI_BF16) return launch<bf16, false>(a, w, bias, out, M, N, K, stream, 0);
    if (dtype_out == LI_F32) return launch<float, false>(a, w, bias, out, M, N, K, stream, 1);
    return li_fail("linear (tcgen05): unsupported output dtype %d", dtype_out);
}

// 0 while no launch of the tcgen05 kernel has given up a wait; else which role did
// (1 producer, 2 tensor-core issuer, 3 epilogue).  Meaningful after a synchronisation.
LI_EXPORT int li_tcgen05_status() { return g_error_host ? *g_error_host : 0; }
