// out[M, N] = a[M, K] w[N, K]^T (+ bias) in bfloat16 for few rows of a
// (decode: M = number of sequences): a kernel that is bound by reading every
// weight once from HBM.
//
// Swap of the usual roles: 16 rows of the weight matrix are the M side of a
// tensor-core tile (mma.sync m16n8k16, bfloat16 in, float accumulate), the
// tokens are its N side (8 per tile, up to 8 tiles).  Both operands are read
// with 16-byte loads straight from global memory into fragment registers: the
// sum over k does not care about the order of k, so the 8 consecutive
// elements a thread loads are taken as the k-pairs the fragment layout wants,
// the same permutation on both operands.  Weights stream past L1 (ld.global.cs);
// the activations (a few KB) stay in L1.
//
// A CTA of 4, 8 or 16 warps owns 16 weight rows and a range of k; each warp a
// contiguous sub-range.  Warps are summed through shared memory in fixed
// order.  When 16-row tiles alone do not fill the GPU, k is split over
// several CTAs (split count depends on N and K only, never on M): each writes
// float partial sums to a workspace, and the CTA that arrives last (a counter
// per tile) adds them in split order.  Within this kernel a token's result
// therefore does not depend on how many other tokens are in the batch; which
// kernel a product goes to does depend on the step's size (linear.cu), so across
// those choices a token's result is the same up to rounding only.
//
// Requires K % 8 == 0 and 16-byte aligned operands; M <= 64.
#define LI_PDL_KIND 2
#include "common.cuh"
#include "no_alloc.h"
#include "gemv_epilogue.cuh"
#include "row_scale.cuh"

#include <mutex>

namespace {

constexpr int kMaxM = 64;
constexpr size_t kWorkspaceFloats = 4u << 20;     // 16 MB of partial sums
constexpr int kMaxTiles = 1 << 16;
constexpr int kTargetCtas = 1480;                 // about ten CTAs a multiprocessor keep enough loads in flight

struct Workspace {
    float* partial = nullptr;
    unsigned* counters = nullptr;
};
Workspace g_ws[16];

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint4 ld_cached(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

enum { kEpiNone = 0, kEpiSwiglu = 1, kEpiRope = 2, kEpiAddScaled = 3 };

template <int NT, int WARPS, typename Tout, int kEpi>
__global__ void __launch_bounds__(WARPS * 32)
gemv_bf16_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, const float* __restrict__ bias, Tout* __restrict__ out,
                 float* __restrict__ partial, unsigned* __restrict__ counters, int M, int N, int K, int ksplit, const RopeArgs rope,
                 const RowScale rs, const AddScaled add) {
    constexpr bool kSwiglu = kEpi == kEpiSwiglu;
    extern __shared__ float red_raw[];                 // [WARPS][NT * 128]
    float (*red)[NT * 128] = reinterpret_cast<float (*)[NT * 128]>(red_raw);
    __shared__ int is_last;
    __shared__ float rs_sm[NT * 8];
    const int tile = blockIdx.x, split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = tile * 16;
    const int chunks = (K + 31) >> 5;
    const int c_begin = (int)((long long)split * chunks / ksplit), c_end = (int)((long long)(split + 1) * chunks / ksplit);
    const int span = c_end - c_begin;
    const int wb = c_begin + (int)((long long)warp * span / WARPS), we = c_begin + (int)((long long)(warp + 1) * span / WARPS);

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;

    int r0 = n0 + g, r1 = n0 + g + 8;
    if (kEpi == kEpiRope) {
        const int tiles_per_head = rope.dh >> 4;
        const int head = tile / tiles_per_head, jt = tile - head * tiles_per_head;
        r0 = head * rope.dh + jt * 8 + g;
        r1 = r0 + (rope.dh >> 1);
    }
    const bool v0 = r0 < N, v1 = r1 < N;
    const bf16* w0 = W + (size_t)(v0 ? r0 : 0) * K;
    const bf16* w1 = W + (size_t)(v1 ? r1 : 0) * K;
    const uint4 zero = make_uint4(0, 0, 0, 0);

    // Weights do not depend on the kernel before this one: the first round of loads is issued
    // before waiting for it (programmatic dependent launch), the activations after.  Later
    // rounds are fetched one ahead of the round being multiplied.
    constexpr int U = 4;
    uint4 a[U], b[U], an[U], bn[U];
    auto load_w = [&](uint4 (&wa)[U], uint4 (&wb2)[U], int c) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = ((c + u) << 5) + t * 8;
            const bool ok = (c + u) < we && k < K;
            wa[u] = (ok && v0) ? ld_stream(w0 + k) : zero;
            wb2[u] = (ok && v1) ? ld_stream(w1 + k) : zero;
        }
    };
    pdl_launch_dependents();
    load_w(a, b, wb);
    pdl_wait();
    // What the epilogue needs from memory is asked for now and used after the weights have streamed past: the partial
    // sums of squares for the tokens' factors (when a lane has at most kPre parts per token), and the old values of
    // the residual stream.
    constexpr int kPre = 4;                                          // parts a lane holds per token: up to 128 parts
    constexpr int kTok = NT * 8 > WARPS ? NT * 8 / WARPS : 1;        // tokens a warp computes the factor of
    float pre[kTok][kPre];
    const bool pre_fits = rs.ssq != nullptr && rs.nparts <= 32 * kPre;
#pragma unroll
    for (int ti = 0; ti < kTok; ++ti) {
        const int tok = warp + ti * WARPS;
#pragma unroll
        for (int q = 0; q < kPre; ++q) {
            const int p = lane + 32 * q;
            pre[ti][q] = (pre_fits && tok < M && p < rs.nparts) ? __ldcg(rs.ssq + (size_t)tok * rs.nparts + p) : 0.0f;
        }
    }
    // Many tokens: registers are short, so the factors are finished here, behind one round trip that the first weights
    // (already on their way) cover; few tokens: after the loop.
    constexpr bool kFactorsFirst = NT >= 4;
    auto finish_factors = [&]() {
#pragma unroll
        for (int ti = 0; ti < kTok; ++ti) {
            const int tok = warp + ti * WARPS;
            const float ssum = warp_sum(((pre[ti][0] + pre[ti][1]) + pre[ti][2]) + pre[ti][3]);
            if (lane == 0 && tok < M) rs_sm[tok] = 1.0f / sqrtf(ssum / rs.width + rs.eps);
        }
    };
    if (kFactorsFirst && pre_fits) finish_factors();
    constexpr int kXPre = kEpi == kEpiAddScaled ? (NT * 128 + WARPS * 32 - 1) / (WARPS * 32) : 1;
    float xpre[kXPre];
    if constexpr (kEpi == kEpiAddScaled) {
#pragma unroll
        for (int q = 0; q < kXPre; ++q) {
            const int e = threadIdx.x + q * WARPS * 32;
            const int l = e & 31, ji = e >> 5, i = ji & 3, j = ji >> 2;
            const int row = n0 + (l >> 2) + ((i >> 1) << 3), tok = j * 8 + ((l & 3) << 1) + (i & 1);
            xpre[q] = (e < NT * 128 && row < N && tok < M) ? __ldcg(add.x32 + (size_t)tok * N + row) : 0.0f;
        }
    }
    for (int c = wb; c < we; c += U) {
        if (c + U < we) load_w(an, bn, c + U);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = ((c + u) << 5) + t * 8;
            const bool ok = (c + u) < we && k < K;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int tok = j * 8 + g;
                const uint4 x = (ok && tok < M) ? ld_cached(X + (size_t)tok * K + k) : zero;
                mma_bf16(acc[j], a[u].x, b[u].x, a[u].y, b[u].y, x.x, x.y);
                mma_bf16(acc[j], a[u].z, b[u].z, a[u].w, b[u].w, x.z, x.w);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            a[u] = an[u];
            b[u] = bn[u];
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][(j * 4 + i) * 32 + lane] = acc[j][i];
    if (rs.ssq) {
        // the tokens' factors; the same order of summation either way (a lane's parts ascending, then the butterfly)
        if (pre_fits) {
            if (!kFactorsFirst) finish_factors();
        } else {
            row_scales_of_warp<1>(rs, M, warp, WARPS, lane, rs_sm);
        }
    }
    const float* factors = rs.ssq ? rs_sm : nullptr;
    __syncthreads();

    auto warps_sum = [&](int e) {
        float v = red[0][e];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) v += red[w][e];
        return v;
    };
    if (kEpi == kEpiRope) {
        store_rope<NT>(warps_sum, bias, reinterpret_cast<bf16*>(out), tile, M, N, rope, (int)threadIdx.x, WARPS * 32, factors);       // never split along k
        return;
    }
    auto finish = [&](auto get) {
        if constexpr (kEpi == kEpiAddScaled) {
            __shared__ float tile_sm[NT * 8 * 16];
            store_add_scaled<NT>(get, bias, add, xpre, tile, (int)gridDim.x, M, N, (int)threadIdx.x, WARPS * 32, tile_sm, [] { __syncthreads(); });
        } else {
            store_elements<NT, Tout, kSwiglu>(get, bias, out, n0, M, N, (int)threadIdx.x, WARPS * 32, factors);
        }
    };
    if (ksplit == 1) {
        finish(warps_sum);
        return;
    }
    const size_t pbase = ((size_t)split * gridDim.x + tile) * (NT * 128);
    for (int e = threadIdx.x; e < NT * 128; e += WARPS * 32) partial[pbase + e] = warps_sum(e);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(&counters[tile], 1u);
        is_last = (prev == (unsigned)(ksplit - 1));
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const size_t tiles = gridDim.x;
    auto splits_sum = [&](int e) {
        float v = 0.0f;
        for (int s = 0; s < ksplit; ++s) v += __ldcg(&partial[((size_t)s * tiles + tile) * (NT * 128) + e]);
        return v;
    };
    if (threadIdx.x == 0) counters[tile] = 0;          // ready for the next launch on this stream
    finish(splits_sum);
}

int ensure_workspace(Workspace** ws) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return li_fail("linear (gemv): cudaGetDevice: %s", cudaGetErrorString(e));
    LI_REQUIRE(dev >= 0 && dev < 16, "linear (gemv): device index %d out of range", dev);
    Workspace& w = g_ws[dev];
    if (!w.partial) {
        // first call on this device; must happen outside stream capture
        e = cudaMalloc(&w.partial, kWorkspaceFloats * sizeof(float));
        if (e != cudaSuccess) return li_fail("linear (gemv): cannot allocate the split-k workspace: %s", cudaGetErrorString(e));
        e = cudaMalloc(&w.counters, kMaxTiles * sizeof(unsigned));
        if (e == cudaSuccess) e = cudaMemset(w.counters, 0, kMaxTiles * sizeof(unsigned));
        if (e != cudaSuccess) return li_fail("linear (gemv): cannot allocate the tile counters: %s", cudaGetErrorString(e));
    }
    *ws = &w;
    return 0;
}

// How a product is cut: warps per CTA (each warp should have about four 32-element chunks
// of k per round of loads) and CTAs along k.  Depends on N and K only, never on M.
void choose_shape(int ntiles, int K, int nt, int* warps, int* ksplit) {
    const int chunks = (K + 31) / 32;
    int w = 4;
    if (ntiles < kTargetCtas) w = chunks >= 48 ? 16 : (chunks >= 24 ? 8 : 4);
    else if (ntiles < 4 * kTargetCtas && chunks >= 32) w = 8;
    (void)nt;
    int ks = 1;
    const int ctas_wanted = kTargetCtas * 4 / w;
    if (ntiles < ctas_wanted) {
        ks = ceil_div(ctas_wanted, ntiles);
        const int by_work = chunks / (w * 4) > 0 ? chunks / (w * 4) : 1;  // at least four chunks a warp
        if (ks > by_work) ks = by_work;
    }
    while (ks > 1 && (size_t)ks * ntiles * 8 * 128 > kWorkspaceFloats) --ks;      // sized for 64 tokens whatever M is
    *warps = w;
    *ksplit = ks;
}

template <int NT, int WARPS, typename Tout, int kEpi>
int launch_kernel(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, int ksplit, Workspace* ws,
                  cudaStream_t stream, const RopeArgs& rope = RopeArgs{}, const RowScale& rs = RowScale{}, const AddScaled& add = AddScaled{}) {
    constexpr int kSwiglu = kEpi;
    dim3 grid(ceil_div(N, 16), ksplit);
    constexpr size_t smem = (size_t)WARPS * NT * 128 * sizeof(float);
    if (smem > 48 * 1024) {
        static bool raised = false;
        if (!raised) {
            cudaError_t e = cudaFuncSetAttribute(gemv_bf16_kernel<NT, WARPS, Tout, kSwiglu>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return li_fail("linear (gemv): cannot raise shared memory to %zu: %s", smem, cudaGetErrorString(e));
            raised = true;
        }
    }
    li_launch_pdl(gemv_bf16_kernel<NT, WARPS, Tout, kSwiglu>, grid, dim3(WARPS * 32), smem, stream, (const bf16*)a, (const bf16*)w, bias,
                  (Tout*)out, ws->partial, ws->counters, M, N, K, ksplit, rope, rs, add);
    return li_check_launch("linear (gemv)");
}

template <int NT, typename Tout, int kEpi>
int launch(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream, const RowScale& rs,
           const AddScaled& add = AddScaled{}) {
    const int ntiles = ceil_div(N, 16);
    int warps = 4, ksplit = 1;
    choose_shape(ntiles, K, NT, &warps, &ksplit);
    Workspace* ws = nullptr;
    if (int rc = ensure_workspace(&ws)) return rc;
    LI_REQUIRE(ntiles <= kMaxTiles || ksplit == 1, "linear (gemv): N=%d has too many tiles for split-k", N);
    if (warps == 16) return launch_kernel<NT, 16, Tout, kEpi>(a, w, bias, out, M, N, K, ksplit, ws, stream, RopeArgs{}, rs, add);
    if (warps >= 8) return launch_kernel<NT, 8, Tout, kEpi>(a, w, bias, out, M, N, K, ksplit, ws, stream, RopeArgs{}, rs, add);
    return launch_kernel<NT, 4, Tout, kEpi>(a, w, bias, out, M, N, K, ksplit, ws, stream, RopeArgs{}, rs, add);
}

template <typename Tout, int kEpi>
int launch_nt(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream, const RowScale& rs,
              const AddScaled& add = AddScaled{}) {
    if (M <= 8) return launch<1, Tout, kEpi>(a, w, bias, out, M, N, K, stream, rs, add);
    if (M <= 16) return launch<2, Tout, kEpi>(a, w, bias, out, M, N, K, stream, rs, add);
    if (M <= 32) return launch<4, Tout, kEpi>(a, w, bias, out, M, N, K, stream, rs, add);
    return launch<8, Tout, kEpi>(a, w, bias, out, M, N, K, stream, rs, add);
}

template <int NT>
int launch_rope(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, const RopeArgs& rope, const RowScale& rs,
                cudaStream_t stream) {
    const int ntiles = ceil_div(N, 16);
    int warps = 4, ksplit = 1;
    choose_shape(ntiles, K, NT, &warps, &ksplit);
    Workspace* ws = nullptr;
    if (int rc = ensure_workspace(&ws)) return rc;
    // the epilogue needs both halves of a pair in one CTA and the whole sum: no split along k
    if (warps == 16) return launch_kernel<NT, 16, bf16, kEpiRope>(a, w, bias, out, M, N, K, 1, ws, stream, rope, rs);
    if (warps >= 8) return launch_kernel<NT, 8, bf16, kEpiRope>(a, w, bias, out, M, N, K, 1, ws, stream, rope, rs);
    return launch_kernel<NT, 4, bf16, kEpiRope>(a, w, bias, out, M, N, K, 1, ws, stream, rope, rs);
}

}  // namespace

// The fused q|k|v projection with rotary encoding and cache write in its epilogue, for few tokens.
bool li_gemv_rope_accepts(const void* a, const void* w, int M, int N, int K, int nh, int nkv, int dh, int rotary_dim) {
    return M >= 1 && M <= kMaxM && K % 8 == 0 && dh % 16 == 0 && rotary_dim == dh && N == (nh + 2 * nkv) * dh &&
           ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0);
}

int li_linear_gemv_rope(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, const int* positions,
                        const float* denom, const int* slot_mapping, void* kcache, void* vcache, int nh, int nkv, int dh,
                        int page_size, int num_pages, int write, const RowScale& rs, cudaStream_t stream) {
    RopeArgs ra{positions, denom, slot_mapping, (bf16*)kcache, (bf16*)vcache, nh, nkv, dh, page_size, num_pages, write};
    if (M <= 8) return launch_rope<1>(a, w, bias, out, M, N, K, ra, rs, stream);
    if (M <= 16) return launch_rope<2>(a, w, bias, out, M, N, K, ra, rs, stream);
    if (M <= 32) return launch_rope<4>(a, w, bias, out, M, N, K, ra, rs, stream);
    return launch_rope<8>(a, w, bias, out, M, N, K, ra, rs, stream);
}

bool li_gemv_bf16_accepts(int M, int N, int K) { return M >= 1 && M <= kMaxM && K % 8 == 0 && N >= 1; }

int li_linear_gemv_bf16(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                        int epilogue, cudaStream_t stream, const RowScale& rs) {
    LI_REQUIRE(li_gemv_bf16_accepts(M, N, K), "linear (gemv): refuses M=%d N=%d K=%d (M <= %d, K a multiple of 8)", M, N, K, kMaxM);
    LI_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0), "linear (gemv): operands must be 16-byte aligned");
    if (epilogue == LI_EPILOGUE_SWIGLU) {
        LI_REQUIRE(N % 16 == 0 && bias == nullptr && dtype_out == LI_BF16,
                   "linear (gemv): the swiglu epilogue needs N a multiple of 16, no bias and bfloat16 output");
        return launch_nt<bf16, kEpiSwiglu>(a, w, bias, out, M, N, K, stream, rs);
    }
    if (dtype_out == LI_BF16) return launch_nt<bf16, kEpiNone>(a, w, bias, out, M, N, K, stream, rs);
    if (dtype_out == LI_F32) return launch_nt<float, kEpiNone>(a, w, bias, out, M, N, K, stream, rs);
    return li_fail("linear (gemv): unsupported output dtype %d", dtype_out);
}

// x32 += a w^T (+ bias), hprime = bfloat16(norm_weight * x32), ssq_out[token, tile] = sums of squares (row_scale.cuh).
int li_gemv_bf16_tiles(int N) { return ceil_div(N, 16); }

int li_linear_gemv_bf16_add_scaled(const void* a, const void* w, const float* bias, int M, int N, int K, const AddScaled& add,
                                   cudaStream_t stream) {
    LI_REQUIRE(li_gemv_bf16_accepts(M, N, K), "linear + add (gemv): refuses M=%d N=%d K=%d (M <= %d, K a multiple of 8)", M, N, K, kMaxM);
    LI_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0), "linear + add (gemv): operands must be 16-byte aligned");
    return launch_nt<bf16, kEpiAddScaled>(a, w, bias, add.hprime, M, N, K, stream, RowScale{}, add);
}

// ---- the entry point that allocates nothing (no_alloc.h) ---------------------------------

namespace {

// Scratch of li_linear_gemv_static.  In host code these names are stand-ins, not device
// addresses: the addresses come from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) float g_static_partial[LI_STATIC_PARTIAL_FLOATS];
static __device__ __align__(256) unsigned g_static_counters[LI_STATIC_TILES];

Workspace g_static_ws[16];
std::mutex g_static_lock;

int static_workspace(Workspace** ws) {
    std::lock_guard<std::mutex> guard(g_static_lock);      // two host threads may make their first call together
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return li_fail("linear (gemv, static scratch): cudaGetDevice: %s", cudaGetErrorString(e));
    LI_REQUIRE(dev >= 0 && dev < 16, "linear (gemv, static scratch): device index %d out of range", dev);
    Workspace& w = g_static_ws[dev];
    if (!w.partial) {
        // first call on this device (it is the current one): ask where the arrays live on it
        void *p = nullptr, *c = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_partial);
        if (e != cudaSuccess) return li_fail("linear (gemv, static scratch): cudaGetSymbolAddress(partial): %s", cudaGetErrorString(e));
        e = cudaGetSymbolAddress(&c, g_static_counters);
        if (e != cudaSuccess) return li_fail("linear (gemv, static scratch): cudaGetSymbolAddress(counters): %s", cudaGetErrorString(e));
        w.counters = static_cast<unsigned*>(c);
        w.partial = static_cast<float*>(p);
    }
    *ws = &w;
    return 0;
}

template <int NT, typename Tout>
int launch_static(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream) {
    const int ntiles = ceil_div(N, 16);
    int warps = 4, ksplit = 1;
    choose_shape(ntiles, K, NT, &warps, &ksplit);
    Workspace* ws = nullptr;
    if (int rc = static_workspace(&ws)) return rc;
    if (ksplit > 1) {
        LI_REQUIRE(ntiles <= LI_STATIC_TILES && (size_t)ksplit * ntiles * NT * 128 <= LI_STATIC_PARTIAL_FLOATS,
                   "linear (gemv, static scratch): M=%d N=%d K=%d needs %zu floats of partial sums and %d counters; the built-in scratch holds %u and %d",
                   M, N, K, (size_t)ksplit * ntiles * NT * 128, ntiles, (unsigned)LI_STATIC_PARTIAL_FLOATS, LI_STATIC_TILES);
        // the arrays keep what the last call left: the counters of this call's tiles start at zero
        cudaError_t e = cudaMemsetAsync(ws->counters, 0, (size_t)ntiles * sizeof(unsigned), stream);
        if (e != cudaSuccess) return li_fail("linear (gemv, static scratch): clearing the counters: %s", cudaGetErrorString(e));
    }
    if (warps == 16) return launch_kernel<NT, 16, Tout, kEpiNone>(a, w, bias, out, M, N, K, ksplit, ws, stream);
    if (warps >= 8) return launch_kernel<NT, 8, Tout, kEpiNone>(a, w, bias, out, M, N, K, ksplit, ws, stream);
    return launch_kernel<NT, 4, Tout, kEpiNone>(a, w, bias, out, M, N, K, ksplit, ws, stream);
}

template <typename Tout>
int launch_static_nt(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, cudaStream_t stream) {
    if (M <= 8) return launch_static<1, Tout>(a, w, bias, out, M, N, K, stream);
    if (M <= 16) return launch_static<2, Tout>(a, w, bias, out, M, N, K, stream);
    if (M <= 32) return launch_static<4, Tout>(a, w, bias, out, M, N, K, stream);
    return launch_static<8, Tout>(a, w, bias, out, M, N, K, stream);
}

}  // namespace

LI_EXPORT int li_linear_gemv_static(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int K,
                                    cudaStream_t stream) {
    LI_REQUIRE(a && w && out, "linear (gemv, static scratch): null operand");
    LI_REQUIRE(li_gemv_bf16_accepts(M, N, K), "linear (gemv, static scratch): refuses M=%d N=%d K=%d (1 <= M <= %d, K a multiple of 8)", M, N, K, kMaxM);
    LI_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0), "linear (gemv, static scratch): operands must be 16-byte aligned");
    if (dtype_out == LI_BF16) return launch_static_nt<bf16>(a, w, bias, out, M, N, K, stream);
    if (dtype_out == LI_F32) return launch_static_nt<float>(a, w, bias, out, M, N, K, stream);
    return li_fail("linear (gemv, static scratch): unsupported output dtype %d", dtype_out);
}
