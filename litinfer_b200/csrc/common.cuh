// Shared helpers of the kernels: error reporting across the C interface,
// element types, 32-bit conversions and reductions.
//
// Every exported function returns 0 on success.  On failure it stores a
// message that li_last_error() returns, and launches nothing (or reports the
// launch error).  Arithmetic that the engine promises in 32-bit (norms,
// softmax, rotation angles, residual sums) uses float and the full-precision
// math functions; this library is compiled without fast-math.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#define LI_EXPORT extern "C" __attribute__((visibility("default")))

enum LiDtype : int { LI_F32 = 0, LI_BF16 = 1 };
// What a matrix product does to its result: nothing, or the SwiGLU of interleaved gate and up columns.
enum LiEpilogue : int { LI_EPILOGUE_NONE = 0, LI_EPILOGUE_SWIGLU = 1 };

int li_fail(const char* fmt, ...);            // stores the message, returns 1
int li_check_launch(const char* what);        // cudaGetLastError -> message

#define LI_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) return li_fail(__VA_ARGS__); \
    } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// The order of the additions is fixed by the block size, not by the data.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    r = warp_sum(r);
    return r;
}

// 2^x by the hardware approximation (about two units in the last place): used where the result is rounded to bfloat16
// right after (attention probabilities) while the running sums stay in float.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x without the special-function unit, for -125 <= x < 128 (below that it returns 2^-125, not 0): x = n + f with n the
// nearest integer (read off the low mantissa bits of x + 1.5 * 2^23) and |f| <= 1/2, 2^f by a quartic (relative error
// below 3e-6), n added to the exponent.  Where a kernel's exponentials outnumber what that unit delivers (16 a clock
// and multiprocessor), some of them go this way through the multiply-add pipe.
__device__ __forceinline__ float poly_exp2(float x) {
    x = fmaxf(x, -125.0f);
    const float t = x + 12582912.0f;
    const float f = x - (t - 12582912.0f);
    float p = 0.009570099413394928f;
    p = fmaf(p, f, 0.05591785907745361f);
    p = fmaf(p, f, 0.240247443318367f);
    p = fmaf(p, f, 0.6931217908859253f);
    p = fmaf(p, f, 0.9999992847442627f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

// up * gate / (1 + exp(-gate)) (src/ops/swiglu/op.cpp:17-23) in float.  For an output that is rounded to 16 bits the
// exponential and the quotient come from the fast units (errors near 2^-21, far below that rounding): an epilogue in which
// one warp works through its row alone is bound by the length of this chain of instructions.
template <typename Tout>
__device__ __forceinline__ float swiglu_of(float gate, float up) {
    if constexpr (sizeof(Tout) == 2) return up * __fdividef(gate, 1.0f + fast_exp2(-1.4426950408889634f * gate));
    else return up * (gate / (1.0f + expf(-gate)));
}

// Programmatic dependent launch.  A kernel launched through li_launch_pdl may begin while
// the kernel before it on the stream is still running; it must not touch memory that kernel
// writes (or still reads and this one overwrites) before pdl_wait(), which returns once the
// kernel before has finished and its writes are visible.  pdl_launch_dependents() lets the
// kernel after this one start being scheduled.  Both are no-ops for a plain launch.  Used on
// the decode path, where a step is a chain of short kernels and launch latency shows.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// LITINFER_B200_PDL=0 in the environment turns the overlap off (for measurements); LITINFER_B200_PDL_OFF=<mask> turns it
// off for the kernels of some source files only (LI_PDL_KIND of the file: 1 tcgen05 GEMM, 2 weight-streaming products,
// 4 attention, 8 the rest), to find which overlap a fault needs.
bool li_pdl_enabled(int kind);
#ifndef LI_PDL_KIND
#define LI_PDL_KIND 8
#endif

template <typename... KArgs, typename... Args>
static inline cudaError_t li_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = li_pdl_enabled(LI_PDL_KIND) ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the CTAs grouped into clusters of `cluster` (thread-block clusters: CTAs of a cluster run at the same
// time on neighbouring multiprocessors).  The grid must be a multiple of the cluster in every dimension.
template <typename... KArgs, typename... Args>
static inline cudaError_t li_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, dim3 cluster,
                                        Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = cluster.x;
        attr[na].val.clusterDim.y = cluster.y;
        attr[na].val.clusterDim.z = cluster.z;
        ++na;
    }
    if (li_pdl_enabled(LI_PDL_KIND)) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }
