// Embedding gather, RMSNorm (plain, fused with the residual add, gathered
// rows), residual add and SwiGLU.
//
// RMSNorm per row: ss = sum x_j^2; r = 1 / sqrt(ss / H + eps); y_j = (w_j x_j) r,
// all in float, one rounding of y (LitInfer: src/ops/rms_norm/op.cpp:13-24).
// SwiGLU: up * gate / (1 + exp(-gate)) (src/ops/swiglu/op.cpp:17-23).
// One block per row; every thread owns the elements j = tid, tid + B, ... in
// both passes, so the second pass re-reads only what the same thread wrote.
#include "common.cuh"

namespace {

constexpr int kRowThreads = 256;

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out, int H, int V) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);          // ids are validated on the host; never read outside the table
    const T* row = table + (size_t)id * H;
    float* dst = out + (size_t)t * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) dst[j] = to_float(row[j]);
}

// mode 0: y = norm(x[row]); mode 1: x[row] += delta[row] first (stored back).
template <typename T, bool kAdd>
__global__ void rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const int* __restrict__ rows,
                               const float* __restrict__ w, float eps, T* __restrict__ out, int H, int T_rows) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    if (src < 0 || src >= T_rows) src = 0;
    float* xr = x + (size_t)src * H;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = xr[j];
        if (kAdd) {
            v += to_float(delta[(size_t)src * H + j]);
            xr[j] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = from_float<T>((w[j] * xr[j]) * rinv);
}

// The same for widths that are a multiple of 4 and fit 4 float4 a thread: the row stays in
// registers between the sum of squares and the scaling, and all loads are 16 bytes wide.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const unsigned*>(&a);
    r.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

constexpr int kVecPerThread = 4;

template <typename T, bool kAdd>
__global__ void rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ delta, const int* __restrict__ rows,
                                   const float* __restrict__ w, float eps, T* __restrict__ out, int H, int T_rows) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    if (src < 0 || src >= T_rows) src = 0;
    float* xr = x + (size_t)src * H;
    const int nvec = H >> 2;
    float4 v[kVecPerThread];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kVecPerThread; ++i) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < nvec) {
            v[i] = load4(xr + 4 * q);
            if (kAdd) {
                const float4 d = load4(delta + (size_t)src * H + 4 * q);
                v[i].x += d.x; v[i].y += d.y; v[i].z += d.z; v[i].w += d.w;
                store4(xr + 4 * q, v[i]);
            }
            ss += v[i].x * v[i].x;
            ss += v[i].y * v[i].y;
            ss += v[i].z * v[i].z;
            ss += v[i].w * v[i].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < kVecPerThread; ++i) {
        const int q = threadIdx.x + i * blockDim.x;
        if (q < nvec) {
            const float4 ww = load4(w + 4 * q);
            store4(o + 4 * q, make_float4((ww.x * v[i].x) * rinv, (ww.y * v[i].y) * rinv, (ww.z * v[i].z) * rinv, (ww.w * v[i].w) * rinv));
        }
    }
}

template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* __restrict__ delta, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) x[i] += to_float(delta[i]);
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I, long long n) {
    pdl_launch_dependents();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        const long long t = i / I;
        const int j = (int)(i - t * I);
        const float g = to_float(gate_up[t * 2 * I + j]);
        const float u = to_float(gate_up[t * 2 * I + I + j]);
        out[i] = from_float<T>(swiglu_of<T>(g, u));
    }
}

int grid_for(long long n, int threads) {
    long long b = ceil_div_ll(n, threads);
    if (b > 148LL * 16) b = 148LL * 16;
    return (int)(b < 1 ? 1 : b);
}

}  // namespace

LI_EXPORT int li_embedding(const void* table, int dtype, const int* ids, float* out, int T, int H, int V, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && H > 0 && V > 0, "embedding: bad sizes T=%d H=%d V=%d", T, H, V);
    if (T == 0) return 0;
    if (dtype == LI_F32)
        li_launch_pdl(embedding_kernel<float>, dim3(T), dim3(kRowThreads), 0, stream, (const float*)table, ids, out, H, V);
    else if (dtype == LI_BF16)
        li_launch_pdl(embedding_kernel<bf16>, dim3(T), dim3(kRowThreads), 0, stream, (const bf16*)table, ids, out, H, V);
    else
        return li_fail("embedding: unknown dtype %d", dtype);
    return li_check_launch("embedding");
}

template <bool kAdd>
static int launch_norm(float* x, const void* delta, int dtype, const int* rows, const float* w, float eps, void* out, int R, int T,
                       int H, cudaStream_t stream, const char* what) {
    LI_REQUIRE(R >= 0 && H > 0, "%s: bad sizes rows=%d H=%d", what, R, H);
    if (R == 0) return 0;
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "%s: unknown dtype %d", what, dtype);
    const bool aligned = ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)delta % 16 == 0);
    if (H % 4 == 0 && H / 4 <= 1024 * kVecPerThread && aligned) {
        int threads = ceil_div(H / 4, kVecPerThread);
        threads = ceil_div(threads, 32) * 32;
        if (threads < 64) threads = 64;
        if (dtype == LI_F32)
            li_launch_pdl(rmsnorm_vec_kernel<float, kAdd>, dim3(R), dim3(threads), 0, stream, x, (const float*)delta, rows, w, eps, (float*)out, H, T);
        else
            li_launch_pdl(rmsnorm_vec_kernel<bf16, kAdd>, dim3(R), dim3(threads), 0, stream, x, (const bf16*)delta, rows, w, eps, (bf16*)out, H, T);
        return li_check_launch(what);
    }
    if (dtype == LI_F32)
        li_launch_pdl(rmsnorm_kernel<float, kAdd>, dim3(R), dim3(kRowThreads), 0, stream, x, (const float*)delta, rows, w, eps, (float*)out, H, T);
    else
        li_launch_pdl(rmsnorm_kernel<bf16, kAdd>, dim3(R), dim3(kRowThreads), 0, stream, x, (const bf16*)delta, rows, w, eps, (bf16*)out, H, T);
    return li_check_launch(what);
}

LI_EXPORT int li_rmsnorm(const float* x, const float* w, float eps, void* out, int dtype, int T, int H, cudaStream_t stream) {
    return launch_norm<false>(const_cast<float*>(x), nullptr, dtype, nullptr, w, eps, out, T, T, H, stream, "rmsnorm");
}

LI_EXPORT int li_add_rmsnorm(float* x, const void* delta, int dtype, const float* w, float eps, void* out, int T, int H,
                             cudaStream_t stream) {
    return launch_norm<true>(x, delta, dtype, nullptr, w, eps, out, T, T, H, stream, "add_rmsnorm");
}

LI_EXPORT int li_gather_rmsnorm(const float* x, const int* rows, const float* w, float eps, void* out, int dtype, int R, int T, int H,
                                cudaStream_t stream) {
    return launch_norm<false>(const_cast<float*>(x), nullptr, dtype, rows, w, eps, out, R, T, H, stream, "gather_rmsnorm");
}

LI_EXPORT int li_residual_add(float* x, const void* delta, int dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype == LI_F32)
        residual_add_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>(x, (const float*)delta, n);
    else if (dtype == LI_BF16)
        residual_add_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>(x, (const bf16*)delta, n);
    else
        return li_fail("residual_add: unknown dtype %d", dtype);
    return li_check_launch("residual_add");
}

// The device's resident copy of the requests' block tables (a row per state slot) and the step's view of it.  `updates`
// (from the host runtime's packer): a count, then triples (slot, logical page, page id).  CTA s brings the row of
// sequence s up to date (the triples of its slot; two sequences of one request write the same values) and copies its
// first max_blocks entries into the step's table, the sink page beyond the row's width.  LitInfer builds and uploads a
// table per layer and step (src/llaisys/models/qwen2.cpp:993-1003); here a step uploads what changed.
namespace {
__global__ void table_gather_kernel(int* __restrict__ resident, int rows, int cols, const int* __restrict__ updates, int update_cap,
                                    const int* __restrict__ slots, int* __restrict__ out, int max_blocks, int trash_page) {
    const int s = blockIdx.x;
    int slot = slots[s];
    if (slot < 0 || slot >= rows) slot = rows - 1;                  // the last row is never written: all sink page
    int n = updates[0];
    if (n > update_cap) n = update_cap;
    int* row = resident + (size_t)slot * cols;
    if (slot != rows - 1)
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const int* u = updates + 1 + 3 * i;
            if (u[0] == slot && u[1] >= 0 && u[1] < cols) row[u[1]] = u[2];
        }
    __syncthreads();
    for (int b = threadIdx.x; b < max_blocks; b += blockDim.x) out[(size_t)s * max_blocks + b] = b < cols ? row[b] : trash_page;
}
}  // namespace

LI_EXPORT int li_table_gather(int* resident, int rows, int cols, const int* updates, int update_cap, const int* slots, int* out, int S,
                              int max_blocks, int trash_page, cudaStream_t stream) {
    LI_REQUIRE(rows >= 1 && cols >= 1 && S >= 0 && max_blocks >= 1 && update_cap >= 0, "table_gather: bad sizes rows=%d cols=%d S=%d max_blocks=%d cap=%d",
               rows, cols, S, max_blocks, update_cap);
    if (S == 0) return 0;
    table_gather_kernel<<<S, 128, 0, stream>>>(resident, rows, cols, updates, update_cap, slots, out, max_blocks, trash_page);
    return li_check_launch("table_gather");
}

// x *= factor (an embedding scale) and x = cap * tanh(x / cap) (a cap on the logits), in place on float32.
namespace {
__global__ void scale_kernel(float* __restrict__ x, long long n, float factor) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= factor;
}
__global__ void logit_cap_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}
}  // namespace

namespace {
// out[r, :] = src[rows[r], :] for float rows (the wanted logits out of a captured step's fixed layout)
__global__ void gather_rows_kernel(const float* __restrict__ src, const int* __restrict__ rows, float* __restrict__ out, int n_src, long long width) {
    pdl_launch_dependents();
    pdl_wait();
    int r = rows[blockIdx.y];
    r = r < 0 ? 0 : (r >= n_src ? n_src - 1 : r);          // validated on the host; never read outside the source
    const float* s = src + (size_t)r * width;
    float* o = out + (size_t)blockIdx.y * width;
    for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < width; j += (long long)gridDim.x * blockDim.x) o[j] = s[j];
}
}  // namespace

LI_EXPORT int li_gather_rows(const float* src, const int* rows, float* out, int n_src, int n_rows, long long width, cudaStream_t stream) {
    LI_REQUIRE(n_src >= 1 && n_rows >= 0 && n_rows <= 65535 && width >= 1, "gather_rows: bad sizes (%d source rows, %d rows, width %lld)", n_src, n_rows, width);
    if (n_rows == 0) return 0;
    const unsigned bx = (unsigned)((width + 1023) / 1024 < 64 ? (width + 1023) / 1024 : 64);
    li_launch_pdl(gather_rows_kernel, dim3(bx, n_rows), dim3(256), 0, stream, src, rows, out, n_src, width);
    return li_check_launch("gather_rows");
}

LI_EXPORT int li_scale_inplace(float* x, long long n, float factor, cudaStream_t stream) {
    LI_REQUIRE(n >= 0 && n <= (1LL << 40), "scale: bad size %lld", n);
    if (n == 0) return 0;
    li_launch_pdl(scale_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, factor);
    return li_check_launch("scale");
}

LI_EXPORT int li_logit_cap(float* x, long long n, float cap, cudaStream_t stream) {
    LI_REQUIRE(n >= 0 && n <= (1LL << 40), "logit_cap: bad size %lld", n);
    LI_REQUIRE(cap > 0.0f, "logit_cap: the cap must be positive, got %g", (double)cap);
    if (n == 0) return 0;
    li_launch_pdl(logit_cap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, cap);
    return li_check_launch("logit_cap");
}

LI_EXPORT int li_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && I > 0, "swiglu: bad sizes T=%d I=%d", T, I);
    const long long n = (long long)T * I;
    if (n == 0) return 0;
    if (dtype == LI_F32)
        swiglu_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)gate_up, (float*)out, I, n);
    else if (dtype == LI_BF16)
        swiglu_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I, n);
    else
        return li_fail("swiglu: unknown dtype %d", dtype);
    return li_check_launch("swiglu");
}

// out[tok, :] = hprime[tok, :] / sqrt(sum of ssq[:, tok] / width + eps): the normalised activation itself, for a
// consumer that cannot take the factor into its own product (row_scale.cuh).  bfloat16.
namespace {
__global__ void apply_row_scale_kernel(const bf16* __restrict__ hprime, const float* __restrict__ ssq, int nparts, float width, float eps,
                                       bf16* __restrict__ out, int M, int H) {
    __shared__ float factor;
    pdl_launch_dependents();
    pdl_wait();
    const int tok = blockIdx.x;
    if (threadIdx.x < 32) {
        float s = 0.0f;
        for (int p = threadIdx.x; p < nparts; p += 32) s += ssq[(size_t)tok * nparts + p];
        s = warp_sum(s);
        if (threadIdx.x == 0) factor = 1.0f / sqrtf(s / width + eps);
    }
    __syncthreads();
    const float f = factor;
    for (int j = threadIdx.x; j < H; j += blockDim.x) out[(size_t)tok * H + j] = __float2bfloat16_rn(__bfloat162float(hprime[(size_t)tok * H + j]) * f);
}
}  // namespace

LI_EXPORT int li_apply_row_scale(const void* hprime, const float* ssq, int nparts, int width, float eps, void* out, int M, int H,
                                 cudaStream_t stream) {
    LI_REQUIRE(M >= 0 && H > 0 && nparts >= 1 && width >= 1, "apply_row_scale: bad sizes M=%d H=%d parts=%d width=%d", M, H, nparts, width);
    if (M == 0) return 0;
    li_launch_pdl(apply_row_scale_kernel, dim3(M), dim3(256), 0, stream, (const bf16*)hprime, ssq, nparts, (float)width, eps, (bf16*)out, M, H);
    return li_check_launch("apply_row_scale");
}
