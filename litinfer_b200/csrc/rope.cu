// Rotary position encoding of q and k, fused with the write of k and v into
// the paged cache.
//
// Rotate-half pairing on the first rotary_dim elements of each head
// (LitInfer: src/ops/rope/op.cpp:13-20, 33-39): phi = float(pos) / denom[j],
// (a, b) = (x[j], x[j + rotary_dim/2]), x'[j] = a cos - b sin,
// x'[j + rotary_dim/2] = b cos + a sin, in float with sincosf.  q is rotated in
// place inside the fused qkv row; k is rotated and stored, v stored as is, at
// the token's slot (page = slot / page_size, offset = slot % page_size):
// keys as kcache[page][kv_head][offset][:], values transposed as
// vcache[page][kv_head][:][offset], which is how the tensor-core attention
// kernels want to read them (LitInfer caches k after rotation as well,
// src/llaisys/models/qwen2.cpp:626-673).
#include "common.cuh"
#include "rope_epilogue.cuh"
#include "row_scale.cuh"

namespace {

// A block takes one token and ``heads_per_block`` of its heads (query heads first, then key heads); a thread
// owns pairs (j, j + half), so nothing is shared.  Few tokens (decode): one head a block, small and many
// blocks, short latency.  Many tokens (prefill): all heads of a token in one block, fewer and fuller blocks.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const float* __restrict__ denom,
                                     int rotary_dim, const int* __restrict__ slot_mapping, T* __restrict__ kcache,
                                     T* __restrict__ vcache, int nh, int nkv, int dh, int page_size, int num_pages, int write,
                                     int write_v, int heads_per_block) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int half = rotary_dim >> 1;
    const float pos = (float)positions[t];
    T* row = qkv + (size_t)t * (nh + 2 * nkv) * dh;
    const int head_lo = blockIdx.y * heads_per_block;
    const int head_hi = min(nh + nkv, head_lo + heads_per_block);
    int page = 0, off = 0;
    bool slot_ok = false;
    if (write && head_hi > nh) {
        const int slot = slot_mapping[t];
        page = slot / page_size;
        off = slot - page * page_size;
        slot_ok = slot >= 0 && page < num_pages;       // validated on the host; never write outside the cache
    }
    // rotation pairs of the block's heads, spread over its threads
    const int nheads = head_hi - head_lo;
    for (int i = threadIdx.x; i < nheads * half; i += blockDim.x) {
        const int hl = i / half, j = i - hl * half;
        const int head = head_lo + hl;
        float s, c;
        sincosf(pos / denom[j], &s, &c);
        if (head < nh) {
            T* x = row + (size_t)head * dh;
            const float a = to_float(x[j]), b = to_float(x[j + half]);
            x[j] = from_float<T>(a * c - b * s);
            x[j + half] = from_float<T>(b * c + a * s);
        } else if (slot_ok) {
            const int h = head - nh;
            const T* k = row + (size_t)head * dh;
            T* kdst = kcache + (((size_t)page * nkv + h) * page_size + off) * dh;
            const float a = to_float(k[j]), b = to_float(k[j + half]);
            kdst[j] = from_float<T>(a * c - b * s);
            kdst[j + half] = from_float<T>(b * c + a * s);
        }
    }
    if (!slot_ok) return;
    for (int head = max(head_lo, nh); head < head_hi; ++head) {
        const int h = head - nh;
        const T* k = row + (size_t)head * dh;
        const T* v = row + (size_t)(nh + nkv + h) * dh;
        T* kdst = kcache + (((size_t)page * nkv + h) * page_size + off) * dh;
        T* vdst = vcache + ((size_t)page * nkv + h) * dh * page_size + off;      // values are cached transposed
        for (int d = rotary_dim + threadIdx.x; d < dh; d += blockDim.x) kdst[d] = k[d];
        if (write_v)
            for (int d = threadIdx.x; d < dh; d += blockDim.x) vdst[(size_t)d * page_size] = v[d];
    }
}

// The values of many tokens (prefill) into the transposed cache, 16 tokens and one key/value head per block:
// the tile goes through shared memory, so that each output column's 16 slots are written as one 32-byte
// piece when the 16 tokens sit in consecutive slots of one page (the usual case), instead of 16 scattered
// two-byte writes.  Tokens whose slots are not such a run are written one by one.
template <typename T>
__global__ void v_cache_write_kernel(const T* __restrict__ qkv, const int* __restrict__ slot_mapping, T* __restrict__ vcache,
                                     int total, int nh, int nkv, int dh, int page_size, int num_pages) {
    extern __shared__ __align__(16) unsigned char vt_raw[];
    T* vt = reinterpret_cast<T*>(vt_raw);              // [dh][16 + 2]: padded against bank conflicts
    __shared__ int slots[16];
    constexpr int LD = 18;
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * 16, h = blockIdx.y;
    const int n = min(16, total - t0);
    const int row = (nh + 2 * nkv) * dh;
    if (threadIdx.x < 16) slots[threadIdx.x] = threadIdx.x < n ? slot_mapping[t0 + threadIdx.x] : -1;
    for (int i = threadIdx.x; i < n * dh; i += blockDim.x) {
        const int tk = i / dh, d = i - tk * dh;
        vt[d * LD + tk] = qkv[(size_t)(t0 + tk) * row + (size_t)(nh + nkv + h) * dh + d];
    }
    __syncthreads();
    const int s0 = slots[0];
    bool run = n == 16 && s0 >= 0 && (s0 % 16) == 0 && (s0 / page_size) < num_pages && (s0 % page_size) + 16 <= page_size;
    if (run)
        for (int i = 1; i < 16; ++i) run = run && slots[i] == s0 + i;
    if (run) {
        const int page = s0 / page_size, off = s0 - page * page_size;
        T* dst = vcache + ((size_t)page * nkv + h) * dh * page_size + off;
        for (int d = threadIdx.x; d < dh; d += blockDim.x) {
            T* o = dst + (size_t)d * page_size;
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = vt[d * LD + i];
        }
    } else {
        for (int i = threadIdx.x; i < n * dh; i += blockDim.x) {
            const int tk = i / dh, d = i - tk * dh;
            const int slot = slots[tk];
            const int page = slot / page_size, off = slot - page * page_size;
            if (slot < 0 || page >= num_pages) continue;
            vcache[(((size_t)page * nkv + h) * dh + d) * page_size + off] = vt[d * LD + tk];
        }
    }
}

// cos and sin of every (token, pair) of a step, for kernels that rotate as an epilogue: out[t][j] = (cos, sin)(pos_t / denom_j)
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ denom, int half, float2* __restrict__ out, int total) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int t = i / half, j = i - t * half;
    float sn, cs;
    sincosf((float)positions[t] / denom[j], &sn, &cs);
    out[i] = make_float2(cs, sn);
}

}  // namespace

LI_EXPORT int li_rope_table(const int* positions, const float* denom, int half, float* out, int T, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && half > 0, "rope_table: bad sizes T=%d half=%d", T, half);
    if (T == 0) return 0;
    const long long total = (long long)T * half;
    LI_REQUIRE(total <= 2147483647LL, "rope_table: too many entries");
    li_launch_pdl(rope_table_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, positions, denom, half,
                  reinterpret_cast<float2*>(out), (int)total);
    return li_check_launch("rope_table");
}

LI_EXPORT int li_rope_kv_write(void* qkv, int dtype, const int* positions, const float* denom, int rotary_dim,
                               const int* slot_mapping, void* kcache, void* vcache, int T, int nh, int nkv, int dh, int page_size,
                               int num_pages, int write, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && dh > 0 && page_size > 0, "rope_kv_write: bad sizes");
    // rotary_dim 0: nothing is rotated (a model without rotary positions); keys and values are stored as they are
    LI_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= dh, "rope_kv_write: rotary_dim %d must be even and at most head_dim %d",
               rotary_dim, dh);
    LI_REQUIRE(rotary_dim == 0 || denom != nullptr, "rope_kv_write: rotary_dim %d without denominators", rotary_dim);
    if (T == 0) return 0;
    LI_REQUIRE(T <= 2147483647 && nh + nkv <= 65535, "rope_kv_write: too many heads for one launch");
    const int heads_per_block = T >= 64 ? nh + nkv : 1;
    const int threads = T >= 64 ? 256 : (dh >= 128 ? 64 : 32);
    const dim3 grid(T, ceil_div(nh + nkv, heads_per_block));
    const size_t smem = 0;
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "rope_kv_write: unknown dtype %d", dtype);
    // many tokens: the values go through a kernel of their own that writes the transposed cache in 32-byte pieces
    const bool v_separate = write && T >= 64;
    const int write_v = v_separate ? 0 : 1;
    if (dtype == LI_F32)
        li_launch_pdl(rope_kv_write_kernel<float>, dim3(grid), dim3(threads), smem, stream, (float*)qkv, positions, denom, rotary_dim,
                      slot_mapping, (float*)kcache, (float*)vcache, nh, nkv, dh, page_size, num_pages, write, write_v, heads_per_block);
    else
        li_launch_pdl(rope_kv_write_kernel<bf16>, dim3(grid), dim3(threads), smem, stream, (bf16*)qkv, positions, denom, rotary_dim,
                      slot_mapping, (bf16*)kcache, (bf16*)vcache, nh, nkv, dh, page_size, num_pages, write, write_v, heads_per_block);
    if (int rc = li_check_launch("rope_kv_write")) return rc;
    if (v_separate) {
        const dim3 vgrid(ceil_div(T, 16), nkv);
        const size_t vsmem = (size_t)dh * 18 * (dtype == LI_F32 ? 4 : 2);
        LI_REQUIRE(vsmem <= 48 * 1024, "rope_kv_write: head_dim %d is too large", dh);
        if (dtype == LI_F32)
            li_launch_pdl(v_cache_write_kernel<float>, vgrid, dim3(128), vsmem, stream, (const float*)qkv, slot_mapping, (float*)vcache, T, nh,
                          nkv, dh, page_size, num_pages);
        else
            li_launch_pdl(v_cache_write_kernel<bf16>, vgrid, dim3(128), vsmem, stream, (const bf16*)qkv, slot_mapping, (bf16*)vcache, T, nh,
                          nkv, dh, page_size, num_pages);
        return li_check_launch("rope_kv_write (values)");
    }
    return 0;
}

// The q|k|v projection followed by rope_kv_write.  For a few bfloat16 tokens (decode) both run as one
// kernel: the weight-streaming product applies the rotation and writes the cache in its epilogue.
// Otherwise: the product, then the kernel above.
int li_linear_gemv_rope(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, const int* positions,
                        const float* denom, const int* slot_mapping, void* kcache, void* vcache, int nh, int nkv, int dh,
                        int page_size, int num_pages, int write, const RowScale& rs, cudaStream_t stream);
bool li_gemv_rope_accepts(const void* a, const void* w, int M, int N, int K, int nh, int nkv, int dh, int rotary_dim);
bool li_tcgen05_rope_wanted(const void* a, const void* w, const void* out, int M, int N, int K);
int li_linear_tcgen05_rope(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, const RopeEpilogue& rope,
                           cudaStream_t stream);
extern "C" int li_linear(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N, int K,
                         int epilogue, cudaStream_t stream);
extern "C" int li_linear_scaled(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N,
                                int K, int epilogue, const float* ssq, int nparts, int width, float eps, cudaStream_t stream);

LI_EXPORT int li_linear_rope_kv(const void* a, const void* w, const float* bias, void* qkv, int dtype, const int* positions,
                                const float* denom, int rotary_dim, const int* slot_mapping, void* kcache, void* vcache, int T,
                                int K, int nh, int nkv, int dh, int page_size, int num_pages, int write, int allow_fused,
                                const float* ssq, int nparts, int width, float eps, const float* cos_sin, cudaStream_t stream) {
    // ssq (or nullptr): partial sums of squares for a factor per token on the product, as in li_linear_scaled
    // cos_sin (or nullptr): the step's table from li_rope_table; with it a long bfloat16 step rotates and writes the cache
    // in the epilogue of the tensor-memory product (head_dim 128)
    const int N = (nh + 2 * nkv) * dh;
    if (T == 0) return 0;
    if (allow_fused && cos_sin && !ssq && dtype == LI_BF16 && T > 64 && dh == 128 && rotary_dim == 128 && page_size % 16 == 0 &&
        li_tcgen05_rope_wanted(a, w, qkv, T, N, K)) {
        RopeEpilogue re;
        re.cos_sin = cos_sin;
        re.slot_mapping = slot_mapping;
        re.kcache = (bf16*)kcache;
        re.vcache = (bf16*)vcache;
        re.nh = nh;
        re.nkv = nkv;
        re.page_size = page_size;
        re.num_pages = num_pages;
        re.write = write;
        return li_linear_tcgen05_rope(a, w, bias, qkv, T, N, K, re, stream);
    }
    RowScale rs;
    if (ssq) {
        LI_REQUIRE(nparts >= 1 && width >= 1, "linear_rope_kv: bad partial sums (%d parts, width %d)", nparts, width);
        rs.ssq = ssq;
        rs.nparts = nparts;
        rs.width = (float)width;
        rs.eps = eps;
    }
    if (allow_fused && dtype == LI_BF16 && li_gemv_rope_accepts(a, w, T, N, K, nh, nkv, dh, rotary_dim))
        return li_linear_gemv_rope(a, w, bias, qkv, T, N, K, positions, denom, slot_mapping, kcache, vcache, nh, nkv, dh, page_size,
                                   num_pages, write, rs, stream);
    if (ssq) {
        if (int rc = li_linear_scaled(a, w, bias, qkv, dtype, dtype, T, N, K, LI_EPILOGUE_NONE, ssq, nparts, width, eps, stream)) return rc;
    } else if (int rc = li_linear(a, w, bias, qkv, dtype, dtype, T, N, K, LI_EPILOGUE_NONE, stream)) return rc;
    return li_rope_kv_write(qkv, dtype, positions, denom, rotary_dim, slot_mapping, kcache, vcache, T, nh, nkv, dh, page_size, num_pages,
                            write, stream);
}
