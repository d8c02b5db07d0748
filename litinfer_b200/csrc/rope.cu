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

namespace {

// One block per (token, head): query heads first, then key/value heads.  A thread owns the
// pair (j, j + half) of its head, so sine and cosine are computed once per pair and nothing is
// shared; blocks are small and many, which keeps the latency of a decode step's launch short.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const float* __restrict__ denom,
                                     int rotary_dim, const int* __restrict__ slot_mapping, T* __restrict__ kcache,
                                     T* __restrict__ vcache, int nh, int nkv, int dh, int page_size, int num_pages, int write) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, head = blockIdx.y;
    const int half = rotary_dim >> 1;
    const float pos = (float)positions[t];
    T* row = qkv + (size_t)t * (nh + 2 * nkv) * dh;
    if (head < nh) {
        T* x = row + (size_t)head * dh;
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            float s, c;
            sincosf(pos / denom[j], &s, &c);
            const float a = to_float(x[j]), b = to_float(x[j + half]);
            x[j] = from_float<T>(a * c - b * s);
            x[j + half] = from_float<T>(b * c + a * s);
        }
        return;
    }
    if (!write) return;
    const int h = head - nh;
    const int slot = slot_mapping[t];
    const int page = slot / page_size, off = slot - page * page_size;
    if (slot < 0 || page >= num_pages) return;       // validated on the host; never write outside the cache
    const T* k = row + (size_t)(nh + h) * dh;
    const T* v = row + (size_t)(nh + nkv + h) * dh;
    T* kdst = kcache + (((size_t)page * nkv + h) * page_size + off) * dh;
    T* vdst = vcache + ((size_t)page * nkv + h) * dh * page_size + off;      // values are cached transposed
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float s, c;
        sincosf(pos / denom[j], &s, &c);
        const float a = to_float(k[j]), b = to_float(k[j + half]);
        kdst[j] = from_float<T>(a * c - b * s);
        kdst[j + half] = from_float<T>(b * c + a * s);
    }
    for (int d = rotary_dim + threadIdx.x; d < dh; d += blockDim.x) kdst[d] = k[d];
    for (int d = threadIdx.x; d < dh; d += blockDim.x) vdst[(size_t)d * page_size] = v[d];
}

}  // namespace

LI_EXPORT int li_rope_kv_write(void* qkv, int dtype, const int* positions, const float* denom, int rotary_dim,
                               const int* slot_mapping, void* kcache, void* vcache, int T, int nh, int nkv, int dh, int page_size,
                               int num_pages, int write, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && dh > 0 && page_size > 0, "rope_kv_write: bad sizes");
    LI_REQUIRE(rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= dh, "rope_kv_write: rotary_dim %d must be even and at most head_dim %d",
               rotary_dim, dh);
    if (T == 0) return 0;
    LI_REQUIRE(T <= 2147483647 && nh + nkv <= 65535, "rope_kv_write: too many heads for one launch");
    const int threads = dh >= 128 ? 64 : 32;
    const dim3 grid(T, nh + nkv);
    const size_t smem = 0;
    if (dtype == LI_F32)
        li_launch_pdl(rope_kv_write_kernel<float>, dim3(grid), dim3(threads), smem, stream, (float*)qkv, positions, denom, rotary_dim, slot_mapping, (float*)kcache,
                                                                   (float*)vcache, nh, nkv, dh, page_size, num_pages, write);
    else if (dtype == LI_BF16)
        li_launch_pdl(rope_kv_write_kernel<bf16>, dim3(grid), dim3(threads), smem, stream, (bf16*)qkv, positions, denom, rotary_dim, slot_mapping, (bf16*)kcache,
                                                                  (bf16*)vcache, nh, nkv, dh, page_size, num_pages, write);
    else
        return li_fail("rope_kv_write: unknown dtype %d", dtype);
    return li_check_launch("rope_kv_write");
}

// The q|k|v projection followed by rope_kv_write.  For a few bfloat16 tokens (decode) both run as one
// kernel: the weight-streaming product applies the rotation and writes the cache in its epilogue.
// Otherwise: the product, then the kernel above.
int li_linear_gemv_rope(const void* a, const void* w, const float* bias, void* out, int M, int N, int K, const int* positions,
                        const float* denom, const int* slot_mapping, void* kcache, void* vcache, int nh, int nkv, int dh,
                        int page_size, int num_pages, int write, cudaStream_t stream);
bool li_gemv_rope_accepts(const void* a, const void* w, int M, int N, int K, int nh, int nkv, int dh, int rotary_dim);
extern "C" int li_linear(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N, int K,
                         int epilogue, cudaStream_t stream);

LI_EXPORT int li_linear_rope_kv(const void* a, const void* w, const float* bias, void* qkv, int dtype, const int* positions,
                                const float* denom, int rotary_dim, const int* slot_mapping, void* kcache, void* vcache, int T,
                                int K, int nh, int nkv, int dh, int page_size, int num_pages, int write, int allow_fused,
                                cudaStream_t stream) {
    const int N = (nh + 2 * nkv) * dh;
    if (T == 0) return 0;
    if (allow_fused && dtype == LI_BF16 && li_gemv_rope_accepts(a, w, T, N, K, nh, nkv, dh, rotary_dim))
        return li_linear_gemv_rope(a, w, bias, qkv, T, N, K, positions, denom, slot_mapping, kcache, vcache, nh, nkv, dh, page_size,
                                   num_pages, write, stream);
    if (int rc = li_linear(a, w, bias, qkv, dtype, dtype, T, N, K, LI_EPILOGUE_NONE, stream)) return rc;
    return li_rope_kv_write(qkv, dtype, positions, denom, rotary_dim, slot_mapping, kcache, vcache, T, nh, nkv, dh, page_size, num_pages,
                            write, stream);
}
