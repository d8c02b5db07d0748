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

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const float* __restrict__ denom,
                                     int rotary_dim, const int* __restrict__ slot_mapping, T* __restrict__ kcache,
                                     T* __restrict__ vcache, int nh, int nkv, int dh, int page_size, int num_pages, int write) {
    extern __shared__ float cs[];                    // cos[half] | sin[half]
    const int t = blockIdx.x;
    const int half = rotary_dim >> 1;
    const float pos = (float)positions[t];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float s, c;
        sincosf(pos / denom[j], &s, &c);
        cs[j] = c;
        cs[half + j] = s;
    }
    __syncthreads();
    const int row = (nh + 2 * nkv) * dh;
    T* q = qkv + (size_t)t * row;
    for (int i = threadIdx.x; i < nh * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        T* x = q + h * dh;
        const float a = to_float(x[j]), b = to_float(x[j + half]);
        x[j] = from_float<T>(a * cs[j] - b * cs[half + j]);
        x[j + half] = from_float<T>(b * cs[j] + a * cs[half + j]);
    }
    if (!write) return;
    const int slot = slot_mapping[t];
    const int page = slot / page_size, off = slot - page * page_size;
    if (slot < 0 || page >= num_pages) return;       // validated on the host; never write outside the cache
    const T* k = q + nh * dh;
    const T* v = k + nkv * dh;
    for (int i = threadIdx.x; i < nkv * dh; i += blockDim.x) {
        const int h = i / dh, d = i - h * dh;
        const size_t dst = (((size_t)page * nkv + h) * page_size + off) * dh + d;
        float kv = to_float(k[i]);
        if (d < rotary_dim) {
            if (d < half) {
                const float b = to_float(k[i + half]);
                kv = kv * cs[d] - b * cs[half + d];
            } else {
                const int j = d - half;
                const float a = to_float(k[i - half]);
                kv = kv * cs[j] + a * cs[half + j];
            }
        }
        kcache[dst] = from_float<T>(kv);
        vcache[((((size_t)page * nkv + h) * dh + d) * page_size) + off] = v[i];      // values are cached transposed
    }
}

}  // namespace

LI_EXPORT int li_rope_kv_write(void* qkv, int dtype, const int* positions, const float* denom, int rotary_dim,
                               const int* slot_mapping, void* kcache, void* vcache, int T, int nh, int nkv, int dh, int page_size,
                               int num_pages, int write, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && dh > 0 && page_size > 0, "rope_kv_write: bad sizes");
    LI_REQUIRE(rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= dh, "rope_kv_write: rotary_dim %d must be even and at most head_dim %d",
               rotary_dim, dh);
    if (T == 0) return 0;
    const size_t smem = (size_t)rotary_dim * sizeof(float);
    LI_REQUIRE(smem <= 48 * 1024, "rope_kv_write: rotary_dim %d is too large", rotary_dim);
    const int threads = 128;
    if (dtype == LI_F32)
        rope_kv_write_kernel<float><<<T, threads, smem, stream>>>((float*)qkv, positions, denom, rotary_dim, slot_mapping, (float*)kcache,
                                                                   (float*)vcache, nh, nkv, dh, page_size, num_pages, write);
    else if (dtype == LI_BF16)
        rope_kv_write_kernel<bf16><<<T, threads, smem, stream>>>((bf16*)qkv, positions, denom, rotary_dim, slot_mapping, (bf16*)kcache,
                                                                  (bf16*)vcache, nh, nkv, dh, page_size, num_pages, write);
    else
        return li_fail("rope_kv_write: unknown dtype %d", dtype);
    return li_check_launch("rope_kv_write");
}
