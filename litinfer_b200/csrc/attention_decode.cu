// Decode attention in bfloat16: one new token per sequence over its paged
// cache, grouped-query, split along the context.
//
// Grid (split, kv head, sequence).  A CTA of 4 warps covers 256 keys at fixed
// absolute positions [256 s, 256 s + 256), each warp 64 of them, for all query
// heads of one key/value head at once (they share every K and V byte read;
// heads are the 16 rows of a tensor-core tile).  Per 16 keys a warp computes
// S = Q K^T and O += P V with mma.sync m16n8k16 (bfloat16 in, float
// accumulate), softmax online in float as in LitInfer's kernel
// (src/ops/paged_attention/op.cpp:194-234).  All operands go from global
// memory straight into fragment registers with 8-byte loads:
//   * the sum over head_dim does not depend on its order, so the 4 consecutive
//     elements a thread loads from a q row and from a key row are used as the
//     element pairs the fragment layout asks for, the same way on both sides;
//   * values are cached transposed, [page][kv_head][head_dim][slot], so that for
//     one output column the 4 consecutive keys a thread needs are contiguous;
//     the score tiles are computed with their key columns permuted to match
//     (tile 0: keys 0,1,4,5,8,9,12,13 of the 16; tile 1: the others).
// Warps are merged through shared memory, CTAs through a float workspace and a
// small second kernel, both in fixed order: split boundaries depend on
// absolute key positions only, so a sequence's result does not depend on the
// batch it is in.  Window: keys below p - window + 1 are masked, splits wholly
// below it are skipped.
//
// Requires head_dim in {16, 32, ..., 128, 256}, at most 16 query heads per
// key/value head, page_size a multiple of 16.
#include "common.cuh"

namespace {

constexpr int kSplit = 256;
constexpr int kWarps = 4;

struct Workspace {
    float* buf = nullptr;
    size_t floats = 0;
};
Workspace g_ws[16];

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 ld8(const bf16* p) { return *reinterpret_cast<const uint2*>(p); }

__device__ __forceinline__ uint2 ld8_stream(const bf16* p) {
    uint2 v;
    asm volatile("ld.global.cs.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}

__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

__host__ __device__ inline void split_range(int ctx, int window, int* first, int* last) {
    const int p = ctx - 1;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    *first = lo / kSplit;
    *last = (ctx - 1) / kSplit;
}

template <int DH>
__global__ void __launch_bounds__(kWarps * 32)
decode_attention_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ ctx_lens,
                        float* __restrict__ part, int nh, int nkv, int page_size, int num_pages, float scale, int window,
                        int nsplit) {
    extern __shared__ float sm[];
    const int split = blockIdx.x, kvh = blockIdx.y, s = blockIdx.z;
    const int ctx = ctx_lens[s];
    const int p = ctx - 1;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int k_begin = split * kSplit;
    const int k_end = min(ctx, k_begin + kSplit);
    if (k_begin >= ctx || k_end <= lo) return;
    const int G = nh / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    constexpr int KS = DH / 16;          // k-steps of the score product
    constexpr int NT = DH / 8;           // column tiles of the output

    // query fragments: rows g and g + 8 are heads kvh * G + g (+ 8)
    const bf16* qrow = qkv + (size_t)s * (nh + 2 * nkv) * DH + (size_t)kvh * G * DH;
    unsigned qa[KS][4];
#pragma unroll
    for (int st = 0; st < KS; ++st) {
        const uint2 r0 = (g < G) ? ld8(qrow + (size_t)g * DH + st * 16 + t * 4) : make_uint2(0, 0);
        const uint2 r1 = (g + 8 < G) ? ld8(qrow + (size_t)(g + 8) * DH + st * 16 + t * 4) : make_uint2(0, 0);
        qa[st][0] = r0.x; qa[st][1] = r1.x; qa[st][2] = r0.y; qa[st][3] = r1.y;
    }
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

    const int* bt = block_table + (size_t)s * max_blocks;
    const int key_c0 = 4 * (g >> 1) + (g & 1);               // key column of this thread's K row in score tile 0; tile 1: + 2
#pragma unroll 1
    for (int b = 0; b < kSplit / 16 / kWarps; ++b) {
        const int key0 = k_begin + (warp * (kSplit / 16 / kWarps) + b) * 16;
        if (key0 >= k_end || key0 + 16 <= lo) continue;       // warp-uniform
        int page = bt[key0 / page_size];
        if (page < 0 || page >= num_pages) page = 0;
        const int off = key0 % page_size;
        const bf16* kbase = kcache + (((size_t)page * nkv + kvh) * page_size + off) * DH;
        const bf16* vbase = vcache + ((size_t)page * nkv + kvh) * DH * page_size + off;
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        const bf16* k0 = kbase + (size_t)key_c0 * DH + t * 4;
        const bf16* k1 = k0 + 2 * DH;
#pragma unroll
        for (int st = 0; st < KS; ++st) {
            const uint2 b0 = ld8_stream(k0 + st * 16);
            const uint2 b1 = ld8_stream(k1 + st * 16);
            mma_bf16(s0, qa[st][0], qa[st][1], qa[st][2], qa[st][3], b0.x, b0.y);
            mma_bf16(s1, qa[st][0], qa[st][1], qa[st][2], qa[st][3], b1.x, b1.y);
        }
        // this thread's keys: key0 + 4 t + {0, 1} (tile 0) and + {2, 3} (tile 1); rows g (c0, c1) and g + 8 (c2, c3)
        const int kk = key0 + 4 * t;
        const bool ok0 = kk >= lo && kk < k_end, ok1 = kk + 1 >= lo && kk + 1 < k_end;
        const bool ok2 = kk + 2 >= lo && kk + 2 < k_end, ok3 = kk + 3 >= lo && kk + 3 < k_end;
        s0[0] = ok0 ? s0[0] * scale : -INFINITY; s0[1] = ok1 ? s0[1] * scale : -INFINITY;
        s0[2] = ok0 ? s0[2] * scale : -INFINITY; s0[3] = ok1 ? s0[3] * scale : -INFINITY;
        s1[0] = ok2 ? s1[0] * scale : -INFINITY; s1[1] = ok3 ? s1[1] * scale : -INFINITY;
        s1[2] = ok2 ? s1[2] * scale : -INFINITY; s1[3] = ok3 ? s1[3] * scale : -INFINITY;
        const float mx0 = quad_max(fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1])));
        const float mx1 = quad_max(fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3])));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);      // finite: at least one key of the 16 is visible
        const float a0 = expf(m0 - mn0), a1 = expf(m1 - mn1);
        const float p00 = expf(s0[0] - mn0), p01 = expf(s0[1] - mn0), p02 = expf(s1[0] - mn0), p03 = expf(s1[1] - mn0);
        const float p10 = expf(s0[2] - mn1), p11 = expf(s0[3] - mn1), p12 = expf(s1[2] - mn1), p13 = expf(s1[3] - mn1);
        l0 = l0 * a0 + (p00 + p01 + p02 + p03);
        l1 = l1 * a1 + (p10 + p11 + p12 + p13);
        m0 = mn0; m1 = mn1;
        const unsigned pa0 = pack_bf16(p00, p01), pa1 = pack_bf16(p10, p11), pa2 = pack_bf16(p02, p03), pa3 = pack_bf16(p12, p13);
        const bf16* vcol = vbase + (size_t)g * page_size + 4 * t;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint2 vb = ld8_stream(vcol + (size_t)j * 8 * page_size);
            o[j][0] *= a0; o[j][1] *= a0; o[j][2] *= a1; o[j][3] *= a1;
            mma_bf16(o[j], pa0, pa1, pa2, pa3, vb.x, vb.y);
        }
    }
    l0 = quad_sum(l0);
    l1 = quad_sum(l1);

    // merge the warps in fixed order: sm_m[w][16] | sm_l[w][16] | sm_o[w][G][DH]
    float* sm_m = sm;
    float* sm_l = sm + kWarps * 16;
    float* sm_o = sm + 2 * kWarps * 16;
    if (t == 0) {
        sm_m[warp * 16 + g] = m0; sm_m[warp * 16 + g + 8] = m1;
        sm_l[warp * 16 + g] = l0; sm_l[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int col = j * 8 + 2 * t;
        if (g < G) {
            sm_o[((size_t)warp * G + g) * DH + col] = o[j][0];
            sm_o[((size_t)warp * G + g) * DH + col + 1] = o[j][1];
        }
        if (g + 8 < G) {
            sm_o[((size_t)warp * G + g + 8) * DH + col] = o[j][2];
            sm_o[((size_t)warp * G + g + 8) * DH + col + 1] = o[j][3];
        }
    }
    __syncthreads();
    // partial layout per (sequence, head, split): DH floats of O, then m, l
    for (int e = threadIdx.x; e < G * DH; e += kWarps * 32) {
        const int r = e / DH, d = e - r * DH;
        float M = sm_m[r];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
        float O = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float f = expf(sm_m[w * 16 + r] - M);
            O += sm_o[((size_t)w * G + r) * DH + d] * f;
            L += sm_l[w * 16 + r] * f;
        }
        float* dst = part + (((size_t)s * nh + kvh * G + r) * nsplit + split) * (DH + 2);
        dst[d] = O;
        if (d == 0) {
            dst[DH] = M;
            dst[DH + 1] = L;
        }
    }
}

template <int DH>
__global__ void decode_combine_kernel(const float* __restrict__ part, const int* __restrict__ ctx_lens, bf16* __restrict__ out, int nh,
                                      int window, int nsplit) {
    const int s = blockIdx.x / nh, h = blockIdx.x - s * nh;
    int first, last;
    split_range(ctx_lens[s], window, &first, &last);
    const float* base = part + ((size_t)s * nh + h) * nsplit * (DH + 2);
    float M = -INFINITY;
    for (int sp = first; sp <= last; ++sp) M = fmaxf(M, base[(size_t)sp * (DH + 2) + DH]);
    for (int d = threadIdx.x; d < DH; d += blockDim.x) {
        float O = 0.0f, L = 0.0f;
        for (int sp = first; sp <= last; ++sp) {
            const float* q = base + (size_t)sp * (DH + 2);
            const float f = expf(q[DH] - M);
            O += q[d] * f;
            L += q[DH + 1] * f;
        }
        out[((size_t)s * nh + h) * DH + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
    }
}

int ensure_workspace(size_t floats, float** buf) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return li_fail("attention (decode): cudaGetDevice: %s", cudaGetErrorString(e));
    LI_REQUIRE(dev >= 0 && dev < 16, "attention (decode): device index %d out of range", dev);
    Workspace& w = g_ws[dev];
    if (w.floats < floats) {
        // grows on demand; the first call of a given size must come before stream capture
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        size_t want = floats < (8u << 20) ? (8u << 20) : floats + floats / 2;
        float* nb = nullptr;
        e = cudaMalloc(&nb, want * sizeof(float));
        if (e != cudaSuccess) {
            (void)st;
            return li_fail("attention (decode): cannot allocate %zu bytes of workspace: %s (a first call of this size inside a stream capture cannot allocate)",
                           want * sizeof(float), cudaGetErrorString(e));
        }
        if (w.buf) cudaFree(w.buf);
        w.buf = nb;
        w.floats = want;
    }
    *buf = w.buf;
    return 0;
}

template <int DH>
int launch(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
           const int* ctx_lens, int S, int nh, int nkv, int page_size, int num_pages, float scale, int window, int max_ctx_len,
           cudaStream_t stream) {
    const int nsplit = ceil_div(max_ctx_len > 0 ? max_ctx_len : 1, kSplit);
    const int G = nh / nkv;
    float* part = nullptr;
    if (int rc = ensure_workspace((size_t)S * nh * nsplit * (DH + 2), &part)) return rc;
    const size_t smem = (2 * kWarps * 16 + (size_t)kWarps * G * DH) * sizeof(float);
    static bool attr_set = false;
    if (!attr_set && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
        if (e != cudaSuccess) return li_fail("attention (decode): cannot raise shared memory: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    LI_REQUIRE(smem <= 100 * 1024, "attention (decode): shared memory %zu too large", smem);
    LI_REQUIRE(S <= 65535 && nkv <= 65535, "attention (decode): batch %d or kv heads %d too large for one launch", S, nkv);
    dim3 grid(nsplit, nkv, S);
    decode_attention_kernel<DH><<<grid, kWarps * 32, smem, stream>>>((const bf16*)qkv, (const bf16*)kcache, (const bf16*)vcache,
                                                                      block_table, max_blocks, ctx_lens, part, nh, nkv, page_size,
                                                                      num_pages, scale, window, nsplit);
    if (int rc = li_check_launch("attention (decode)")) return rc;
    decode_combine_kernel<DH><<<S * nh, DH < 32 ? 32 : (DH > 128 ? 128 : DH), 0, stream>>>(part, ctx_lens, (bf16*)out, nh, window, nsplit);
    return li_check_launch("attention (decode combine)");
}

}  // namespace

bool li_attention_decode_accepts(int nh, int nkv, int dh, int page_size) {
    const bool dh_ok = (dh % 16 == 0 && dh >= 16 && dh <= 128) || dh == 256;
    return dh_ok && nh % nkv == 0 && nh / nkv <= 16 && page_size % 16 == 0;
}

int li_attention_decode(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                        const int* ctx_lens, int S, int nh, int nkv, int dh, int page_size, int num_pages, float scale, int window,
                        int max_ctx_len, cudaStream_t stream) {
#define LI_CASE(D)                                                                                                             \
    case D:                                                                                                                    \
        return launch<D>(qkv, out, kcache, vcache, block_table, max_blocks, ctx_lens, S, nh, nkv, page_size, num_pages, scale, \
                         window, max_ctx_len, stream);
    switch (dh) {
        LI_CASE(16) LI_CASE(32) LI_CASE(48) LI_CASE(64) LI_CASE(80) LI_CASE(96) LI_CASE(112) LI_CASE(128) LI_CASE(256)
        default:
            return li_fail("attention (decode): head_dim %d is not supported by this kernel", dh);
    }
#undef LI_CASE
}
