// The inner step shared by the bfloat16 attention kernels: 16 query rows
// against 16 cached keys with mma.sync m16n8k16, online softmax in float.
//
// Operands go from global memory straight into fragment registers with 8-byte
// loads, no shared memory and no ldmatrix:
//   * S = Q K^T sums over head_dim, in any order: the 4 consecutive elements a
//     thread loads from a query row and from a key row serve as the element
//     pairs (2t, 2t+1) and (2t+8, 2t+9) of the fragment layout on both sides;
//   * O += P V sums over keys, in any order, and values are cached transposed
//     ([head_dim][slot]): for an output column the 4 consecutive keys a thread
//     loads are pairs of the fragment layout too, provided the score tiles
//     carry their key columns in the matching order.  Tile 0 holds keys
//     0,1,4,5,8,9,12,13 of the 16, tile 1 keys 2,3,6,7,10,11,14,15: thread t of
//     a quad then owns the scores of keys 4t..4t+3.
// Softmax recurrence as in LitInfer (src/ops/paged_attention/op.cpp:194-234):
// m' = max(m, s); alpha = exp(m - m'); p = exp(s - m'); l = l alpha + sum p;
// O = O alpha + p V.  Rows whose keys are all masked so far keep m = -inf.
#pragma once

#include "common.cuh"

namespace attn {

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Queries are read past L1 (from L2): inside a persistent kernel they were written a moment ago by another
// multiprocessor, and L1 is not kept coherent with that.
__device__ __forceinline__ uint2 ld8(const bf16* p) { return __ldcg(reinterpret_cast<const uint2*>(p)); }
__device__ __forceinline__ uint4 ld16(const bf16* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ uint2 ld8_stream(const bf16* p) {
    uint2 v;
    asm volatile("ld.global.cs.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ uint2 ld8_keep(const bf16* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }

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

// Running state of a warp's 16 rows: this thread sees rows g (index 0) and g + 8 (index 1).
template <int DH>
struct RowState {
    float o[DH / 8][4];
    float m[2], l[2];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int j = 0; j < DH / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.0f;
    }
};

// Query fragments of 16 rows: row_lo / row_hi point at the head_dim elements of rows g and g + 8 (nullptr: a row of zeros).
template <int DH>
__device__ __forceinline__ void load_q(unsigned (&qa)[DH / 16][4], const bf16* row_lo, const bf16* row_hi, int t) {
#pragma unroll
    for (int st = 0; st < DH / 16; ++st) {
        const uint2 r0 = row_lo ? ld8(row_lo + st * 16 + t * 4) : make_uint2(0, 0);
        const uint2 r1 = row_hi ? ld8(row_hi + st * 16 + t * 4) : make_uint2(0, 0);
        qa[st][0] = r0.x; qa[st][1] = r1.x; qa[st][2] = r0.y; qa[st][3] = r1.y;
    }
}

// Fragments of one block of 16 keys.  kbase: the block's first key row ([16][DH], rows DH
// apart); vbase: the block's first slot in the transposed values ([DH][page_size]).
// kStream: the cache is read once (decode) and should not displace other data.
template <int DH>
struct KFrag {
    uint2 t0[DH / 16], t1[DH / 16];      // score tile 0 / tile 1
};
template <int DH>
struct VFrag {
    uint2 v[DH / 8];
};

template <int DH, bool kStream>
__device__ __forceinline__ void load_k(KFrag<DH>& k, const bf16* kbase, int g, int t) {
    const int key_c0 = 4 * (g >> 1) + (g & 1);
    const bf16* k0 = kbase + (size_t)key_c0 * DH + t * 4;
    const bf16* k1 = k0 + 2 * DH;
#pragma unroll
    for (int s = 0; s < DH / 16; ++s) {
        k.t0[s] = kStream ? ld8_stream(k0 + s * 16) : ld8_keep(k0 + s * 16);
        k.t1[s] = kStream ? ld8_stream(k1 + s * 16) : ld8_keep(k1 + s * 16);
    }
}

template <int DH, bool kStream>
__device__ __forceinline__ void load_v(VFrag<DH>& v, const bf16* vbase, int page_size, int g, int t) {
    const bf16* vcol = vbase + (size_t)g * page_size + 4 * t;
#pragma unroll
    for (int j = 0; j < DH / 8; ++j) v.v[j] = kStream ? ld8_stream(vcol + (size_t)j * 8 * page_size) : ld8_keep(vcol + (size_t)j * 8 * page_size);
}

// 16 rows against the 16 keys whose fragments are given; key0 is the absolute position of the
// block's first key.  A key is visible to row r iff lo[r] <= key <= hi[r].
template <int DH>
__device__ __forceinline__ void compute16(RowState<DH>& st, const unsigned (&qa)[DH / 16][4], const KFrag<DH>& kf, const VFrag<DH>& vf,
                                          int key0, const int (&lo)[2], const int (&hi)[2], float scale, int t) {
    constexpr int KS = DH / 16, NT = DH / 8;
    const uint2* kb0 = kf.t0;
    const uint2* kb1 = kf.t1;
    const uint2* vb = vf.v;
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < KS; ++s) {
        mma_bf16(s0, qa[s][0], qa[s][1], qa[s][2], qa[s][3], kb0[s].x, kb0[s].y);
        mma_bf16(s1, qa[s][0], qa[s][1], qa[s][2], qa[s][3], kb1[s].x, kb1[s].y);
    }
    // this thread's keys: key0 + 4 t + {0, 1} (tile 0) and + {2, 3} (tile 1)
    const int kk = key0 + 4 * t;
    float p[2][4];
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float v0 = (kk >= lo[r] && kk <= hi[r]) ? s0[2 * r] * scale : -INFINITY;
        const float v1 = (kk + 1 >= lo[r] && kk + 1 <= hi[r]) ? s0[2 * r + 1] * scale : -INFINITY;
        const float v2 = (kk + 2 >= lo[r] && kk + 2 <= hi[r]) ? s1[2 * r] * scale : -INFINITY;
        const float v3 = (kk + 3 >= lo[r] && kk + 3 <= hi[r]) ? s1[2 * r + 1] * scale : -INFINITY;
        const float mx = quad_max(fmaxf(fmaxf(v0, v1), fmaxf(v2, v3)));
        const float mn = fmaxf(st.m[r], mx);
        const float ms = (mn == -INFINITY) ? 0.0f : mn;         // nothing visible yet: keep everything at zero
        alpha[r] = expf(st.m[r] - ms);
        p[r][0] = expf(v0 - ms); p[r][1] = expf(v1 - ms); p[r][2] = expf(v2 - ms); p[r][3] = expf(v3 - ms);
        st.l[r] = st.l[r] * alpha[r] + (p[r][0] + p[r][1] + p[r][2] + p[r][3]);
        st.m[r] = mn;
    }
    const unsigned pa0 = pack_bf16(p[0][0], p[0][1]), pa1 = pack_bf16(p[1][0], p[1][1]);
    const unsigned pa2 = pack_bf16(p[0][2], p[0][3]), pa3 = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        st.o[j][0] *= alpha[0]; st.o[j][1] *= alpha[0]; st.o[j][2] *= alpha[1]; st.o[j][3] *= alpha[1];
        mma_bf16(st.o[j], pa0, pa1, pa2, pa3, vb[j].x, vb[j].y);
    }
}

// ---- the same step on 32 keys with 16-byte loads (decode: half as many memory requests per byte) ----
//
// Thread t of a quad owns keys 8t .. 8t+7 of the block: a 16-byte load of a value column gives it both
// k-steps of P V (keys 8t..8t+3 and 8t+4..8t+7), and score tile 2s+h carries in column n the key
// 8 (n >> 1) + 4 s + 2 h + (n & 1).  Along head_dim a 16-byte load of a key row (8 elements) serves two
// k-steps of Q K^T; the query fragments are permuted the same way (load_q32).  head_dim = 32 F + 16 R.

template <int DH>
struct KFrag32 {
    uint4 k[4][DH / 32 > 0 ? DH / 32 : 1];
    uint2 tail[4];
};
template <int DH>
struct VFrag32 {
    uint4 v[DH / 8];
};

template <int DH>
__device__ __forceinline__ void load_q32(unsigned (&qa)[DH / 16][4], const bf16* row_lo, const bf16* row_hi, int t) {
    constexpr int F = DH / 32, R = (DH % 32) / 16;
#pragma unroll
    for (int f = 0; f < F; ++f) {
        const uint4 a = row_lo ? ld16(row_lo + f * 32 + t * 8) : make_uint4(0, 0, 0, 0);
        const uint4 b = row_hi ? ld16(row_hi + f * 32 + t * 8) : make_uint4(0, 0, 0, 0);
        qa[2 * f][0] = a.x; qa[2 * f][1] = b.x; qa[2 * f][2] = a.y; qa[2 * f][3] = b.y;
        qa[2 * f + 1][0] = a.z; qa[2 * f + 1][1] = b.z; qa[2 * f + 1][2] = a.w; qa[2 * f + 1][3] = b.w;
    }
    if (R) {
        const uint2 a = row_lo ? ld8(row_lo + F * 32 + t * 4) : make_uint2(0, 0);
        const uint2 b = row_hi ? ld8(row_hi + F * 32 + t * 4) : make_uint2(0, 0);
        qa[DH / 16 - 1][0] = a.x; qa[DH / 16 - 1][1] = b.x; qa[DH / 16 - 1][2] = a.y; qa[DH / 16 - 1][3] = b.y;
    }
}

__device__ __forceinline__ uint4 ld16_stream(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// kgroup: the first of the 8 key rows [8 (g >> 1), 8 (g >> 1) + 8) of the block, which lie in one page
// ([8][DH], rows DH apart).  This thread's rows in the four score tiles are (g & 1) + {0, 2, 4, 6} of them.
template <int DH>
__device__ __forceinline__ void load_k32(KFrag32<DH>& kf, const bf16* kgroup, int g, int t) {
    constexpr int F = DH / 32, R = (DH % 32) / 16;
#pragma unroll
    for (int tau = 0; tau < 4; ++tau) {
        const bf16* row = kgroup + (size_t)((g & 1) + 4 * (tau >> 1) + 2 * (tau & 1)) * DH;
#pragma unroll
        for (int f = 0; f < F; ++f) kf.k[tau][f] = ld16_stream(row + f * 32 + t * 8);
        if (R) kf.tail[tau] = ld8_stream(row + F * 32 + t * 4);
    }
}

// vkeys: slot of key 8 t of the block in the transposed values of its page ([DH][page_size]), for this thread's t.
template <int DH>
__device__ __forceinline__ void load_v32(VFrag32<DH>& vf, const bf16* vkeys, int page_size, int g) {
#pragma unroll
    for (int j = 0; j < DH / 8; ++j) vf.v[j] = ld16_stream(vkeys + (size_t)(j * 8 + g) * page_size);
}

template <int DH>
__device__ __forceinline__ void compute32(RowState<DH>& st, const unsigned (&qa)[DH / 16][4], const KFrag32<DH>& kf, const VFrag32<DH>& vf,
                                          int key0, const int (&lo)[2], const int (&hi)[2], float scale, int t) {
    constexpr int F = DH / 32, R = (DH % 32) / 16, NT = DH / 8;
    float sc[4][4];
#pragma unroll
    for (int tau = 0; tau < 4; ++tau) {
        sc[tau][0] = sc[tau][1] = sc[tau][2] = sc[tau][3] = 0.0f;
#pragma unroll
        for (int f = 0; f < F; ++f) {
            mma_bf16(sc[tau], qa[2 * f][0], qa[2 * f][1], qa[2 * f][2], qa[2 * f][3], kf.k[tau][f].x, kf.k[tau][f].y);
            mma_bf16(sc[tau], qa[2 * f + 1][0], qa[2 * f + 1][1], qa[2 * f + 1][2], qa[2 * f + 1][3], kf.k[tau][f].z, kf.k[tau][f].w);
        }
        if (R) mma_bf16(sc[tau], qa[DH / 16 - 1][0], qa[DH / 16 - 1][1], qa[DH / 16 - 1][2], qa[DH / 16 - 1][3], kf.tail[tau].x, kf.tail[tau].y);
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float mx = -INFINITY;
#pragma unroll
        for (int tau = 0; tau < 4; ++tau) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + 8 * t + 4 * (tau >> 1) + 2 * (tau & 1) + e;
                float& v = sc[tau][2 * r + e];
                v = (key >= lo[r] && key <= hi[r]) ? v * scale : -INFINITY;
                mx = fmaxf(mx, v);
            }
        }
        mx = quad_max(mx);
        const float mn = fmaxf(st.m[r], mx);
        const float ms = (mn == -INFINITY) ? 0.0f : mn;
        alpha[r] = expf(st.m[r] - ms);
        float sum = 0.0f;
#pragma unroll
        for (int tau = 0; tau < 4; ++tau) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float& v = sc[tau][2 * r + e];
                v = expf(v - ms);
                sum += v;
            }
        }
        st.l[r] = st.l[r] * alpha[r] + sum;
        st.m[r] = mn;
    }
    unsigned pa[2][4];
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2) {
        pa[s2][0] = pack_bf16(sc[2 * s2][0], sc[2 * s2][1]);
        pa[s2][1] = pack_bf16(sc[2 * s2][2], sc[2 * s2][3]);
        pa[s2][2] = pack_bf16(sc[2 * s2 + 1][0], sc[2 * s2 + 1][1]);
        pa[s2][3] = pack_bf16(sc[2 * s2 + 1][2], sc[2 * s2 + 1][3]);
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        st.o[j][0] *= alpha[0]; st.o[j][1] *= alpha[0]; st.o[j][2] *= alpha[1]; st.o[j][3] *= alpha[1];
        mma_bf16(st.o[j], pa[0][0], pa[0][1], pa[0][2], pa[0][3], vf.v[j].x, vf.v[j].y);
        mma_bf16(st.o[j], pa[1][0], pa[1][1], pa[1][2], pa[1][3], vf.v[j].z, vf.v[j].w);
    }
}

}  // namespace attn
