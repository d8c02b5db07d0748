// The epilogue of the tcgen05 GEMM kernels for one 32-column piece of one row of the product (this thread's row of an
// accumulator): bias in float or SwiGLU of interleaved columns, one rounding, stores of 16 bytes where alignment allows.
#pragma once

#include "common.cuh"

// v: columns col0 .. col0 + 31 of row `row` of a w^T.  kSwiglu: the columns come as 8 gate, 8 up, 8 gate, 8 up and give 16
// activations up * gate / (1 + exp(-gate)) (src/ops/swiglu/op.cpp:17-23) at columns col0 / 2 .. of a row of N / 2.
template <typename Tout, bool kSwiglu>
__device__ __forceinline__ void gemm_store_piece(int row, int col0, float (&v)[32], const float* __restrict__ bias, Tout* __restrict__ out,
                                                 int M, int N) {
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
                    a16[8 * h + i] = swiglu_of<Tout>(gate, up);
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
