// RMSNorm between two products without a kernel of its own, for few tokens (decode).
//
//     y = w_norm * x / sqrt(mean(x^2) + eps)      (src/ops/rms_norm/op.cpp:13-24)
//     out = y W^T = rinv(x) * ((w_norm * x) W^T),   rinv(x) = 1 / sqrt(mean(x^2) + eps) per token
//
// The product that writes into the residual stream x (o, down) adds its columns to x in its epilogue and,
// while it has them, stores h' = bfloat16(w_norm * x) for the next product and the sum of x^2 over its own
// columns, per token (AddScaled).  The next product (q|k|v, gate|up) multiplies h' as it is and scales each
// token's row of the result by rinv, which it gets from the partial sums, added in the order of the parts
// (RowScale).  Nothing waits for anything: every CTA works on its own columns.  Sum of squares, reciprocal
// root and the residual sum are float32; h' is rounded once, like the normalised activation it stands for.
#pragma once

#include "common.cuh"

struct RowScale {
    const float* ssq = nullptr;    // [M, nparts] partial sums of x^2; nullptr: no scaling
    int nparts = 0;
    float width = 1.0f;            // number of elements the sums cover (the hidden size)
    float eps = 0.0f;
};

struct AddScaled {
    float* x32 = nullptr;          // [M, N] residual stream, updated in place
    const float* norm_weight = nullptr;   // [N]
    bf16* hprime = nullptr;        // [M, N] bfloat16(norm_weight * x32)
    float* ssq_out = nullptr;      // [M, tiles of this product]
};

// rinv of token `tok` from the partial sums: lanes take every 32nd part in ascending order, then a butterfly.
__device__ __forceinline__ float row_scale_of(const RowScale& rs, int tok, int lane) {
    float s = 0.0f;
    for (int p = lane; p < rs.nparts; p += 32) s += __ldcg(rs.ssq + (size_t)tok * rs.nparts + p);
    s = warp_sum(s);
    return 1.0f / sqrtf(s / rs.width + rs.eps);
}

// The same for the tokens first, first + stride, ... < M of one warp into out_sm[token], with the loads of TB tokens
// in flight at once (up to 128 parts; the order of summation is that of row_scale_of).
template <int TB>
__device__ __forceinline__ void row_scales_of_warp(const RowScale& rs, int M, int first, int stride, int lane, float* out_sm) {
    for (int t0 = first; t0 < M; t0 += TB * stride) {
        if (rs.nparts <= 128) {
            float pre[TB][4];
#pragma unroll
            for (int ti = 0; ti < TB; ++ti) {
                const int tok = t0 + ti * stride;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int p = lane + 32 * q;
                    pre[ti][q] = (tok < M && p < rs.nparts) ? __ldcg(rs.ssq + (size_t)tok * rs.nparts + p) : 0.0f;
                }
            }
#pragma unroll
            for (int ti = 0; ti < TB; ++ti) {
                const int tok = t0 + ti * stride;
                const float ssum = warp_sum(((pre[ti][0] + pre[ti][1]) + pre[ti][2]) + pre[ti][3]);
                if (lane == 0 && tok < M) out_sm[tok] = 1.0f / sqrtf(ssum / rs.width + rs.eps);
            }
        } else {
            for (int ti = 0; ti < TB; ++ti) {
                const int tok = t0 + ti * stride;
                if (tok < M) {
                    const float r = row_scale_of(rs, tok, lane);
                    if (lane == 0) out_sm[tok] = r;
                }
            }
        }
    }
}
