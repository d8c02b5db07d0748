// Choosing the next token on the device: argmax, and temperature / top-k /
// top-p sampling, one block per logits row.
//
// Candidates as LitInfer's sampler keeps them (src/llaisys/models/qwen2.cpp:890-920):
// z = logits / temperature; the top_k largest if 0 < k < V; softmax over
// those; the shortest prefix, in descending order, whose cumulative
// probability reaches top_p if 0 < p < 1.  Instead of sorting, the two
// thresholds are found by bisection over the order-preserving integer image
// of a float (32 steps each, every step one pass over the row):
//   t_k = smallest t with  #{z_i > t} < k                  (the k-th largest value)
//   t_p = smallest t with  sum_{z_i > t} prob_i < top_p    (a token stays iff the
//         probability mass of strictly larger candidates is below top_p)
// Equal values stay or go together.  The draw is Gumbel-max over the
// candidates, argmax(z_i + g_i), g_i = -log(-log(u_i)), with u_i a hash of
// (seed, index of the output token, i): exact sampling from the candidates'
// softmax that depends on nothing outside the request.  The first maximum wins
// ties (src/ops/argmax/op.cpp:28-33).  All sums are in a fixed order.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ float gumbel(unsigned long long key, int token) {
    const unsigned long long bits = splitmix64(key ^ ((unsigned long long)token * 0xD1342543DE82EF95ull)) >> 41;   // 23 bits
    const float u = ((float)bits + 0.5f) * (1.0f / 8388608.0f);                                                    // in (0, 1), exact
    return -logf(-logf(u));
}

__device__ __forceinline__ unsigned sortable(float f) {
    const unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Best {
    float v;
    int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ Best block_best(Best x, Best* scratch /* 32 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    Best r = (lane < nwarps) ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = better(r, y);
    }
    return r;
}

__device__ Best row_argmax(const float* row, int V, Best* scratch) {
    Best b{-INFINITY, 0x7fffffff};
    // eight loads in flight per thread: the row comes from L2 and one load at a time would wait out its latency each time
    constexpr int U = 8;
    int i = threadIdx.x;
    for (; i + (U - 1) * (int)blockDim.x < V; i += U * blockDim.x) {
        float v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = row[i + u * blockDim.x];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (v[u] > b.v) b = Best{v[u], i + u * (int)blockDim.x};      // ascending index per thread: the first maximum stays
    }
    for (; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > b.v) b = Best{v, i};
    }
    b = block_best(b, scratch);
    if (b.i == 0x7fffffff) b.i = 0;             // a row of NaN or -inf
    return b;
}

__global__ void __launch_bounds__(kThreads) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
    __shared__ Best scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const Best b = row_argmax(logits + (size_t)blockIdx.x * V, V, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = b.i;
}

// Few rows of a large vocabulary (decode): one CTA a row would read its 600 KB alone while the rest of the GPU waits.  A row
// is cut into kChunks pieces; the CTA that finishes a row last (a counter per row) picks the best of the pieces, the
// first maximum again: pieces are compared in ascending order of their indices.
constexpr int kChunks = 16;
constexpr int kChunkRows = 1024;                 // rows the static scratch below holds
__device__ Best g_chunk_best[kChunkRows * kChunks];
__device__ unsigned g_chunk_done[kChunkRows];    // zero between launches

__global__ void __launch_bounds__(256) argmax_chunks_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
    __shared__ Best scratch[32];
    __shared__ int is_last;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, chunk = blockIdx.x;
    const int per = (((V + kChunks - 1) / kChunks) + 3) & ~3;
    const int lo = chunk * per, hi = min(V, lo + per);
    Best b{-INFINITY, 0x7fffffff};
    if (lo < hi) {
        b = row_argmax(logits + (size_t)row * V + lo, hi - lo, scratch);
        // a chunk without a finite maximum (all NaN or -inf) must not win with a made-up index
        if (!(b.v > -INFINITY)) b = Best{-INFINITY, 0x7fffffff};
        else b.i += lo;
    }
    if (threadIdx.x == 0) {
        g_chunk_best[row * kChunks + chunk] = b;
        __threadfence();
        is_last = atomicAdd(&g_chunk_done[row], 1u) == (unsigned)(kChunks - 1);
    }
    __syncthreads();
    if (!is_last || threadIdx.x != 0) return;
    __threadfence();
    Best r{-INFINITY, 0x7fffffff};
    for (int c = 0; c < kChunks; ++c) {
        const volatile Best* p = &g_chunk_best[row * kChunks + c];
        r = better(r, Best{p->v, p->i});
    }
    out[row] = r.i == 0x7fffffff ? 0 : r.i;      // a row of NaN or -inf
    g_chunk_done[row] = 0;                       // ready for the next launch on this stream
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const float* __restrict__ logits, const int* __restrict__ params,
                                                          int* __restrict__ out, int V) {
    __shared__ Best scratch[32];
    __shared__ float fscratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * V;
    const int* pr = params + r * 6;
    const float temperature = __int_as_float(pr[0]);
    const int top_k = pr[1];
    const float top_p = __int_as_float(pr[2]);
    const unsigned long long seed = (unsigned long long)(unsigned)pr[3] | ((unsigned long long)(unsigned)pr[4] << 32);
    const unsigned long long index = (unsigned long long)(long long)pr[5];

    const Best top = row_argmax(row, V, scratch);
    if (temperature <= 0.0f || top_k == 1) {
        if (threadIdx.x == 0) out[r] = top.i;
        return;
    }
    const float zmax = top.v / temperature;
    unsigned keep_from = 0;                       // candidates: sortable(z_i) >= keep_from

    if (top_k > 0 && top_k < V) {
        unsigned lo = 0, hi = 0xFFFFFFFFu;
        while (lo < hi) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            float cnt = 0.0f;                     // counts below 2^24 are exact in float
            for (int i = threadIdx.x; i < V; i += blockDim.x) cnt += (sortable(row[i] / temperature) > mid) ? 1.0f : 0.0f;
            cnt = block_sum(cnt, fscratch);
            if (cnt < (float)top_k) hi = mid; else lo = mid + 1;
        }
        keep_from = lo;
    }
    if (top_p > 0.0f && top_p < 1.0f) {
        float z = 0.0f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float zi = row[i] / temperature;
            if (sortable(zi) >= keep_from) z += expf(zi - zmax);
        }
        z = block_sum(z, fscratch);
        const float target = top_p * z;           // compare unnormalised masses with top_p * Z
        unsigned lo = keep_from, hi = 0xFFFFFFFFu;
        while (lo < hi) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            float mass = 0.0f;
            for (int i = threadIdx.x; i < V; i += blockDim.x) {
                const float zi = row[i] / temperature;
                if (sortable(zi) > mid) mass += expf(zi - zmax);
            }
            mass = block_sum(mass, fscratch);
            if (mass < target) hi = mid; else lo = mid + 1;
        }
        if (lo > keep_from) keep_from = lo;
    }
    const unsigned long long key = splitmix64(seed ^ splitmix64(index));
    Best b{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float zi = row[i] / temperature;
        if (sortable(zi) >= keep_from) {
            const float v = zi + gumbel(key, i);
            if (v > b.v) b = Best{v, i};
        }
    }
    b = block_best(b, scratch);
    if (threadIdx.x == 0) out[r] = (b.i == 0x7fffffff) ? top.i : b.i;
}

}  // namespace

LI_EXPORT int li_argmax(const float* logits, int* out, int R, int V, cudaStream_t stream) {
    LI_REQUIRE(R >= 0 && V > 0, "argmax: bad sizes R=%d V=%d", R, V);
    if (R == 0) return 0;
    if (R <= 64 && R <= kChunkRows && V >= 16384) {
        li_launch_pdl(argmax_chunks_kernel, dim3(kChunks, R), dim3(256), 0, stream, logits, out, V);
        return li_check_launch("argmax (chunks)");
    }
    li_launch_pdl(argmax_kernel, dim3(R), dim3(kThreads), 0, stream, logits, out, V);
    return li_check_launch("argmax");
}

LI_EXPORT int li_sample(const float* logits, const int* params, int* out, int R, int V, cudaStream_t stream) {
    LI_REQUIRE(R >= 0 && V > 0, "sample: bad sizes R=%d V=%d", R, V);
    LI_REQUIRE(V < (1 << 24), "sample: vocabulary %d is too large", V);
    if (R == 0) return 0;
    li_launch_pdl(sample_kernel, dim3(R), dim3(kThreads), 0, stream, logits, params, out, V);
    return li_check_launch("sample");
}
