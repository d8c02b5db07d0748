// Choosing the next token on the device: argmax, and temperature / top-k /
// top-p sampling, one block per logits row.
//
// Candidates as LitInfer's sampler keeps them (src/llaisys/models/qwen2.cpp:890-920):
// z = logits / temperature; the top_k largest if 0 < k < V; softmax over
// those; the shortest prefix, in descending order, whose cumulative
// probability reaches top_p if 0 < p < 1.  Instead of sorting, two thresholds
// over the order-preserving integer image of a float decide who stays:
//   t_k = smallest t with  #{z_i > t} < k                  (the k-th largest value)
//   t_p = smallest t with  sum_{z_i > t} prob_i < top_p    (a token stays iff the
//         probability mass of strictly larger candidates is below top_p)
// t_k comes from radix selection (three passes over the row with a histogram
// in shared memory); the values at or above it are gathered into shared
// memory in a fixed order, and t_p and the draw are found there.  Rows whose
// candidates do not fit (a flat distribution with top_p alone) and small
// vocabularies take bisection over the whole row, 32 passes a threshold.
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

// f(i, row[i]) for this thread's elements i = threadIdx.x, + blockDim.x, ... in ascending order, eight loads in flight:
// the row comes from L2, and one load at a time would wait out its latency each time
template <typename F>
__device__ __forceinline__ void for_each_element(const float* __restrict__ row, int V, F f) {
    constexpr int U = 8;
    int i = threadIdx.x;
    for (; i + (U - 1) * (int)blockDim.x < V; i += U * blockDim.x) {
        float v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = row[i + u * blockDim.x];
#pragma unroll
        for (int u = 0; u < U; ++u) f(i + u * (int)blockDim.x, v[u]);
    }
    for (; i < V; i += blockDim.x) f(i, row[i]);
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

// The thresholds by bisection with a pass over the whole row per step (64 passes for top-k and top-p): for small
// vocabularies, and where the selection below cannot be used.
__device__ void sample_row_by_bisection(const float* __restrict__ row, int V, float temperature, int top_k, float top_p,
                                        unsigned long long seed, unsigned long long index, Best top, int* __restrict__ out_token,
                                        Best* scratch, float* fscratch) {
    const float zmax = top.v / temperature;
    unsigned keep_from = 0;                       // candidates: sortable(z_i) >= keep_from

    if (top_k > 0 && top_k < V) {
        unsigned lo = 0, hi = 0xFFFFFFFFu;
        while (lo < hi) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            float cnt = 0.0f;                     // counts below 2^24 are exact in float
            for_each_element(row, V, [&](int, float x) { cnt += (sortable(x / temperature) > mid) ? 1.0f : 0.0f; });
            cnt = block_sum(cnt, fscratch);
            if (cnt < (float)top_k) hi = mid; else lo = mid + 1;
        }
        keep_from = lo;
    }
    if (top_p > 0.0f && top_p < 1.0f) {
        float z = 0.0f;
        for_each_element(row, V, [&](int, float x) {
            const float zi = x / temperature;
            if (sortable(zi) >= keep_from) z += expf(zi - zmax);
        });
        z = block_sum(z, fscratch);
        const float target = top_p * z;           // compare unnormalised masses with top_p * Z
        unsigned lo = keep_from, hi = 0xFFFFFFFFu;
        while (lo < hi) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            float mass = 0.0f;
            for_each_element(row, V, [&](int, float x) {
                const float zi = x / temperature;
                if (sortable(zi) > mid) mass += expf(zi - zmax);
            });
            mass = block_sum(mass, fscratch);
            if (mass < target) hi = mid; else lo = mid + 1;
        }
        if (lo > keep_from) keep_from = lo;
    }
    const unsigned long long key = splitmix64(seed ^ splitmix64(index));
    Best b{-INFINITY, 0x7fffffff};
    for_each_element(row, V, [&](int i, float x) {
        const float zi = x / temperature;
        if (sortable(zi) >= keep_from) {
            const float v = zi + gumbel(key, i);
            if (v > b.v) b = Best{v, i};
        }
    });
    b = block_best(b, scratch);
    if (threadIdx.x == 0) *out_token = (b.i == 0x7fffffff) ? top.i : b.i;
}

// Temperature alone (no top-k, no top-p): the draw is one reduction, argmax(z_i + g_i) over the whole row, and is cut into
// pieces over many CTAs like argmax_chunks_kernel.  Rows with other options are left to sample_kernel (`handled` says which).
constexpr int kDrawChunks = 64;                  // the draw costs a hash and two logarithms per token: more, smaller pieces
__device__ Best g_draw_best[kChunkRows * kDrawChunks];
__device__ unsigned g_draw_done[kChunkRows];     // zero between launches

__global__ void __launch_bounds__(256) sample_temperature_chunks_kernel(const float* __restrict__ logits, const int* __restrict__ params,
                                                                        int* __restrict__ out, int V) {
    __shared__ Best scratch[32];
    __shared__ int is_last;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, chunk = blockIdx.x;
    const int* pr = params + row * 6;
    const float temperature = __int_as_float(pr[0]);
    const int top_k = pr[1];
    const float top_p = __int_as_float(pr[2]);
    const bool plain = temperature > 0.0f && !(top_k > 0 && top_k < V) && top_k != 1 && !(top_p > 0.0f && top_p < 1.0f);
    if (!plain) return;                                  // the whole grid row agrees
    const unsigned long long seed = (unsigned long long)(unsigned)pr[3] | ((unsigned long long)(unsigned)pr[4] << 32);
    const unsigned long long key = splitmix64(seed ^ splitmix64((unsigned long long)(long long)pr[5]));
    const int per = (((V + kDrawChunks - 1) / kDrawChunks) + 3) & ~3;
    const int lo = chunk * per, hi = min(V, lo + per);
    Best b{-INFINITY, 0x7fffffff};
    if (lo < hi) {
        for_each_element(logits + (size_t)row * V + lo, hi - lo, [&](int i, float x) {
            const float v = x / temperature + gumbel(key, lo + i);
            if (v > b.v) b = Best{v, lo + i};
        });
        b = block_best(b, scratch);
    }
    if (threadIdx.x == 0) {
        g_draw_best[row * kDrawChunks + chunk] = b;
        __threadfence();
        is_last = atomicAdd(&g_draw_done[row], 1u) == (unsigned)(kDrawChunks - 1);
    }
    __syncthreads();
    if (!is_last || threadIdx.x != 0) return;
    __threadfence();
    Best r{-INFINITY, 0x7fffffff};
    for (int c = 0; c < kDrawChunks; ++c) {
        const volatile Best* p = &g_draw_best[row * kDrawChunks + c];
        r = better(r, Best{p->v, p->i});
    }
    if (r.i != 0x7fffffff) out[row] = r.i;               // else (nothing finite) sample_kernel's answer stands: the first maximum
    g_draw_done[row] = 0;
}

__device__ __forceinline__ float unsortable(unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k); }

// Large vocabularies.  The same candidates and the same draw with few passes over the row: the k-th largest value by
// radix selection on the sortable image of z (three passes: 11, 11 and 10 bits, a histogram in shared memory each), the
// candidates (at most kCand of them) gathered into shared memory in a fixed order, and top-p and the draw done there.
// With top-p alone the kCand largest are gathered first: if they hold at least top_p of the mass, the cut lies among them
// (a token below them has at least that mass above it); if not (a very flat distribution), the bisection above runs.
constexpr int kCand = 4096;

struct SelectShared {
    unsigned hist[2048];
    unsigned ckey[kCand];
    int cidx[kCand];
    unsigned scan[kThreads];
    unsigned warp_total[32];
    unsigned prefix, need;
};

// One round of the selection: among the keys that match `prefix` under `mask`, the digit (`bits` bits at `shift`) that
// holds the need-th largest; prefix and need are updated in shared memory.  extra(i, z, key) is called for every element.
template <typename Extra>
__device__ void select_round(const float* __restrict__ row, int V, float temperature, unsigned mask, int shift, int bits, SelectShared& sh,
                             Extra extra) {
    const int nb = 1 << bits;
    for (int i = threadIdx.x; i < nb; i += blockDim.x) sh.hist[i] = 0;
    __syncthreads();
    const unsigned prefix = sh.prefix;
    for_each_element(row, V, [&](int i, float x) {
        const float z = x / temperature;
        const unsigned key = sortable(z);
        extra(i, z, key);
        if ((key & mask) == prefix) atomicAdd(&sh.hist[(key >> shift) & (unsigned)(nb - 1)], 1u);       // integer counts: any order
    });
    __syncthreads();
    if (threadIdx.x < 32) {
        // lane l takes the digits nb - 1 - (per * l) downwards
        const int per = nb / 32, lane = threadIdx.x;
        unsigned mine = 0;
        for (int j = 0; j < per; ++j) mine += sh.hist[nb - 1 - (lane * per + j)];
        unsigned incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned y = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += y;
        }
        const unsigned before = incl - mine, need = sh.need;
        if (before < need && need <= incl) {
            unsigned run = before;
            for (int j = 0; j < per; ++j) {
                const int d = nb - 1 - (lane * per + j);
                const unsigned c = sh.hist[d];
                if (run + c >= need) {
                    sh.prefix = prefix | ((unsigned)d << shift);
                    sh.need = need - run;
                    break;
                }
                run += c;
            }
        }
    }
    __syncthreads();
}

__device__ unsigned block_exclusive_scan(unsigned v, SelectShared& sh, unsigned* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
    }
    if (lane == 31) sh.warp_total[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const unsigned w = lane < (int)(blockDim.x >> 5) ? sh.warp_total[lane] : 0u;
        unsigned wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned y = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += y;
        }
        sh.warp_total[lane] = wi - w;                   // exclusive
        if (lane == 31) sh.scan[0] = wi;                // the total
    }
    __syncthreads();
    *total = sh.scan[0];
    const unsigned r = sh.warp_total[warp] + incl - v;
    __syncthreads();
    return r;
}

// chunked_plain: rows with temperature alone are drawn by sample_temperature_chunks_kernel, launched after this kernel; here
// they only get the first maximum as a stand-in (which stays if the row has nothing finite).
__global__ void __launch_bounds__(kThreads) sample_kernel(const float* __restrict__ logits, const int* __restrict__ params,
                                                          int* __restrict__ out, int V, int chunked_plain) {
    __shared__ Best scratch[32];
    __shared__ float fscratch[32];
    __shared__ SelectShared sh;
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

    const bool use_k = top_k > 0 && top_k < V, use_p = top_p > 0.0f && top_p < 1.0f;
    if (chunked_plain && temperature > 0.0f && top_k != 1 && !use_k && !use_p) {
        if (threadIdx.x == 0) out[r] = 0;                // stands only if the row has nothing finite (what the first maximum would give)
        return;
    }
    const Best top = row_argmax(row, V, scratch);
    if (temperature <= 0.0f || top_k == 1) {
        if (threadIdx.x == 0) out[r] = top.i;
        return;
    }
    if (V <= kCand || !(use_k || use_p) || (use_k && top_k > kCand)) {
        sample_row_by_bisection(row, V, temperature, top_k, top_p, seed, index, top, out + r, scratch, fscratch);
        return;
    }
    const float zmax = top.v / temperature;
    // the k-th largest key (top-k), or the kCand-th largest (top-p alone)
    if (threadIdx.x == 0) {
        sh.prefix = 0;
        sh.need = use_k ? (unsigned)top_k : (unsigned)kCand;
    }
    __syncthreads();
    float zsum = 0.0f;                                   // over the whole row, for top-p alone: sum of exp(z - zmax) in a fixed order
    select_round(row, V, temperature, 0u, 21, 11, sh, [&](int, float z, unsigned) { zsum += expf(z - zmax); });
    select_round(row, V, temperature, 0xFFE00000u, 10, 11, sh, [](int, float, unsigned) {});
    select_round(row, V, temperature, 0xFFFFFC00u, 0, 10, sh, [](int, float, unsigned) {});
    const unsigned kth = sh.prefix;
    // candidates: keys >= the k-th largest (top-k: equal values stay together), keys > the kCand-th largest (top-p alone)
    const unsigned low = use_k ? kth : kth + 1u;          // kth < 0xFFFFFFFF: it is the key of a finite or infinite float, never all ones
    unsigned mine = 0;
    for_each_element(row, V, [&](int, float x) { mine += sortable(x / temperature) >= low ? 1u : 0u; });
    unsigned total = 0;
    unsigned at = block_exclusive_scan(mine, sh, &total);
    if (total > (unsigned)kCand || total == 0) {          // more equal values than fit, or nothing finite: the slow way decides
        sample_row_by_bisection(row, V, temperature, top_k, top_p, seed, index, top, out + r, scratch, fscratch);
        return;
    }
    for_each_element(row, V, [&](int i, float x) {
        const unsigned key = sortable(x / temperature);
        if (key >= low) {
            sh.ckey[at] = key;
            sh.cidx[at] = i;
            ++at;
        }
    });
    __syncthreads();
    const int C = (int)total;
    unsigned keep_from = low;
    if (use_p) {
        float zc = 0.0f;
        for (int j = threadIdx.x; j < C; j += blockDim.x) zc += expf(unsortable(sh.ckey[j]) - zmax);
        zc = block_sum(zc, fscratch);
        float target;
        if (use_k) {
            target = top_p * zc;                          // the mass after top-k
        } else {
            const float zall = block_sum(zsum, fscratch);
            target = top_p * zall;
            if (!(zc >= target)) {                        // the gathered tokens hold less than top_p of the mass: the cut is below them
                sample_row_by_bisection(row, V, temperature, top_k, top_p, seed, index, top, out + r, scratch, fscratch);
                return;
            }
        }
        unsigned lo = low, hi = 0xFFFFFFFFu;
        while (lo < hi) {
            const unsigned mid = lo + ((hi - lo) >> 1);
            float mass = 0.0f;
            for (int j = threadIdx.x; j < C; j += blockDim.x) {
                const unsigned key = sh.ckey[j];
                if (key > mid) mass += expf(unsortable(key) - zmax);
            }
            mass = block_sum(mass, fscratch);
            if (mass < target) hi = mid; else lo = mid + 1;
        }
        if (lo > keep_from) keep_from = lo;
    }
    const unsigned long long key = splitmix64(seed ^ splitmix64(index));
    Best b{-INFINITY, 0x7fffffff};
    for (int j = threadIdx.x; j < C; j += blockDim.x) {
        const unsigned kj = sh.ckey[j];
        if (kj >= keep_from) {
            const int i = sh.cidx[j];
            const float v = unsortable(kj) + gumbel(key, i);
            if (v > b.v || (v == b.v && i < b.i)) b = Best{v, i};
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
    // few rows of a large vocabulary: rows with temperature alone are drawn over many CTAs by a second kernel
    const int chunked_plain = (R <= 64 && R <= kChunkRows && V >= 16384) ? 1 : 0;
    li_launch_pdl(sample_kernel, dim3(R), dim3(kThreads), 0, stream, logits, params, out, V, chunked_plain);
    if (int rc = li_check_launch("sample")) return rc;
    if (chunked_plain) {
        li_launch_pdl(sample_temperature_chunks_kernel, dim3(kDrawChunks, R), dim3(256), 0, stream, logits, params, out, V);
        return li_check_launch("sample (temperature, chunks)");
    }
    return 0;
}
