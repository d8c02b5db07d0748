// The fused decode step (decode_step.h says what it is and why).  In short: one persistent CTA per multiprocessor,
// a producer warp that streams this CTA's share of every weight matrix through a ring of shared-memory stages with
// cp.async.bulk, eight consumer warps that multiply what has arrived and run the phases of every layer, grid-wide
// barriers between the phases.
//
// Work of a product is cut into units of 16 weight rows with the whole of k (for q|k|v the rows j..j+7 and
// j+head_dim/2..+7 of one head, so that a rotation pair ends up in one unit, as in gemv_bf16.cu); unit u of a phase
// belongs to CTA (u + rotation) mod CTAs, the rotation running on from phase to phase so that the bytes spread evenly.
// A unit goes through the ring in chunks of up to stage_k columns: 16 rows x chunk, each row a bulk copy of its own
// into a row of the stage (rows 64 bytes apart from a multiple of 128, which makes the 16-byte fragment loads free of
// bank conflicts).  The eight consumer warps split a chunk by groups of 32 columns, keep float accumulators in the
// mma layout, add them up through shared memory in warp order when the unit's last chunk is done and run the
// product's epilogue (gemv_epilogue.cuh).  The tokens' activations are read from global memory past L1 (they were
// written a moment ago by other multiprocessors), requested before the wait for the chunk they meet.
//
// Nothing here depends on how many sequences the step holds beyond the tile of 8 or 16 tokens, and every sum has a
// fixed order: a sequence's logits do not depend on the others in the step.
#include "attention_decode_unit.cuh"
#include "decode_step.h"
#include "gemv_epilogue.cuh"
#include "tcgen05.cuh"

namespace {

using tc::mbar_arrive;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::mbar_wait;
using tc::smem_u32;

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;              // the last warp is the producer
constexpr int kMaxStages = 16;
constexpr int kMaxStageK = 1024;
constexpr int kGranulesPerWarp = kMaxStageK / 32 / kConsumerWarps;      // groups of 32 columns a warp takes of one chunk
constexpr int kRowPad = 64;                            // bytes between the rows of a stage beyond the chunk itself
constexpr unsigned long long kWaitLimitNs = 1000000000ull;              // one second: far beyond any legitimate wait
constexpr int kSmemBudget = 227 * 1024;
constexpr int kHeaderBytes = 2048;

enum { kStatusBarrier = 21, kStatusStage = 22, kStatusProducer = 23 };
enum { kPhaseQkv = 0, kPhaseO = 1, kPhaseGateUp = 2, kPhaseDown = 3, kPhaseHead = 4 };

struct __align__(16) Header {
    unsigned long long full[kMaxStages];
    unsigned long long empty[kMaxStages];
    int is_last;
    int barrier_ok;
    volatile int abort;
    int pad;
    volatile int go[2];            // per unit of a split product: whether to go on (no abort seen), alternating
    unsigned issued;               // chunks the producer has issued so far (release / acquire)
    LiDecodeLayer layer;           // the running layer's description: one round trip to global memory per layer, not one per field
    float rs[16];                  // the tokens' factors of the norm before the running product
    float tile[16 * 16];           // new residual values of one unit, [token][row of the unit]
};
static_assert(sizeof(Header) <= kHeaderBytes, "header outgrew its place");

// One weight matrix as a phase sees it.
struct Matrix {
    const bf16* w;
    int N, K;
    int units;                     // of 16 rows
    int rope_dh;                   // > 0: rows of a unit are the two halves of rotation pairs of heads of this size
    int rot;                       // unit u belongs to CTA (u + rot) mod CTAs
};

__device__ __forceinline__ int chunk_of(int K, int stage_k) {
    const int n = (K + stage_k - 1) / stage_k;
    return (((K + n - 1) / n) + 31) & ~31;
}

__device__ __forceinline__ int unit_row(const Matrix& m, int u, int r) {
    if (m.rope_dh > 0) {
        const int tph = m.rope_dh >> 4;
        const int head = u / tph, jt = u - head * tph;
        return head * m.rope_dh + jt * 8 + (r & 7) + ((r >> 3) ? (m.rope_dh >> 1) : 0);
    }
    return u * 16 + r;
}

// first unit of this CTA in a matrix; its units are first, first + ctas, ...
__device__ __forceinline__ int first_unit(const Matrix& m, int cta, int ctas) {
    int f = (cta - m.rot) % ctas;
    return f < 0 ? f + ctas : f;
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint4 lds16(const unsigned char* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

struct Shape {
    int hidden, q_dim, qkv_dim, inter, vocab, dh;
};

__device__ __forceinline__ Matrix matrix_of(const LiDecodeStep& p, const LiDecodeLayer* L, int phase, int layer, int ctas) {
    const int H = p.hidden, QD = p.heads * p.head_dim, QKV = (p.heads + 2 * p.kv_heads) * p.head_dim, I = p.intermediate;
    const int u_qkv = QKV >> 4, u_o = (H + 15) >> 4, u_gu = (2 * I) >> 4, u_dn = (H + 15) >> 4;
    const long long per_layer = (long long)u_qkv + u_o + u_gu + u_dn;
    Matrix m;
    m.rope_dh = 0;
    long long before = per_layer * layer;
    if (phase == kPhaseQkv) {
        m.w = (const bf16*)L->w_qkv; m.N = QKV; m.K = H; m.units = u_qkv; m.rope_dh = p.head_dim;
    } else if (phase == kPhaseO) {
        m.w = (const bf16*)L->w_o; m.N = H; m.K = QD; m.units = u_o; before += u_qkv;
    } else if (phase == kPhaseGateUp) {
        m.w = (const bf16*)L->w_gate_up; m.N = 2 * I; m.K = H; m.units = u_gu; before += u_qkv + u_o;
    } else if (phase == kPhaseDown) {
        m.w = (const bf16*)L->w_down; m.N = H; m.K = I; m.units = u_dn; before += u_qkv + u_o + u_gu;
    } else {
        m.w = (const bf16*)p.lm_head; m.N = p.vocab; m.K = H; m.units = (p.vocab + 15) >> 4; before = per_layer * p.num_layers;
    }
    m.rot = (int)(before % ctas);
    return m;
}

// ---------------------------------------------------------------------------------------------------------
// producer: every chunk of every unit of this CTA, in the order the consumers take them
// ---------------------------------------------------------------------------------------------------------
__device__ void produce(const LiDecodeStep& p, Header& hd, unsigned char* ring, int stage_bytes, int row_stride, int lane, int* status) {
    const int cta = blockIdx.x, ctas = gridDim.x;
    const int S = p.stages;
    long long it = 0;
    bool ok = true;
    auto walk = [&](const Matrix& m) {
        const int kc = chunk_of(m.K, p.stage_k);
        for (int u = first_unit(m, cta, ctas); u < m.units && ok; u += ctas) {
            const int row = unit_row(m, u, lane & 15);
            const bool valid = lane < 16 && row < m.N;
            const unsigned nvalid = __popc(__ballot_sync(0xffffffffu, valid));
            for (int k0 = 0; k0 < m.K; k0 += kc) {
                const int s = (int)(it % S);
                if (it >= S) {
                    ok = mbar_wait(&hd.empty[s], (unsigned)(((it / S) & 1) ^ 1), kWaitLimitNs) && !hd.abort;
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                const unsigned bytes = (unsigned)(min(kc, m.K - k0) * 2);
                if (lane == 0) mbar_expect_tx(&hd.full[s], bytes * nvalid);
                __syncwarp();
                if (valid) bulk_load(ring + (size_t)s * stage_bytes + (size_t)(lane & 15) * row_stride, m.w + (size_t)row * m.K + k0, bytes, &hd.full[s]);
                ++it;
                // chunk it - 1 is on its way: from now on the stage's barrier is in the phase of that chunk (see wait_issued)
                if (lane == 0) asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(&hd.issued)), "r"((unsigned)it) : "memory");
            }
        }
    };
    for (int l = 0; l < p.num_layers && ok; ++l)
        for (int ph = kPhaseQkv; ph <= kPhaseDown && ok; ++ph) walk(matrix_of(p, p.layers + l, ph, l, ctas));
    if (ok && p.rows > 0) walk(matrix_of(p, nullptr, kPhaseHead, 0, ctas));
    if (!ok) {
        // something gave up: what this warp has in flight must land before the CTA's shared memory goes away
        if (lane == 0 && !hd.abort) atomicCAS(status, 0, kStatusProducer);
        hd.abort = 1;
        for (long long i = (it > S ? it - S : 0); i < it; ++i) mbar_wait(&hd.full[i % S], (unsigned)((i / S) & 1), kWaitLimitNs);
    }
}

// ---------------------------------------------------------------------------------------------------------
// consumers
// ---------------------------------------------------------------------------------------------------------
struct Consumer {
    Header* hd;
    unsigned char* ring;
    float* scratch;                // [2][8][NT * 128] sums of the warps (also the attention unit's scratch)
    unsigned char* xbuf;           // the running product's activations, [8 NT][x_cols] bfloat16, rows xstride bytes apart
    int xstride, x_cols;
    int stage_bytes, row_stride, S, stage_k;
    long long it;                  // chunks taken so far: the producer counts the same way
    unsigned barriers;             // grid-wide barriers passed so far
    int tid, warp, lane;
    int* status;
    bool ok;
    bool debug;
    bool watch;
};

// The kernel is deliberately cut into functions that are not inlined: a layer walks through all of them, twenty-eight
// times a step, and what matters is that their code together stays within the instruction cache (inlined into one body
// with every loop unrolled it came to 300 KB and a fifth of the instruction fetches missed).

// Grid-wide barrier among the consumers of all CTAs.  Thread 0 of each CTA arrives on the counter and waits, with a
// limit, until all have; the fences around it make what every thread of the CTA wrote before visible to every thread
// of every CTA after.
__device__ __noinline__ void grid_barrier(Consumer& c, unsigned* counter) {
    consumer_sync();
    c.barriers += 1;
    if (c.tid == 0) {
        if (c.debug) {
            c.status[1 + (blockIdx.x & 511)] = (int)c.barriers;          // a mark in host memory: the barrier this CTA is about to wait at
            if (blockIdx.x == 0 && c.barriers < 250) {                  // and when: nanoseconds, low 32 bits (exit time below)
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                c.status[1 + 500 + 2 * c.barriers] = (int)(unsigned)now;
            }
        }
        const unsigned target = c.barriers * gridDim.x;
        __threadfence();
        atomicAdd(counter, 1u);
        bool ok = false;
        unsigned long long t0 = 0;
#pragma unroll 1
        for (unsigned spin = 0;; ++spin) {
            if (ld_acquire(counter) >= target) {
                ok = true;
                break;
            }
            if ((spin & 63u) == 63u) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                else if (now - t0 > kWaitLimitNs) break;
                if (c.hd->abort) break;
            }
        }
        __threadfence();
        if (c.debug && blockIdx.x == 0 && c.barriers < 250) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            c.status[1 + 500 + 2 * c.barriers + 1] = (int)(unsigned)now;
        }
        if (!ok) {
            atomicCAS(c.status, 0, kStatusBarrier);
            c.hd->abort = 1;
        }
        c.hd->barrier_ok = ok ? 1 : 0;
    }
    consumer_sync();
    if (!c.hd->barrier_ok) c.ok = false;
}

// Debugging: a time stamp of CTA 0 for sub-step `id` of the layer that is being watched (ns, low 32 bits).
__device__ __noinline__ void stamp(const Consumer& c, int id) {
    if (c.debug && c.watch && blockIdx.x == 0 && c.tid == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        c.status[1 + 800 + (id & 63)] = (int)(unsigned)now;
    }
}

// The tokens' factor 1 / sqrt(mean(x^2) + eps) from the partial sums behind an activation: a lane's parts in ascending
// order, then the butterfly (the order of row_scale_of), with the loads of up to 128 parts in flight at once.
__device__ __forceinline__ float factor_of(const RowScale& rs, int tok, int lane) {
    float s;
    if (rs.nparts <= 128) {
        float pre[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int p = lane + 32 * q;
            pre[q] = p < rs.nparts ? __ldcg(rs.ssq + (size_t)tok * rs.nparts + p) : 0.0f;
        }
        s = ((pre[0] + pre[1]) + pre[2]) + pre[3];
    } else {
        s = 0.0f;
#pragma unroll 1
        for (int p = lane; p < rs.nparts; p += 32) s += __ldcg(rs.ssq + (size_t)tok * rs.nparts + p);
    }
    s = warp_sum(s);
    return 1.0f / sqrtf(s / rs.width + rs.eps);
}

// What a product needs of the step before its first unit: the factors of its `rows` rows into hd.rs (ssq == nullptr:
// none) and the rows' activations in the shared buffer (rows beyond `rows` as zeros); then a barrier among the consumers.
// Row r of the product is token row_tok[r] (nullptr: r).
template <int NT>
__device__ __noinline__ void begin_product(Consumer& c, const bf16* __restrict__ X, int K, int rows, const float* ssq, int nparts, int width,
                                           float eps, const int* row_tok) {
    const int per_row = K >> 3;                                           // 16-byte pieces of a row
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // eight loads in flight per thread before the first store: one round trip to L2 for up to 32 KB, not one per piece
    constexpr int B = 8;
#pragma unroll 1
    for (int i0 = c.tid; i0 < NT * 8 * per_row; i0 += B * kConsumers) {
        uint4 v[B];
#pragma unroll
        for (int q8 = 0; q8 < B; ++q8) {
            const int i = i0 + q8 * kConsumers;
            const int r = i / per_row, q = i - r * per_row;
            const bool in = i < NT * 8 * per_row && r < rows;
            const int tok = in ? (row_tok ? row_tok[r] : r) : 0;
            v[q8] = in ? __ldcg(reinterpret_cast<const uint4*>(X + (size_t)tok * K) + q) : zero;
        }
#pragma unroll
        for (int q8 = 0; q8 < B; ++q8) {
            const int i = i0 + q8 * kConsumers;
            const int r = i / per_row, q = i - r * per_row;
            if (i < NT * 8 * per_row) *reinterpret_cast<uint4*>(c.xbuf + (size_t)r * c.xstride + q * 16) = v[q8];
        }
    }
    if (ssq) {
        RowScale rs;
        rs.ssq = ssq;
        rs.nparts = nparts;
        rs.width = (float)width;
        rs.eps = eps;
#pragma unroll 1
        for (int r = c.warp; r < rows; r += kConsumerWarps) {
            const float f = factor_of(rs, row_tok ? row_tok[r] : r, c.lane);
            if (c.lane == 0) c.hd->rs[r] = f;
        }
    }
    consumer_sync();
}

// A warp that walks units of its own may be several rounds of the ring ahead of the producer, and a barrier's parity
// tells apart only neighbouring phases.  So before it waits for chunk `it` to land it waits (bounded) until the producer
// has issued that chunk: from then on the stage's barrier can only be in that chunk's phase.
__device__ __forceinline__ bool wait_issued(const Header& hd, long long it) {
    unsigned long long t0 = 0;
#pragma unroll 1
    for (unsigned spin = 0;; ++spin) {
        unsigned v;
        asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(&hd.issued)) : "memory");
        if ((int)(v - (unsigned)it) > 0) return true;
        __nanosleep(64);                                                  // the other warps of this multiprocessor have work to issue
        if ((spin & 63u) == 63u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs || hd.abort) return false;
        }
    }
}

// One unit of a product whose activations are in the shared buffer, by one warp alone: the unit's chunks (the ring's
// chunks it .. it + nch - 1) times the tokens, into this lane's accumulators (rows g and g + 8 of the unit, tokens
// 8 j + 2 t and + 1).  The CTA's units of such a product go to its warps in turn; no warp waits for another.
template <int NT>
__device__ __noinline__ void unit_mma(const Consumer& c, int K, int kc, int nch, long long it, float (&out)[NT][4]) {
    const int g = c.lane >> 2, t = c.lane & 3;
    float acc[NT][4], acc2[NT][4];                 // in registers: `out` is the caller's memory
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
        acc2[j][0] = acc2[j][1] = acc2[j][2] = acc2[j][3] = 0.0f;
    }
#pragma unroll 1
    for (int ci = 0; ci < nch; ++ci, ++it) {
        const int k0 = ci * kc, kn = min(kc, K - k0);
        const int s = (int)(it % c.S);
        stamp(c, 16 + 4 * ci);
        const bool issued = wait_issued(*c.hd, it);
        stamp(c, 17 + 4 * ci);
        if (!issued || !mbar_wait(&c.hd->full[s], (unsigned)((it / c.S) & 1), kWaitLimitNs)) {
            atomicCAS(c.status, 0, kStatusStage);
            c.hd->abort = 1;
        }
        stamp(c, 18 + 4 * ci);
        const unsigned char* a0 = c.ring + (size_t)s * c.stage_bytes + (size_t)g * c.row_stride + t * 16;
        const unsigned char* a1 = a0 + 8 * (size_t)c.row_stride;
        const unsigned char* xb = c.xbuf + (size_t)g * c.xstride + (size_t)(k0 + t * 8) * 2;
        // whole groups of 32 columns, two at a time into accumulators of their own (two chains of dependent mma instead of
        // one); then, if the chunk ends inside a group, that group with the lanes beyond its end masked to zero.  Every
        // load stays inside the stage's row and the buffer's row, whatever they hold there.
        const int whole = kn >> 5;
        int gr = 0;
#pragma unroll 2
        for (; gr + 2 <= whole; gr += 2) {
            const uint4 a = lds16(a0 + gr * 64), b = lds16(a1 + gr * 64);
            const uint4 a2 = lds16(a0 + gr * 64 + 64), b2 = lds16(a1 + gr * 64 + 64);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 x = lds16(xb + (size_t)j * 8 * c.xstride + gr * 64);
                const uint4 x2 = lds16(xb + (size_t)j * 8 * c.xstride + gr * 64 + 64);
                mma_bf16(acc[j], a.x, b.x, a.y, b.y, x.x, x.y);
                mma_bf16(acc2[j], a2.x, b2.x, a2.y, b2.y, x2.x, x2.y);
                mma_bf16(acc[j], a.z, b.z, a.w, b.w, x.z, x.w);
                mma_bf16(acc2[j], a2.z, b2.z, a2.w, b2.w, x2.z, x2.w);
            }
        }
#pragma unroll 1
        for (; gr * 32 < kn; ++gr) {                                     // one more whole group and / or the chunk's ragged end (the same for all lanes)
            const unsigned keep = (gr * 32 + t * 8 < kn) ? 0xffffffffu : 0u;
            uint4 a = lds16(a0 + gr * 64), b = lds16(a1 + gr * 64);
            a.x &= keep; a.y &= keep; a.z &= keep; a.w &= keep;
            b.x &= keep; b.y &= keep; b.z &= keep; b.w &= keep;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                uint4 x = lds16(xb + (size_t)j * 8 * c.xstride + gr * 64);
                x.x &= keep; x.y &= keep; x.z &= keep; x.w &= keep;
                mma_bf16(acc[j], a.x, b.x, a.y, b.y, x.x, x.y);
                mma_bf16(acc[j], a.z, b.z, a.w, b.w, x.z, x.w);
            }
        }
        __syncwarp();
        if (c.lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&c.hd->empty[s])), "r"(kConsumerWarps) : "memory");
        stamp(c, 19 + 4 * ci);
    }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) out[j][i] = acc[j][i] + acc2[j][i];
}

// The product into the residual stream whose activations do not fit the shared buffer (the down projection: a row of
// them is as wide as the feed-forward): x32 += act w^T; hprime = bfloat16(norm_weight * x32); ssq_out = sums of squares
// per unit.  The eight warps split every chunk by groups of 32 columns, read the tokens' side from global memory past
// L1, one chunk ahead of the one they multiply, and add up through shared memory in warp order at the end of a unit.
template <int NT>
__device__ __noinline__ void product_split_add(Consumer& c, const Matrix& m, const bf16* __restrict__ X, int M, float* x32,
                                               const float* norm_weight, bf16* hprime, float* ssq_out, int nparts) {
    const int cta = blockIdx.x, ctas = gridDim.x;
    const int g = c.lane >> 2, t = c.lane & 3;
    const int kc = chunk_of(m.K, c.stage_k);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const bf16* xr[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int tok = j * 8 + g;
        xr[j] = tok < M ? X + (size_t)tok * m.K : nullptr;
    }
    auto load_x = [&](uint4 (&bx)[NT][kGranulesPerWarp], int k0) {
        const int kn = min(kc, m.K - k0);
#pragma unroll
        for (int q = 0; q < kGranulesPerWarp; ++q) {
            const int kk = (c.warp + q * kConsumerWarps) * 32 + t * 8;
#pragma unroll
            for (int j = 0; j < NT; ++j) bx[j][q] = (kk < kn && xr[j]) ? __ldcg(reinterpret_cast<const uint4*>(xr[j] + k0 + kk)) : zero;
        }
    };
    AddScaled add;
    add.x32 = x32;
    add.norm_weight = norm_weight;
    add.hprime = hprime;
    add.ssq_out = ssq_out;
    int parity = 0;
#pragma unroll 1
    for (int u = first_unit(m, cta, ctas); u < m.units && c.ok; u += ctas) {
        float xpre[1];
        {
            const int e = c.tid, ln = e & 31, ji = e >> 5, i = ji & 3, j = ji >> 2;
            const int row = u * 16 + (ln >> 2) + ((i >> 1) << 3), tok = j * 8 + ((ln & 3) << 1) + (i & 1);
            xpre[0] = (e < NT * 128 && row < m.N && tok < M) ? __ldcg(x32 + (size_t)tok * m.N + row) : 0.0f;
        }
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
        uint4 bx[NT][kGranulesPerWarp], bn[NT][kGranulesPerWarp];
        load_x(bx, 0);
#pragma unroll 1
        for (int k0 = 0; k0 < m.K; k0 += kc) {
            const int s = (int)(c.it % c.S);
            const int kn = min(kc, m.K - k0);
            if (k0 + kc < m.K) load_x(bn, k0 + kc);                      // the next chunk's tokens while this one is multiplied
            if (!mbar_wait(&c.hd->full[s], (unsigned)((c.it / c.S) & 1), kWaitLimitNs)) {
                atomicCAS(c.status, 0, kStatusStage);
                c.hd->abort = 1;
            }
            const unsigned char* st = c.ring + (size_t)s * c.stage_bytes;
#pragma unroll
            for (int q = 0; q < kGranulesPerWarp; ++q) {
                const int k32 = (c.warp + q * kConsumerWarps) * 32, kk = k32 + t * 8;
                if (k32 < kn) {                                          // the same for the whole warp: mma.sync wants all its lanes
                    // a chunk that ends inside this group of 32 columns: the lanes beyond its end multiply zeros
                    const unsigned keep = kk < kn ? 0xffffffffu : 0u;
                    uint4 a = lds16(st + (size_t)g * c.row_stride + kk * 2), b = lds16(st + (size_t)(g + 8) * c.row_stride + kk * 2);
                    a.x &= keep; a.y &= keep; a.z &= keep; a.w &= keep;
                    b.x &= keep; b.y &= keep; b.z &= keep; b.w &= keep;
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        mma_bf16(acc[j], a.x, b.x, a.y, b.y, bx[j][q].x, bx[j][q].y);
                        mma_bf16(acc[j], a.z, b.z, a.w, b.w, bx[j][q].z, bx[j][q].w);
                    }
                }
            }
            __syncwarp();
            if (c.lane == 0) mbar_arrive(&c.hd->empty[s]);
            ++c.it;
#pragma unroll
            for (int q = 0; q < kGranulesPerWarp; ++q)
#pragma unroll
                for (int j = 0; j < NT; ++j) bx[j][q] = bn[j][q];
        }
        float* red = c.scratch + (size_t)parity * kConsumerWarps * NT * 128;
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[(size_t)c.warp * NT * 128 + (j * 4 + i) * 32 + c.lane] = acc[j][i];
        if (c.tid == 0) c.hd->go[parity] = c.hd->abort ? 0 : 1;          // one thread reads the flag: all must take the same way
        consumer_sync();
        if (!c.hd->go[parity]) {
            c.ok = false;
            break;
        }
        auto get = [&](int e) {
            float v = red[e];
#pragma unroll
            for (int w = 1; w < kConsumerWarps; ++w) v += red[(size_t)w * NT * 128 + e];
            return v;
        };
        store_add_scaled<NT>(get, nullptr, add, xpre, u, nparts, M, m.N, c.tid, kConsumers, c.hd->tile, [] { consumer_sync(); });
        parity ^= 1;
    }
    // chunks of units that were skipped after a failure are left to the producer's own bounded waits
}

// The same product by warps on whole units (its activations are in the shared buffer): this lane's rows g and g + 8 of
// the unit for its tokens; the squares are added over the unit's 16 rows by a butterfly over g.  The norm's weights of
// the two rows and the stream's old values are asked for before the unit's chunks.
template <int NT>
__device__ __noinline__ void product_warps_add(Consumer& c, const Matrix& m, int M, float* x32, const float* norm_weight, bf16* hprime,
                                               float* ssq_out, int nparts) {
    const int cta = blockIdx.x, ctas = gridDim.x;
    const int g = c.lane >> 2, t = c.lane & 3;
    const int kc = chunk_of(m.K, c.stage_k), nch = (m.K + kc - 1) / kc;
    const int first = first_unit(m, cta, ctas);
    const int mine = first < m.units ? (m.units - first + ctas - 1) / ctas : 0;
    const int H = m.N;
#pragma unroll 1
    for (int i = c.warp; i < mine; i += kConsumerWarps) {
        const int u = first + i * ctas;
        float nw[2], xold[NT][4];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int row = u * 16 + g + 8 * hh;
            nw[hh] = row < H ? norm_weight[row] : 0.0f;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const int tok = j * 8 + 2 * t + b;
                    xold[j][2 * hh + b] = (row < H && tok < M) ? __ldcg(x32 + (size_t)tok * H + row) : 0.0f;
                }
        }
        float acc[NT][4];
        unit_mma<NT>(c, m.K, kc, nch, c.it + (long long)i * nch, acc);
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const int tok = j * 8 + 2 * t + b;
                float sq = 0.0f;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int row = u * 16 + g + 8 * hh;
                    float x = 0.0f;
                    if (row < H && tok < M) {
                        x = xold[j][2 * hh + b] + acc[j][2 * hh + b];
                        __stcg(x32 + (size_t)tok * H + row, x);
                        hprime[(size_t)tok * H + row] = __float2bfloat16_rn(nw[hh] * x);
                    }
                    sq += x * x;
                }
                sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                sq += __shfl_xor_sync(0xffffffffu, sq, 8);
                sq += __shfl_xor_sync(0xffffffffu, sq, 16);
                if (g == 0 && tok < M) ssq_out[(size_t)tok * nparts + u] = sq;
            }
    }
    c.it += (long long)mine * nch;
}

// q|k|v by warps on whole units: the norm's factor, bias, rotary encoding (rotate-half: rows g and g + 8 of a unit are
// the two halves of pair 8 jt + g of one head, src/ops/rope/op.cpp:13-20) and the write of k and v into the paged cache
// (values transposed).  q and k are rounded to bfloat16 by the projection before they are rotated, as everywhere here.
template <int NT, int DH>
__device__ __noinline__ void product_warps_qkv(Consumer& c, const Matrix& m, const LiDecodeStep& p, const LiDecodeLayer* L) {
    const int cta = blockIdx.x, ctas = gridDim.x;
    const int g = c.lane >> 2, t = c.lane & 3;
    const int kc = chunk_of(m.K, c.stage_k), nch = (m.K + kc - 1) / kc;
    const int first = first_unit(m, cta, ctas);
    const int mine = first < m.units ? (m.units - first + ctas - 1) / ctas : 0;
    const int M = p.M, nh = p.heads, nkv = p.kv_heads, QKV = m.N;
    constexpr int tph = DH >> 4, half = DH >> 1;
    const int* slots = p.slot_mapping[L->group];
#pragma unroll 1
    for (int i = c.warp; i < mine; i += kConsumerWarps) {
        const int u = first + i * ctas;
        const int head = u / tph, jj = (u - head * tph) * 8 + g;
        const int r0 = head * DH + jj, r1 = r0 + half;
        const float b0 = L->b_qkv ? L->b_qkv[r0] : 0.0f, b1 = L->b_qkv ? L->b_qkv[r1] : 0.0f;
        const float den = head < nh + nkv ? L->rope_denom[jj] : 1.0f;
        int pos[NT][2], slot[NT][2];
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const int tok = j * 8 + 2 * t + b;
                pos[j][b] = tok < M ? p.positions[tok] : 0;
                slot[j][b] = (tok < M && head >= nh) ? slots[tok] : -1;
            }
        float acc[NT][4];
        unit_mma<NT>(c, m.K, kc, nch, c.it + (long long)i * nch, acc);
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const int tok = j * 8 + 2 * t + b;
                if (tok >= M) continue;
                float x0 = acc[j][b] * c.hd->rs[tok] + b0, x1 = acc[j][2 + b] * c.hd->rs[tok] + b1;
                float y0 = x0, y1 = x1;
                if (head < nh + nkv) {
                    float sn, cs;
                    sincosf((float)pos[j][b] / den, &sn, &cs);
                    x0 = __bfloat162float(__float2bfloat16_rn(x0));
                    x1 = __bfloat162float(__float2bfloat16_rn(x1));
                    y0 = x0 * cs - x1 * sn;
                    y1 = x1 * cs + x0 * sn;
                }
                if (head < nh) {
                    ((bf16*)p.qkv)[(size_t)tok * QKV + r0] = __float2bfloat16_rn(y0);
                    ((bf16*)p.qkv)[(size_t)tok * QKV + r1] = __float2bfloat16_rn(y1);
                } else if (L->write_cache) {
                    const int sl = slot[j][b];
                    const int page = sl / p.page_size, off = sl - page * p.page_size;
                    if (sl < 0 || page >= L->num_pages) continue;        // validated on the host; never write outside the cache
                    if (head < nh + nkv) {
                        bf16* dst = (bf16*)L->kcache + (((size_t)page * nkv + (head - nh)) * p.page_size + off) * DH;
                        dst[jj] = __float2bfloat16_rn(y0);
                        dst[jj + half] = __float2bfloat16_rn(y1);
                    } else {
                        bf16* dst = (bf16*)L->vcache + ((size_t)page * nkv + (head - nh - nkv)) * DH * p.page_size + off;
                        dst[(size_t)jj * p.page_size] = __float2bfloat16_rn(y0);
                        dst[(size_t)(jj + half) * p.page_size] = __float2bfloat16_rn(y1);
                    }
                }
            }
    }
    c.it += (long long)mine * nch;
}

// gate|up with the norm's factor and SwiGLU (rows g and g + 8 of a unit are gate and up of column 8 u + g), or, with
// `logits`, the plain product into float rows (the lm_head: rows of the logits are the wanted tokens).
template <int NT>
__device__ __noinline__ void product_warps_out(Consumer& c, const Matrix& m, int rows, bf16* act, int inter, float* logits) {
    const int cta = blockIdx.x, ctas = gridDim.x;
    const int g = c.lane >> 2, t = c.lane & 3;
    const int kc = chunk_of(m.K, c.stage_k), nch = (m.K + kc - 1) / kc;
    const int first = first_unit(m, cta, ctas);
    const int mine = first < m.units ? (m.units - first + ctas - 1) / ctas : 0;
#pragma unroll 1
    for (int i = c.warp; i < mine; i += kConsumerWarps) {
        const int u = first + i * ctas;
        float acc[NT][4];
        unit_mma<NT>(c, m.K, kc, nch, c.it + (long long)i * nch, acc);
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const int row = j * 8 + 2 * t + b;
                if (row >= rows) continue;
                const float f = c.hd->rs[row];
                if (logits) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int v = u * 16 + g + 8 * hh;
                        if (v < m.N) logits[(size_t)row * m.N + v] = acc[j][2 * hh + b] * f;
                    }
                } else {
                    const int col = u * 8 + g;
                    if (col < inter) act[(size_t)row * inter + col] = __float2bfloat16_rn(swiglu_of<bf16>(acc[j][b] * f, acc[j][2 + b] * f));
                }
            }
    }
    c.it += (long long)mine * nch;
}

// The barrier behind q|k|v, taken once, by whoever of the attention phase comes first (see consume).
struct Meet {
    Consumer* c;
    unsigned* counter;
    bool* met;
    __device__ __forceinline__ void operator()() const {
        if (!*met) grid_barrier(*c, counter);
        *met = true;
    }
};

template <int DH>
__device__ __noinline__ void attention_unit(Consumer& c, const LiDecodeStep& p, const LiDecodeLayer* L, int split, int kvh, int s, Meet meet) {
    attn_decode::decode_attention_unit<DH, 32>(split, kvh, s, c.tid, (const bf16*)p.qkv, (const bf16*)L->kcache, (const bf16*)L->vcache,
                                                p.block_table[L->group], p.max_blocks, p.ctx_lens, p.old_lens, nullptr, p.attn_part,
                                                p.attn_counters, (bf16*)p.attn, p.heads, p.kv_heads, p.page_size, L->num_pages, L->scale,
                                                L->window, p.splits, c.scratch, &c.hd->is_last, [] { consumer_sync(); }, meet);
    consumer_sync();                                                     // the scratch is free for the next unit
}

template <int NT, int DH>
__device__ void consume(const LiDecodeStep& p, Consumer& c) {
    const int cta = blockIdx.x, ctas = gridDim.x;
    const int M = p.M, H = p.hidden, nkv = p.kv_heads, I = p.intermediate;
    const int parts = (H + 15) >> 4;
    Header& hd = *c.hd;

    // ---- embedding: x32 = table[ids]; h_a = bfloat16(norm_first * x32); sums of squares per 16 columns ----
#pragma unroll 1
    for (int u = cta; u < parts; u += ctas) {
        const int tok = c.tid >> 4, col = u * 16 + (c.tid & 15);
        float x = 0.0f;
        if (tok < M && col < H) {
            int id = p.token_ids[tok];
            id = id < 0 ? 0 : (id >= p.vocab ? p.vocab - 1 : id);
            x = __bfloat162float(((const bf16*)p.embedding)[(size_t)id * H + col]);
            p.x32[(size_t)tok * H + col] = x;
            ((bf16*)p.h_a)[(size_t)tok * H + col] = __float2bfloat16_rn(p.norm_first[col] * x);
        }
        hd.tile[c.tid] = x;
        consumer_sync();
        if (c.tid < M) {
            float sq = 0.0f;
#pragma unroll
            for (int r = 0; r < 16; ++r) sq += hd.tile[c.tid * 16 + r] * hd.tile[c.tid * 16 + r];
            p.ssq_a[(size_t)c.tid * parts + u] = sq;
        }
        consumer_sync();
    }
    grid_barrier(c, p.barrier);

    float eps_in = p.eps_first;
#pragma unroll 1
    for (int l = 0; l < p.num_layers && c.ok; ++l) {
        if (c.tid < (int)(sizeof(LiDecodeLayer) / sizeof(int)))
            reinterpret_cast<int*>(&hd.layer)[c.tid] = reinterpret_cast<const int*>(p.layers + l)[c.tid];       // visible behind begin_product's barrier
        const LiDecodeLayer* L = &hd.layer;
        c.watch = l == 1;
        stamp(c, 0);
        // ---- q|k|v with the norm's factor, bias, rotary encoding and the cache write ----
        begin_product<NT>(c, (const bf16*)p.h_a, H, M, p.ssq_a, parts, H, eps_in, nullptr);
        stamp(c, 1);
        product_warps_qkv<NT, DH>(c, matrix_of(p, L, kPhaseQkv, l, ctas), p, L);
        stamp(c, 2);
        c.watch = false;
        // ---- attention: units of (sequence, kv head, 256 keys); the barrier behind q|k|v is taken inside the first unit,
        //      after its loads of keys and values that this step does not write have been issued ----
        {
            bool met = false;
            const Meet meet{&c, p.barrier, &met};
            int r = (cta - (l * 37) % ctas) % ctas;                      // spread the units' start over the CTAs from layer to layer
            if (r < 0) r += ctas;
            long long base = 0;
#pragma unroll 1
            for (int s = 0; s < M; ++s) {
                int first, last;
                attn_decode::split_range(p.ctx_lens[s], L->window, 256, &first, &last);
                const int nsp = last - first + 1;
                const long long n = (long long)nsp * nkv;
                long long j = base + (((long long)r - base) % ctas + ctas) % ctas;
#pragma unroll 1
                for (; j < base + n; j += ctas) {
                    const int local = (int)(j - base);
                    const int kvh = local / nsp;
                    attention_unit<DH>(c, p, L, first + local - kvh * nsp, kvh, s, meet);
                }
                base += n;
            }
            meet();
            if (!c.ok) break;
            stamp(c, 3);
            grid_barrier(c, p.barrier);
            stamp(c, 4);
        }
        // ---- output projection into the residual stream; h_b = bfloat16(norm_ffn * x32) with its sums of squares ----
        {
            const Matrix m = matrix_of(p, L, kPhaseO, l, ctas);
            begin_product<NT>(c, (const bf16*)p.attn, m.K, M, nullptr, 0, 0, 0.0f, nullptr);
            stamp(c, 5);
            product_warps_add<NT>(c, m, M, p.x32, L->norm_ffn, (bf16*)p.h_b, p.ssq_b, parts);
        }
        stamp(c, 6);
        grid_barrier(c, p.barrier);
        stamp(c, 7);
        // ---- gate|up with the norm's factor and SwiGLU ----
        begin_product<NT>(c, (const bf16*)p.h_b, H, M, p.ssq_b, parts, H, L->eps_ffn, nullptr);
        stamp(c, 8);
        product_warps_out<NT>(c, matrix_of(p, L, kPhaseGateUp, l, ctas), M, (bf16*)p.act, I, nullptr);
        stamp(c, 9);
        grid_barrier(c, p.barrier);
        stamp(c, 10);
        // ---- down projection into the residual stream; h_a = bfloat16(norm_next * x32) with its sums of squares ----
        {
            const Matrix m = matrix_of(p, L, kPhaseDown, l, ctas);
            if (c.x_cols >= m.K) {
                begin_product<NT>(c, (const bf16*)p.act, m.K, M, nullptr, 0, 0, 0.0f, nullptr);
                product_warps_add<NT>(c, m, M, p.x32, L->norm_next, (bf16*)p.h_a, p.ssq_a, parts);
            } else {
                product_split_add<NT>(c, m, (const bf16*)p.act, M, p.x32, L->norm_next, (bf16*)p.h_a, p.ssq_a, parts);
            }
        }
        stamp(c, 12);
        grid_barrier(c, p.barrier);
        stamp(c, 13);
        eps_in = L->eps_next;
    }
    // ---- the wanted rows' logits: the final norm is in h_a and its factor ----
    if (c.ok && p.rows > 0) {
        begin_product<NT>(c, (const bf16*)p.h_a, H, p.rows, p.ssq_a, parts, H, eps_in, p.logit_rows);
        product_warps_out<NT>(c, matrix_of(p, nullptr, kPhaseHead, 0, ctas), p.rows, nullptr, 0, p.logits);
    }
}

template <int NT, int DH>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const __grid_constant__ LiDecodeStep p, int* status, int scratch_bytes) {
    extern __shared__ __align__(128) unsigned char smem[];
    Header& hd = *reinterpret_cast<Header*>(smem);
    float* scratch = reinterpret_cast<float*>(smem + kHeaderBytes);
    const int xstride = p.x_cols > 0 ? p.x_cols * 2 + kRowPad : 0;
    const int xbytes = ((p.M <= 8 ? 8 : 16) * xstride + 127) & ~127;
    unsigned char* xbuf = smem + kHeaderBytes + scratch_bytes;
    unsigned char* ring = xbuf + xbytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_stride = p.stage_k * 2 + kRowPad;
    const int stage_bytes = 16 * row_stride;
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&hd.full[s], 1);
            mbar_init(&hd.empty[s], kConsumerWarps);
        }
        hd.abort = 0;
        hd.issued = 0;
        hd.barrier_ok = 1;
        hd.is_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == kConsumerWarps) {
        produce(p, hd, ring, stage_bytes, row_stride, lane, status);
        return;
    }
    Consumer c;
    c.hd = &hd;
    c.ring = ring;
    c.scratch = scratch;
    c.xbuf = xbuf;
    c.xstride = xstride;
    c.x_cols = p.x_cols;
    c.stage_bytes = stage_bytes;
    c.row_stride = row_stride;
    c.S = p.stages;
    c.stage_k = p.stage_k;
    c.it = 0;
    c.barriers = 0;
    c.tid = threadIdx.x;
    c.warp = warp;
    c.lane = lane;
    c.status = status;
    c.ok = true;
    c.debug = (p.balance & 2) != 0;
    c.watch = false;
    consume<NT, DH>(p, c);
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
int scratch_bytes_for(int M, int heads, int kv_heads, int head_dim, int splits) {
    const int NT = M <= 8 ? 1 : 2, G = heads / kv_heads;
    size_t floats = (size_t)2 * kConsumerWarps * NT * 128;                           // two buffers of the warps' sums
    const size_t attn = (size_t)2 * kConsumerWarps * 16 + (size_t)kConsumerWarps * G * head_dim;   // the attention unit's merge of its warps
    const size_t merge = (size_t)G * (splits + 1);
    if (attn > floats) floats = attn;
    if (merge > floats) floats = merge;
    return (int)((floats * sizeof(float) + 127) / 128 * 128);
}

int xbytes_for(int M, int x_cols) { return x_cols > 0 ? (((M <= 8 ? 8 : 16) * (x_cols * 2 + kRowPad)) + 127) & ~127 : 0; }

// The ring beside `scratch` bytes and the buffer for activations of x_cols columns.
bool plan_for(int M, int scratch, int x_cols, int* stage_k, int* stages) {
    const int ring = kSmemBudget - kHeaderBytes - scratch - xbytes_for(M, x_cols);
    for (int k : {1024, 768, 512, 256}) {
        const int stage = 16 * (k * 2 + kRowPad);
        int n = ring / stage;
        if (n > kMaxStages) n = kMaxStages;
        if (n >= 4) {
            *stage_k = k;
            *stages = n;
            return true;
        }
    }
    return false;
}

struct DeviceInfo {
    int sms = 0;
    bool cooperative = false;
};
DeviceInfo g_info[16];

template <int NT, int DH>
int launch(const LiDecodeStep& p, cudaStream_t stream) {
    tc::EncodeTiledFn encode = nullptr;
    int *err_host = nullptr, *err_dev = nullptr;
    if (int rc = tc::setup(&encode, &err_host, &err_dev)) return rc;
    if (*err_host != 0)
        return li_fail("decode step: an earlier launch gave up waiting (status %d); the results since then are invalid", *err_host);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return li_fail("decode step: cudaGetDevice: %s", cudaGetErrorString(e));
    LI_REQUIRE(dev >= 0 && dev < 16, "decode step: device index %d out of range", dev);
    const int scratch = scratch_bytes_for(p.M, p.heads, p.kv_heads, p.head_dim, p.splits);
    const int row_stride = p.stage_k * 2 + kRowPad;
    const size_t smem = (size_t)kHeaderBytes + scratch + xbytes_for(p.M, p.x_cols) + (size_t)p.stages * 16 * row_stride;
    LI_REQUIRE(smem <= (size_t)kSmemBudget, "decode step: %zu bytes of shared memory do not fit (stage_k %d, %d stages)", smem, p.stage_k, p.stages);
    static bool raised = false;
    if (!raised) {
        e = cudaFuncSetAttribute(decode_step_kernel<NT, DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
        if (e != cudaSuccess) return li_fail("decode step: cannot raise shared memory: %s", cudaGetErrorString(e));
        raised = true;
    }
    DeviceInfo& info = g_info[dev];
    if (info.sms == 0) {
        int sms = 0, coop = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
        info.sms = sms;
        info.cooperative = coop != 0;
    }
    LI_REQUIRE(info.cooperative && info.sms > 0, "decode step: the device does not support cooperative launches");
    static size_t fits = 0;                            // the shared-memory size that was found to fit
    if (fits != smem) {
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel<NT, DH>, kThreads, smem);
        if (e != cudaSuccess || per_sm < 1) return li_fail("decode step: a CTA of %d threads and %zu bytes does not fit a multiprocessor", kThreads, smem);
        fits = smem;
    }
    e = cudaMemsetAsync(p.barrier, 0, sizeof(unsigned), stream);
    if (e != cudaSuccess) return li_fail("decode step: clearing the barrier: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(info.sms);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, decode_step_kernel<NT, DH>, p, err_dev, scratch);
    if (e != cudaSuccess) return li_fail("decode step: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("decode step");
}

}  // namespace

LI_EXPORT int li_decode_step_accepts(int M, int hidden, int heads, int kv_heads, int head_dim, int intermediate, int vocab, int page_size) {
    LI_REQUIRE(M >= 1 && M <= 16, "decode step: %d tokens (the fused step takes 1 to 16)", M);
    LI_REQUIRE(head_dim == 64 || head_dim == 128, "decode step: head_dim %d (the fused step is built for 64 and 128)", head_dim);
    LI_REQUIRE(kv_heads >= 1 && heads % kv_heads == 0 && heads / kv_heads <= 16, "decode step: %d heads on %d key/value heads", heads, kv_heads);
    LI_REQUIRE(hidden >= 16 && hidden % 16 == 0, "decode step: hidden size %d must be a multiple of 16", hidden);
    LI_REQUIRE(intermediate >= 8 && intermediate % 8 == 0, "decode step: intermediate size %d must be a multiple of 8", intermediate);
    LI_REQUIRE(vocab >= 1 && page_size >= 16 && page_size % 16 == 0, "decode step: vocabulary %d, page size %d", vocab, page_size);
    return 0;
}

LI_EXPORT int li_decode_step_plan(int M, int hidden, int heads, int kv_heads, int head_dim, int splits, int* stage_k, int* stages, int* x_cols,
                                  int* scratch_bytes) {
    LI_REQUIRE(M >= 1 && M <= 16 && kv_heads >= 1 && heads % kv_heads == 0 && splits >= 1 && hidden >= 16, "decode step plan: bad sizes");
    const int scratch = scratch_bytes_for(M, heads, kv_heads, head_dim, splits);
    *scratch_bytes = scratch;
    const int widest = hidden > heads * head_dim ? hidden : heads * head_dim;       // q|k|v, gate|up and the head read rows of hidden, o of heads * head_dim
    *x_cols = (widest + 63) & ~63;
    if (!plan_for(M, scratch, *x_cols, stage_k, stages))
        return li_fail("decode step: no ring of weight stages fits beside %d bytes of scratch and a buffer of %d tokens x %d columns (%d heads on %d key/value heads of %d)",
                       scratch, M <= 8 ? 8 : 16, *x_cols, heads, kv_heads, head_dim);
    return 0;
}

LI_EXPORT int li_decode_step(const LiDecodeStep* step, cudaStream_t stream) {
    LI_REQUIRE(step != nullptr && step->layers != nullptr && step->num_layers >= 1, "decode step: no layers");
    const LiDecodeStep& p = *step;
    if (int rc = li_decode_step_accepts(p.M, p.hidden, p.heads, p.kv_heads, p.head_dim, p.intermediate, p.vocab, p.page_size)) return rc;
    LI_REQUIRE(p.rows >= 0 && p.rows <= p.M, "decode step: %d logit rows for %d tokens", p.rows, p.M);
    LI_REQUIRE(p.stage_k >= 32 && p.stage_k <= kMaxStageK && p.stage_k % 64 == 0 && p.stages >= 2 && p.stages <= kMaxStages,
               "decode step: a ring of %d stages of %d columns", p.stages, p.stage_k);
    LI_REQUIRE(p.splits >= 1 && p.max_blocks >= 1, "decode step: %d splits, %d blocks", p.splits, p.max_blocks);
    LI_REQUIRE(p.x_cols % 64 == 0 && p.x_cols >= p.hidden && p.x_cols >= p.heads * p.head_dim,
               "decode step: the shared buffer of %d columns does not hold a row of activations (hidden %d, %d heads of %d)", p.x_cols, p.hidden,
               p.heads, p.head_dim);
    LI_REQUIRE(p.x32 && p.h_a && p.h_b && p.ssq_a && p.ssq_b && p.qkv && p.attn && p.act && p.attn_part && p.attn_counters && p.barrier,
               "decode step: missing scratch");
    LI_REQUIRE(p.embedding && p.norm_first && p.token_ids && p.positions && p.ctx_lens && (p.rows == 0 || (p.lm_head && p.logits && p.logit_rows)),
               "decode step: missing operand");
    const bool one = p.M <= 8;
    if (p.head_dim == 128) return one ? launch<1, 128>(p, stream) : launch<2, 128>(p, stream);
    return one ? launch<1, 64>(p, stream) : launch<2, 64>(p, stream);
}
