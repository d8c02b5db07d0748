// Decode attention in bfloat16: one new token per sequence over its paged
// cache, grouped-query.
//
// Two kernels share one inner step.  Few sequences: grid (split, kv head,
// sequence); a CTA of 8 warps covers 256 keys at fixed absolute positions
// [256 s, 256 s + 256), each warp 32 of them (all its loads are in flight at
// once: one round trip to memory); with more sequences longer ranges, each warp
// walking every 8th block of its CTA's range, so that about one CTA per
// multiprocessor is left.  Many sequences (a CTA per pair fills the GPU):
// one CTA per (sequence, kv head) whose warps walk every 8th block of 32 keys;
// nothing to merge across CTAs.  Either way a warp works for all query heads of
// one key/value head at once (they share every K and V byte read; heads are the
// 16 rows of a tensor-core tile).  Per block a warp computes S = Q K^T and
// O += P V with mma.sync m16n8k16 (bfloat16 in, float accumulate), softmax
// online in float as in LitInfer's kernel (src/ops/paged_attention/op.cpp:194-234).
// All operands go from global memory straight into fragment registers with
// 16-byte loads (8-byte loads and blocks of 16 keys for head_dim 256, where
// registers are short):
//   * the sum over head_dim does not depend on its order, so the 8 consecutive
//     elements a thread loads from a q row and from a key row are used as the
//     element pairs the fragment layout asks for in two k-steps, the same way
//     on both sides;
//   * values are cached transposed, [page][kv_head][head_dim][slot], so that for
//     one output column the 8 consecutive keys a thread needs are contiguous;
//     the score tiles are computed with their key columns permuted to match.
// Warps are merged through shared memory, CTAs through a float workspace by the
// CTA that finishes last (a counter per sequence and kv head), both in fixed
// order: which keys a warp or a CTA takes depends on absolute key positions
// only, so a sequence's result does not depend on the batch it is in, as long
// as the contexts are cut the same way (how long a CTA's range is depends on the
// number of sequences and on the longest context of the step).
// Window: keys below p - window + 1 are masked, blocks wholly below it skipped.
//
// Requires head_dim in {16, 32, ..., 128, 256}, at most 16 query heads per
// key/value head, page_size a multiple of 16.
#define LI_PDL_KIND 4
#include "attention_decode_unit.cuh"

namespace {


struct Workspace {
    float* buf = nullptr;
    size_t floats = 0;
    unsigned* counters = nullptr;
};
constexpr size_t kCounters = 1u << 20;
Workspace g_ws[16];

using namespace attn;
using namespace attn_decode;

template <int DH, int KB, bool kCut>
__global__ void __launch_bounds__(kWarps * 32, 1)
decode_attention_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ ctx_lens,
                        const int* __restrict__ old_lens, const int* __restrict__ q_start, float* __restrict__ part,
                        unsigned* __restrict__ counters, bf16* __restrict__ out, int nh, int nkv, int page_size, int num_pages,
                        float scale, int window, int nsplit, int want) {
    extern __shared__ float sm[];
    __shared__ int is_last;
    pdl_launch_dependents();
    decode_attention_unit<DH, KB, kCut>((int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, (int)threadIdx.x, qkv, kcache, vcache, block_table, max_blocks,
                                  ctx_lens, old_lens, q_start, part, counters, out, nh, nkv, page_size, num_pages, scale, window, nsplit, sm,
                                  &is_last, [] { __syncthreads(); }, [] { pdl_wait(); }, want);
}

// Many sequences at once: with one CTA per (sequence, kv head) the GPU is already full, and splitting the
// context over CTAs would only add partial results to write, merge and wait for.  Each of the CTA's warps
// walks every WARPS-th block of 16 keys with a running softmax; the warps are merged through shared memory in
// warp order at the end.  The assignment of blocks to warps depends on the sequence alone.
template <int DH, int WARPS, int KB>
__global__ void __launch_bounds__(WARPS * 32, 1)
decode_attention_whole_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                              const int* __restrict__ block_table, int max_blocks, const int* __restrict__ ctx_lens,
                              const int* __restrict__ q_start, bf16* __restrict__ out, int nh, int nkv, int page_size, int num_pages,
                              float scale, int window) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int kvh = blockIdx.x, s = blockIdx.y;
    const int tok = q_start ? q_start[s] : s;          // as in the kernel above
    if (q_start && q_start[s + 1] - tok != 1) return;
    const int ctx = ctx_lens[s];
    const int p = ctx - 1;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int G = nh / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const bf16* qrow = qkv + (size_t)tok * (nh + 2 * nkv) * DH + (size_t)kvh * G * DH;
    unsigned qa[DH / 16][4];
    const bf16* q_lo = g < G ? qrow + (size_t)g * DH : nullptr;
    const bf16* q_hi = g + 8 < G ? qrow + (size_t)(g + 8) * DH : nullptr;
    if constexpr (KB == 16) load_q<DH>(qa, q_lo, q_hi, t);
    else load_q32<DH>(qa, q_lo, q_hi, t);
    RowState<DH> st;
    st.init();
    const int lo2[2] = {lo, lo}, hi2[2] = {p, p};
    const int* bt = block_table + (size_t)s * max_blocks;
    const int b_first = lo / KB, b_last = p / KB;
#pragma unroll 1
    for (int b = b_first + warp; b <= b_last; b += WARPS)
        block_step<DH, KB>(st, qa, kcache, vcache, bt, b * KB, kvh, nkv, page_size, num_pages, lo2, hi2, scale, g, t);
    const float m0 = st.m[0], m1 = st.m[1];
    const float l0 = quad_sum(st.l[0]), l1 = quad_sum(st.l[1]);
    float* sm_m = sm;
    float* sm_l = sm + WARPS * 16;
    float* sm_o = sm + 2 * WARPS * 16;
    if (t == 0) {
        sm_m[warp * 16 + g] = m0; sm_m[warp * 16 + g + 8] = m1;
        sm_l[warp * 16 + g] = l0; sm_l[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int j = 0; j < DH / 8; ++j) {
        const int col = j * 8 + 2 * t;
        if (g < G) {
            sm_o[((size_t)warp * G + g) * DH + col] = st.o[j][0];
            sm_o[((size_t)warp * G + g) * DH + col + 1] = st.o[j][1];
        }
        if (g + 8 < G) {
            sm_o[((size_t)warp * G + g + 8) * DH + col] = st.o[j][2];
            sm_o[((size_t)warp * G + g + 8) * DH + col + 1] = st.o[j][3];
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < G * DH; e += WARPS * 32) {
        const int r = e / DH, d = e - r * DH;
        float M = sm_m[r];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
        float O = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = (sm_m[w * 16 + r] == -INFINITY) ? 0.0f : expf(sm_m[w * 16 + r] - M);
            O += sm_o[((size_t)w * G + r) * DH + d] * f;
            L += sm_l[w * 16 + r] * f;
        }
        out[((size_t)tok * nh + kvh * G + r) * DH + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
    }
}

int ensure_workspace(size_t floats, float** buf, unsigned** counters) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return li_fail("attention (decode): cudaGetDevice: %s", cudaGetErrorString(e));
    LI_REQUIRE(dev >= 0 && dev < 16, "attention (decode): device index %d out of range", dev);
    Workspace& w = g_ws[dev];
    if (w.floats < floats) {
        // grows on demand; the first call of a given size must come before stream capture.  The buffer that was
        // outgrown is kept until the process ends: a captured graph may still hold its address.
        size_t want = floats < (8u << 20) ? (8u << 20) : floats + floats / 2;
        float* nb = nullptr;
        e = cudaMalloc(&nb, want * sizeof(float));
        if (e != cudaSuccess) {
            return li_fail("attention (decode): cannot allocate %zu bytes of workspace: %s (a first call of this size inside a stream capture cannot allocate)",
                           want * sizeof(float), cudaGetErrorString(e));
        }
        w.buf = nb;
        w.floats = want;
    }
    if (!w.counters) {
        e = cudaMalloc(&w.counters, kCounters * sizeof(unsigned));
        if (e == cudaSuccess) e = cudaMemset(w.counters, 0, kCounters * sizeof(unsigned));
        if (e != cudaSuccess) return li_fail("attention (decode): cannot allocate the split counters: %s", cudaGetErrorString(e));
    }
    *buf = w.buf;
    *counters = w.counters;
    return 0;
}

template <int DH>
int launch(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
           const int* ctx_lens, const int* old_lens, const int* q_start, int S, int nh, int nkv, int page_size, int num_pages, float scale,
           int window, int max_ctx_len, int expected, cudaStream_t stream) {
    const int G = nh / nkv;
    LI_REQUIRE(S <= 65535 && nkv <= 65535, "attention (decode): batch %d or kv heads %d too large for one launch", S, nkv);
    // `expected`: how many of the S sequences are this kernel's (a step may hold portions beside them, and a captured step
    // is padded with empty sequences): that count, not S, says how the contexts are best cut.  A CTA takes kSplit keys of
    // one (sequence, kv head): a block of 32 per warp and round.  With few pairs one round, so that every load of a CTA is
    // in flight at once and the splits of all pairs fill the GPU (batch 8: 16 pairs x 9 splits of 256 keys).  With more
    // pairs that many CTAs run in several waves, each paying its start, its merge and its exit, so the units get longer:
    // every sequence's context is cut into as many units as leave about one CTA per multiprocessor, of as many rounds as
    // that takes; with one unit per pair, the kernel without a merge takes it.
    constexpr int KBS = DH <= 128 ? 32 : 16;
    const long long pairs = (long long)(expected > 0 && expected < S ? expected : S) * nkv;
    static const int sms = [] {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        return n;
    }();
    const int blocks = ceil_div(max_ctx_len > 0 ? max_ctx_len : 1, KBS * kWarps);          // units of one round that the longest context can have
    const int want = (int)(pairs >= sms ? 1 : sms / pairs);                              // units per pair that fill the GPU once
    if (want == 1 && blocks > 1) {
        // one CTA per (sequence, kv head) fills the GPU: no split of the context
        constexpr int W = 8, KB = KBS;
        const size_t wsmem = (2 * W * 16 + (size_t)W * G * DH) * sizeof(float);
        if (wsmem <= 200 * 1024) {
            static bool raised = false;
            if (!raised && wsmem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(decode_attention_whole_kernel<DH, W, KB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
                if (e != cudaSuccess) return li_fail("attention (decode): cannot raise shared memory: %s", cudaGetErrorString(e));
                raised = true;
            }
            li_launch_pdl(decode_attention_whole_kernel<DH, W, KB>, dim3(nkv, S), dim3(W * 32), wsmem, stream, (const bf16*)qkv, (const bf16*)kcache,
                          (const bf16*)vcache, block_table, max_blocks, ctx_lens, q_start, (bf16*)out, nh, nkv, page_size, num_pages, scale, window);
            return li_check_launch("attention (decode, whole context)");
        }
    }
    // Units of one round if every context up to the longest has no more of them than `want`.  Else every sequence's own
    // context is cut into at most `want` units (attention_decode_unit.cuh): a launch whose longest context is only a bound
    // (a captured step) still gives every sequence units of equal length.  Measured (1.5B shape, contexts of 2,048-2,185,
    // ms a step; units per sequence 2 / 3 / 4 / 6 / 9 = one round): 8 sequences 1.66 / 1.48 / 1.49 / 1.40 / 1.31;
    // 16 sequences 1.75 / 1.58 / 1.59 / 1.63 / 1.64; 32 sequences 1.87 / 2.02 / 2.02 / 2.02 / - (a whole context per CTA
    // 2.04): multiprocessors // pairs, that is 9, 4 and 2, is the best or next to it each time.
    const bool cut = want < blocks;
    const int nsplit = cut ? want : blocks;
    float* part = nullptr;
    unsigned* counters = nullptr;
    if (int rc = ensure_workspace((size_t)S * nh * nsplit * (DH + 2), &part, &counters)) return rc;
    LI_REQUIRE((size_t)S * nkv <= kCounters, "attention (decode): batch %d x %d kv heads exceeds the split counters", S, nkv);
    size_t smem_floats = 2 * kWarps * 16 + (size_t)kWarps * G * DH;
    if (smem_floats < (size_t)G * (nsplit + 1)) smem_floats = (size_t)G * (nsplit + 1);      // the final merge reuses the buffer
    const size_t smem = smem_floats * sizeof(float);
    static bool attr_set = false;
    if (!attr_set && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<DH, KBS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_attention_kernel<DH, KBS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return li_fail("attention (decode): cannot raise shared memory: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    LI_REQUIRE(smem <= 200 * 1024, "attention (decode): shared memory %zu too large", smem);
    LI_REQUIRE(S <= 65535 && nkv <= 65535, "attention (decode): batch %d or kv heads %d too large for one launch", S, nkv);
    dim3 grid(nsplit, nkv, S);
    if (cut)
        li_launch_pdl(decode_attention_kernel<DH, KBS, true>, dim3(grid), dim3(kWarps * 32), smem, stream, (const bf16*)qkv, (const bf16*)kcache,
                      (const bf16*)vcache, block_table, max_blocks, ctx_lens, old_lens, q_start, part, counters, (bf16*)out, nh, nkv, page_size,
                      num_pages, scale, window, nsplit, want);
    else
        li_launch_pdl(decode_attention_kernel<DH, KBS, false>, dim3(grid), dim3(kWarps * 32), smem, stream, (const bf16*)qkv, (const bf16*)kcache,
                      (const bf16*)vcache, block_table, max_blocks, ctx_lens, old_lens, q_start, part, counters, (bf16*)out, nh, nkv, page_size,
                      num_pages, scale, window, nsplit, 0);
    return li_check_launch("attention (decode)");
}

}  // namespace

bool li_attention_decode_accepts(int nh, int nkv, int dh, int page_size) {
    const bool dh_ok = (dh % 16 == 0 && dh >= 16 && dh <= 128) || dh == 256;
    return dh_ok && nh % nkv == 0 && nh / nkv <= 16 && page_size % 16 == 0;
}

int li_attention_decode(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                        const int* ctx_lens, const int* old_lens, const int* q_start, int S, int nh, int nkv, int dh, int page_size, int num_pages,
                        float scale, int window, int max_ctx_len, int expected, cudaStream_t stream) {
#define LI_CASE(D)                                                                                                             \
    case D:                                                                                                                    \
        return launch<D>(qkv, out, kcache, vcache, block_table, max_blocks, ctx_lens, old_lens, q_start, S, nh, nkv, page_size, num_pages, scale, \
                         window, max_ctx_len, expected, stream);
    switch (dh) {
        LI_CASE(16) LI_CASE(32) LI_CASE(48) LI_CASE(64) LI_CASE(80) LI_CASE(96) LI_CASE(112) LI_CASE(128) LI_CASE(256)
        default:
            return li_fail("attention (decode): head_dim %d is not supported by this kernel", dh);
    }
#undef LI_CASE
}
