// Prefill attention in bfloat16: portions of prompts (any length, with or
// without history in the cache) over the paged cache, causal, grouped-query.
// Single tokens in the same batch are portions of length one.
//
// Grid (tile of 64 tokens, query head, sequence); a CTA has 4 warps, each owns
// 16 consecutive tokens of the portion for one head and walks the visible keys
// in blocks of 16 with mma.sync m16n8k16 and an online softmax in float
// (attention_mma.cuh).  The keys and values of the portion itself are already
// in the cache (written by the rope kernel before), so history and new tokens
// are read the same way, through the block table.  The four warps of a CTA
// read the same keys at nearly the same time and share them through L1.
// Token i of a portion of n tokens in a context of c sits at position
// p = c - n + i and sees keys max(0, p - window + 1) .. p.
//
// Requires head_dim in {16, 32, ..., 128, 256} and page_size a multiple of 16.
#include "attention_mma.cuh"

namespace {

using namespace attn;

constexpr int kWarps = 4;
constexpr int kTile = kWarps * 16;

template <int DH>
__global__ void __launch_bounds__(kWarps * 32)
prefill_attention_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ out, const bf16* __restrict__ kcache,
                         const bf16* __restrict__ vcache, const int* __restrict__ block_table, int max_blocks,
                         const int* __restrict__ q_start, const int* __restrict__ ctx_lens, int nh, int nkv, int page_size,
                         int num_pages, float scale, int window) {
    const int s = blockIdx.z, h = blockIdx.y;
    const int tok0 = q_start[s], n = q_start[s + 1] - tok0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i0 = blockIdx.x * kTile + warp * 16;             // first token of this warp within the portion
    if (i0 >= n) return;
    const int g = lane >> 2, t = lane & 3;
    const int ctx = ctx_lens[s];
    const int kvh = h / (nh / nkv);
    const int row_elems = (nh + 2 * nkv) * DH;
    const int r_lo = i0 + g, r_hi = i0 + g + 8;                // this thread's two rows (tokens of the portion)
    const int p_first = ctx - n + i0;
    const int rows = min(16, n - i0);
    const int p_last = p_first + rows - 1;

    unsigned qa[DH / 16][4];
    load_q<DH>(qa, r_lo < n ? qkv + (size_t)(tok0 + r_lo) * row_elems + (size_t)h * DH : nullptr,
               r_hi < n ? qkv + (size_t)(tok0 + r_hi) * row_elems + (size_t)h * DH : nullptr, t);
    RowState<DH> st;
    st.init();
    int lo[2], hi[2];
    hi[0] = r_lo < n ? ctx - n + r_lo : -1;
    hi[1] = r_hi < n ? ctx - n + r_hi : -1;
    lo[0] = (window > 0 && hi[0] - window + 1 > 0) ? hi[0] - window + 1 : 0;
    lo[1] = (window > 0 && hi[1] - window + 1 > 0) ? hi[1] - window + 1 : 0;
    const int key_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;

    const int* bt = block_table + (size_t)s * max_blocks;
    auto page_of = [&](int key0) {
        int page = bt[key0 / page_size];
        return (page < 0 || page >= num_pages) ? 0 : page;
    };
    // keys of the next block are fetched while the current one is computed
    int key0 = (key_lo / 16) * 16;
    int page = page_of(key0);
    KFrag<DH> kcur;
    load_k<DH, false>(kcur, kcache + (((size_t)page * nkv + kvh) * page_size + key0 % page_size) * DH, g, t);
#pragma unroll 1
    for (; key0 <= p_last; key0 += 16) {
        VFrag<DH> vf;
        load_v<DH, false>(vf, vcache + ((size_t)page * nkv + kvh) * DH * page_size + key0 % page_size, page_size, g, t);
        KFrag<DH> knext;
        const int next0 = key0 + 16;
        if (next0 <= p_last) {
            page = page_of(next0);
            load_k<DH, false>(knext, kcache + (((size_t)page * nkv + kvh) * page_size + next0 % page_size) * DH, g, t);
        }
        compute16<DH>(st, qa, kcur, vf, key0, lo, hi, scale, t);
        kcur = knext;
    }
    const float l0 = quad_sum(st.l[0]), l1 = quad_sum(st.l[1]);
    const float inv0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, inv1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
    bf16* o_lo = out + (size_t)(tok0 + r_lo) * nh * DH + (size_t)h * DH;
    bf16* o_hi = out + (size_t)(tok0 + r_hi) * nh * DH + (size_t)h * DH;
#pragma unroll
    for (int j = 0; j < DH / 8; ++j) {
        const int col = j * 8 + 2 * t;
        if (r_lo < n) *reinterpret_cast<unsigned*>(o_lo + col) = pack_bf16(st.o[j][0] * inv0, st.o[j][1] * inv0);
        if (r_hi < n) *reinterpret_cast<unsigned*>(o_hi + col) = pack_bf16(st.o[j][2] * inv1, st.o[j][3] * inv1);
    }
}

template <int DH>
int launch(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
           const int* q_start, const int* ctx_lens, int S, int nh, int nkv, int page_size, int num_pages, float scale, int window,
           int max_q_len, cudaStream_t stream) {
    LI_REQUIRE(S <= 65535 && nh <= 65535, "attention (prefill): batch %d or heads %d too large for one launch", S, nh);
    dim3 grid(ceil_div(max_q_len > 0 ? max_q_len : 1, kTile), nh, S);
    prefill_attention_kernel<DH><<<grid, kWarps * 32, 0, stream>>>((const bf16*)qkv, (bf16*)out, (const bf16*)kcache,
                                                                   (const bf16*)vcache, block_table, max_blocks, q_start, ctx_lens,
                                                                   nh, nkv, page_size, num_pages, scale, window);
    return li_check_launch("attention (prefill)");
}

}  // namespace

bool li_attention_prefill_accepts(int nh, int nkv, int dh, int page_size) {
    const bool dh_ok = (dh % 16 == 0 && dh >= 16 && dh <= 128) || dh == 256;
    return dh_ok && nh % nkv == 0 && page_size % 16 == 0;
}

int li_attention_prefill(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                         const int* q_start, const int* ctx_lens, int T, int S, int nh, int nkv, int dh, int page_size,
                         int num_pages, float scale, int window, int max_q_len, cudaStream_t stream) {
    (void)T;
#define LI_CASE(D)                                                                                                                  \
    case D:                                                                                                                         \
        return launch<D>(qkv, out, kcache, vcache, block_table, max_blocks, q_start, ctx_lens, S, nh, nkv, page_size, num_pages, scale, \
                         window, max_q_len, stream);
    switch (dh) {
        LI_CASE(16) LI_CASE(32) LI_CASE(48) LI_CASE(64) LI_CASE(80) LI_CASE(96) LI_CASE(112) LI_CASE(128) LI_CASE(256)
        default:
            return li_fail("attention (prefill): head_dim %d is not supported by this kernel", dh);
    }
#undef LI_CASE
}
