// li_paged_attention: attention of the step's tokens over the paged cache,
// chosen by dtype and batch shape.
//
//   float32                          -> general kernel (attention_generic.cu)
//   bfloat16, every item one token   -> split-context decode kernel (attention_decode.cu)
//   bfloat16, long portions          -> tcgen05 kernel (attention_tcgen05.cu): head_dim 64 or 128, a portion of
//                                       at least 64 tokens in the batch
//   bfloat16, other portions         -> tiled mma.sync kernel (attention_prefill.cu)
//   bfloat16, portions beside single tokens (`singles` != 0) -> two launches: the decode kernel takes the sequences of
//                                       one token (it finds them by q_start), the kernel for portions skips them.  A
//                                       single token as a portion of length one would occupy a whole tile of 64 or 128
//                                       query rows for each head and read its keys once per query head.
//   sizes those refuse               -> general kernel
#include "common.cuh"

int li_attention_generic(const void* qkv, void* out, const void* kcache, const void* vcache, int dtype, const int* block_table,
                         int max_blocks, const int* seq_of_token, const int* positions, int T, int nh, int nkv, int dh,
                         int page_size, int num_pages, float scale, int window, cudaStream_t stream);
bool li_attention_decode_accepts(int nh, int nkv, int dh, int page_size);
int li_attention_decode(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                        const int* ctx_lens, const int* old_lens, const int* q_start, int S, int nh, int nkv, int dh, int page_size, int num_pages,
                        float scale, int window, int max_ctx_len, int expected, cudaStream_t stream);
bool li_attention_prefill_accepts(int nh, int nkv, int dh, int page_size);
int li_attention_prefill(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                         const int* q_start, const int* ctx_lens, int T, int S, int nh, int nkv, int dh, int page_size,
                         int num_pages, float scale, int window, int max_q_len, int skip_single, cudaStream_t stream);

bool li_attention_tcgen05_accepts(const void* qkv, const void* kcache, const void* vcache, int nh, int nkv, int dh, int page_size);
int li_attention_tcgen05(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                         const int* q_start, const int* ctx_lens, int T, int S, int nh, int nkv, int dh, int page_size, int num_pages,
                         float scale, int window, int max_q_len, int skip_single, const int* units, int unit_slots, cudaStream_t stream);

static int validate(int T, int S, int nh, int nkv, int dh, int page_size, int window) {
    LI_REQUIRE(T >= 0 && S > 0, "attention: bad batch T=%d S=%d", T, S);
    LI_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "attention: %d heads are not a multiple of %d key/value heads", nh, nkv);
    LI_REQUIRE(dh > 0, "attention: bad head_dim %d", dh);
    LI_REQUIRE(page_size >= 1, "attention: bad page size %d", page_size);
    LI_REQUIRE(window >= 0, "attention: bad window %d", window);
    return 0;
}

// The kernels for a step of bfloat16 tokens that are not all single: portions on tcgen05 or mma.sync tiles; with
// `singles` the sequences of one token first, on the decode kernel.
static int attention_portions(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                              const int* q_start, const int* ctx_lens, int T, int S, int nh, int nkv, int dh, int page_size, int num_pages,
                              float scale, int window, int max_q_len, int max_ctx_len, const int* old_lens, int singles, const int* units,
                              int slots_portions, int slots_all, bool* done, cudaStream_t stream) {
    *done = false;
    const bool tc = max_q_len >= 64 && scale > 0.0f && li_attention_tcgen05_accepts(qkv, kcache, vcache, nh, nkv, dh, page_size);
    if (!tc && !li_attention_prefill_accepts(nh, nkv, dh, page_size)) return 0;
    const int split = (singles != 0 && max_q_len > 1 && li_attention_decode_accepts(nh, nkv, dh, page_size)) ? 1 : 0;
    // how many sequences the decode kernel will find: the count if it is known, else (a captured step, whose sequences are
    // rounded up to the next power of two) at least half of them
    const int expected = singles > 0 ? singles : (S + 1) / 2;
    if (split)
        if (int rc = li_attention_decode(qkv, out, kcache, vcache, block_table, max_blocks, ctx_lens, old_lens, q_start, S, nh, nkv, dh,
                                         page_size, num_pages, scale, window, max_ctx_len, expected, stream))
            return rc;
    *done = true;
    if (tc)
        return li_attention_tcgen05(qkv, out, kcache, vcache, block_table, max_blocks, q_start, ctx_lens, T, S, nh, nkv, dh, page_size,
                                    num_pages, scale, window, max_q_len, split, units, split ? slots_portions : slots_all, stream);
    return li_attention_prefill(qkv, out, kcache, vcache, block_table, max_blocks, q_start, ctx_lens, T, S, nh, nkv, dh, page_size,
                                num_pages, scale, window, max_q_len, split, stream);
}

// singles: how many sequences of the step have one token beside longer ones (0: none; negative: not known, there may be).
// units (may be null): the work list of the kernel for long portions (attention_tcgen05.cu), with the number of entries to
// launch when the single tokens are another kernel's and when they are not.
LI_EXPORT int li_paged_attention(const void* qkv, void* out, const void* kcache, const void* vcache, int dtype,
                                 const int* block_table, int max_blocks, const int* q_start, const int* ctx_lens,
                                 const int* seq_of_token, const int* positions, int T, int S, int nh, int nkv, int dh,
                                 int page_size, int num_pages, float scale, int window, int max_q_len, int max_ctx_len,
                                 const int* old_lens, int singles, const int* units, int slots_portions, int slots_all,
                                 cudaStream_t stream) {
    if (int rc = validate(T, S, nh, nkv, dh, page_size, window)) return rc;
    if (T == 0) return 0;
    if (dtype == LI_BF16) {
        if (max_q_len == 1 && T == S && li_attention_decode_accepts(nh, nkv, dh, page_size))
            return li_attention_decode(qkv, out, kcache, vcache, block_table, max_blocks, ctx_lens, old_lens, nullptr, S, nh, nkv, dh, page_size,
                                       num_pages, scale, window, max_ctx_len, S, stream);
        bool done = false;
        const int rc = attention_portions(qkv, out, kcache, vcache, block_table, max_blocks, q_start, ctx_lens, T, S, nh, nkv, dh, page_size,
                                          num_pages, scale, window, max_q_len, max_ctx_len, old_lens, singles, units, slots_portions, slots_all,
                                          &done, stream);
        if (rc || done) return rc;
    }
    return li_attention_generic(qkv, out, kcache, vcache, dtype, block_table, max_blocks, seq_of_token, positions, T, nh, nkv, dh,
                                page_size, num_pages, scale, window, stream);
}

// old_lens (may be null): how many keys of each sequence were in the cache before this step.  Null means all but the
// last one, which is so when every sequence of the step is a request of its own.  The decode kernel may read those
// keys while the kernel that writes the step's keys is still running.
//
// Force one implementation, for tests of each kernel alone: 0 general, 1 decode, 2 prefill (mma.sync), 3 prefill (tcgen05).
// With `singles` 2 and 3 leave the sequences of one token to the decode kernel, as li_paged_attention does.
LI_EXPORT int li_paged_attention_with(int which, const void* qkv, void* out, const void* kcache, const void* vcache, int dtype,
                                      const int* block_table, int max_blocks, const int* q_start, const int* ctx_lens,
                                      const int* seq_of_token, const int* positions, int T, int S, int nh, int nkv, int dh,
                                      int page_size, int num_pages, float scale, int window, int max_q_len, int max_ctx_len,
                                      const int* old_lens, int singles, const int* units, int slots_portions, int slots_all,
                                      cudaStream_t stream) {
    if (int rc = validate(T, S, nh, nkv, dh, page_size, window)) return rc;
    if (T == 0) return 0;
    if (which == 0)
        return li_attention_generic(qkv, out, kcache, vcache, dtype, block_table, max_blocks, seq_of_token, positions, T, nh, nkv,
                                    dh, page_size, num_pages, scale, window, stream);
    LI_REQUIRE(dtype == LI_BF16, "attention: implementation %d takes bfloat16 only", which);
    if (which == 1) {
        LI_REQUIRE(max_q_len == 1 && T == S, "attention: the decode kernel takes one token per sequence");
        LI_REQUIRE(li_attention_decode_accepts(nh, nkv, dh, page_size), "attention: the decode kernel refuses heads=%d/%d head_dim=%d page=%d", nh, nkv, dh, page_size);
        return li_attention_decode(qkv, out, kcache, vcache, block_table, max_blocks, ctx_lens, old_lens, nullptr, S, nh, nkv, dh, page_size, num_pages,
                                   scale, window, max_ctx_len, S, stream);
    }
    if (which == 2 || which == 3) {
        if (which == 2) {
            LI_REQUIRE(li_attention_prefill_accepts(nh, nkv, dh, page_size), "attention: the prefill kernel refuses heads=%d/%d head_dim=%d page=%d", nh, nkv, dh, page_size);
        } else {
            LI_REQUIRE(li_attention_tcgen05_accepts(qkv, kcache, vcache, nh, nkv, dh, page_size), "attention: the tcgen05 kernel refuses heads=%d/%d head_dim=%d page=%d", nh, nkv, dh, page_size);
        }
        const int split = (singles != 0 && max_q_len > 1 && li_attention_decode_accepts(nh, nkv, dh, page_size)) ? 1 : 0;
        if (split)
            if (int rc = li_attention_decode(qkv, out, kcache, vcache, block_table, max_blocks, ctx_lens, old_lens, q_start, S, nh, nkv, dh,
                                             page_size, num_pages, scale, window, max_ctx_len, singles > 0 ? singles : (S + 1) / 2, stream))
                return rc;
        if (which == 2)
            return li_attention_prefill(qkv, out, kcache, vcache, block_table, max_blocks, q_start, ctx_lens, T, S, nh, nkv, dh, page_size,
                                        num_pages, scale, window, max_q_len, split, stream);
        return li_attention_tcgen05(qkv, out, kcache, vcache, block_table, max_blocks, q_start, ctx_lens, T, S, nh, nkv, dh, page_size,
                                    num_pages, scale, window, max_q_len, split, units, split ? slots_portions : slots_all, stream);
    }
    return li_fail("attention: unknown implementation %d", which);
}
