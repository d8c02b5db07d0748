/* The C interface of the kernel library (liblitinfer_b200_*.so), as litinfer_b200/kernels.py calls it through ctypes.
 *
 * All pointers are device pointers unless said otherwise; tensors are row-major and contiguous; dtype 0 is float32,
 * 1 bfloat16; every launch goes to `stream`.  A function returns 0, or non-zero with the text in li_last_error(), and
 * launches nothing in that case: sizes a kernel cannot take are refused, never computed wrongly.
 * LitInfer's counterpart is include/llaisys/*.h (ops.h, models/qwen2.h): one C entry per operator.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- api.cu ---- */
/* The message of the last call that returned non-zero (a static buffer; copy it before the next call). */
const char* li_last_error();

/* 0 if the current device is a B200 (sm_100); the library has code for no other. */
int li_check_device();
/* Which of the launches that follow may NOT begin while the kernel before them still runs (programmatic dependent
 * launch): a mask of 1 tcgen05 GEMMs, 2 weight-streaming products, 4 attention, 8 the rest; 0 lets all overlap (the
 * default), 15 none.  The step function sets it per step.  LITINFER_B200_PDL=0 in the environment keeps all off. */
void li_pdl_allow(int kinds_off);

/* ---- resident block tables (elementwise.cu) ---- */
/* resident [rows, cols] int32: a row per state slot, the last row all sink page.  updates: a count, then triples (slot,
 * logical page, page id).  Applies the triples of each of the S sequences' slots, then copies the first max_blocks
 * entries of each sequence's row into out [S, max_blocks]. */
int li_table_gather(int* resident, int rows, int cols, const int* updates, int update_cap, const int* slots, int* out, int S, int
    max_blocks, int trash_page, cudaStream_t stream);

/* ---- attention.cu ---- */
/* Causal grouped-query attention of a step's tokens over the paged cache.  qkv [T, (nh + 2 nkv) dh] with q
 * rotated; out [T, nh dh]; token t of sequence s at position p sees the cached keys max(0, p - window + 1) .. p
 * through block_table[s]; singles: how many sequences of a step with longer portions have one token (negative: not
 * known); units (may be NULL): the work list of the kernel for long portions, made with the step's metadata (two counts,
 * two unused words, then per entry: sequence, tile of 128 tokens, part | parts << 8, unused), with the number of entries
 * to launch when the single tokens go to the decode kernel and when they do not. */
int li_paged_attention(const void* qkv, void* out, const void* kcache, const void* vcache, int dtype, const int*
    block_table, int max_blocks, const int* q_start, const int* ctx_lens, const int* seq_of_token, const int*
    positions, int T, int S, int nh, int nkv, int dh, int page_size, int num_pages, float scale, int window, int
    max_q_len, int max_ctx_len, const int* old_lens, int singles, const int* units, int slots_portions, int slots_all,
    cudaStream_t stream);

/* The same through one implementation: 0 general, 1 decode, 2 mma.sync tiles, 3 tcgen05 tiles (tests and
 * measurements). */
int li_paged_attention_with(int which, const void* qkv, void* out, const void* kcache, const void* vcache, int dtype,
    const int* block_table, int max_blocks, const int* q_start, const int* ctx_lens, const int* seq_of_token, const
    int* positions, int T, int S, int nh, int nkv, int dh, int page_size, int num_pages, float scale, int window, int
    max_q_len, int max_ctx_len, const int* old_lens, int singles, const int* units, int slots_portions, int slots_all,
    cudaStream_t stream);

/* ---- decode_step.cu: a decode step as one persistent kernel (decode_step.h has the structures) ---- */
struct LiDecodeStep;
int li_decode_step_accepts(int M, int hidden, int heads, int kv_heads, int head_dim, int intermediate, int vocab, int page_size);
int li_decode_step_plan(int M, int hidden, int heads, int kv_heads, int head_dim, int splits, int* stage_k, int* stages, int* x_cols, int*
    scratch_bytes);
int li_decode_step(const LiDecodeStep* step, cudaStream_t stream);

/* ---- elementwise.cu ---- */
/* out[t] = table[ids[t]] as float. */
int li_embedding(const void* table, int dtype, const int* ids, float* out, int T, int H, int V, cudaStream_t stream);

/* out = x / sqrt(mean(x^2) + eps) * w, rows of H; out in the run dtype. */
int li_rmsnorm(const float* x, const float* w, float eps, void* out, int dtype, int T, int H, cudaStream_t stream);

/* x += delta (in place, float), then out = rmsnorm(x). */
int li_add_rmsnorm(float* x, const void* delta, int dtype, const float* w, float eps, void* out, int T, int H,
    cudaStream_t stream);

/* out[r] = rmsnorm(x[rows[r]]): the final norm on the rows whose logits are wanted. */
int li_gather_rmsnorm(const float* x, const int* rows, const float* w, float eps, void* out, int dtype, int R, int T,
    int H, cudaStream_t stream);

/* x += delta over n elements. */
int li_residual_add(float* x, const void* delta, int dtype, long long n, cudaStream_t stream);

/* out[r, :] = src[rows[r], :] for n_rows rows of `width` floats. */
int li_gather_rows(const float* src, const int* rows, float* out, int n_src, int n_rows, long long width, cudaStream_t stream);

/* x *= factor over n floats (an embedding scale). */
int li_scale_inplace(float* x, long long n, float factor, cudaStream_t stream);

/* x = cap * tanh(x / cap) over n floats (a cap on the logits). */
int li_logit_cap(float* x, long long n, float cap, cudaStream_t stream);

/* out[t, i] = up * gate / (1 + exp(-gate)), gate_up [T, 2 I] as gate | up. */
int li_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream);

/* out = hprime * rinv per row, rinv from the partial sums of squares ssq[M, nparts] (the norm that rides on two
 * products, applied on its own). */
int li_apply_row_scale(const void* hprime, const float* ssq, int nparts, int width, float eps, void* out, int M, int
    H, cudaStream_t stream);

/* ---- gemm_tcgen05.cu ---- */
/* Measurements: 0 keeps the rotary epilogue to paired tiles. */
void li_tcgen05_rope_single_tiles(int on);

/* Tests and measurements: force a tile shape of the tcgen05 product (0: by shape). */
void li_tcgen05_force_tile(int tile);

/* Tests and measurements: force the splits of k of the tcgen05 product (0: by shape). */
void li_tcgen05_force_ksplit(int n);

/* ---- gemv_bf16.cu ---- */
/* The weight-streaming product for callers that may not allocate (see no_alloc.h). */
int li_linear_gemv_static(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int
    K, cudaStream_t stream);

/* ---- gemv_tcgen05.cu ---- */
/* Measurements: force the splits of k of the swapped tcgen05 product (0: by shape). */
void li_gemv_tcgen05_force_ksplit(int n);

/* ---- linear.cu ---- */
/* out[M, N] = a[M, K] w[N, K]^T (+ bias), epilogue 0 none / 1 SwiGLU over interleaved gate|up rows; float32 in
 * float32 out, or bfloat16 in, bfloat16 or float out. */
int li_linear(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N,
    int K, int epilogue, cudaStream_t stream);

/* 1 if li_linear_scaled takes this product. */
int li_linear_scaled_accepts(const void* a, const void* w, const void* out, int dtype_in, int M, int N, int K);

/* li_linear with each row of a scaled by rinv from partial sums of squares (a deferred RMSNorm). */
int li_linear_scaled(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M,
    int N, int K, int epilogue, const float* ssq, int nparts, int width, float eps, cudaStream_t stream);

/* How many partial sums per row li_linear_add_scaled leaves for this product (0: it refuses it). */
int li_linear_add_scaled_parts(const void* a, const void* w, const void* x32, const void* hprime, int dtype_in, int M,
    int N, int K);

/* x32 += a w^T (+ bias); hprime = bfloat16(norm_weight * x32); ssq_out[row, part] = sums of x32^2 over the part's
 * columns. */
int li_linear_add_scaled(const void* a, const void* w, const float* bias, float* x32, const float* norm_weight, void*
    hprime, float* ssq_out, int dtype_in, int M, int N, int K, cudaStream_t stream);

/* li_linear through one implementation (tests and measurements). */
int li_linear_with(int which, const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out,
    int M, int N, int K, int epilogue, cudaStream_t stream);

/* ---- rope.cu ---- */
/* out[t, j] = (cos, sin)(positions[t] / denom[j]). */
int li_rope_table(const int* positions, const float* denom, int half, float* out, int T, cudaStream_t stream);

/* Rotate q in place, rotate k and store it, store v (transposed) at slot_mapping[t] of the paged caches. */
int li_rope_kv_write(void* qkv, int dtype, const int* positions, const float* denom, int rotary_dim, const int*
    slot_mapping, void* kcache, void* vcache, int T, int nh, int nkv, int dh, int page_size, int num_pages, int write,
    cudaStream_t stream);

/* The q|k|v product followed by li_rope_kv_write, as one kernel where the shape allows. */
int li_linear_rope_kv(const void* a, const void* w, const float* bias, void* qkv, int dtype, const int* positions,
    const float* denom, int rotary_dim, const int* slot_mapping, void* kcache, void* vcache, int T, int K, int nh, int
    nkv, int dh, int page_size, int num_pages, int write, int allow_fused, const float* ssq, int nparts, int width,
    float eps, const float* cos_sin, cudaStream_t stream);

/* ---- sampling.cu ---- */
/* out[r] = the first maximum of logits[r]. */
int li_argmax(const float* logits, int* out, int R, int V, cudaStream_t stream);

/* out[r] = a draw from logits[r] under (temperature, top_k, top_p, seed, output index) packed in params; Gumbel-
 * max with a counter-based generator, independent of the batch. */
int li_sample(const float* logits, const int* params, int* out, int R, int V, cudaStream_t stream);

/* ---- fill_random.cu ---- */
/* out[i] = mean + std * n(key, i), n standard normal from a counter-based generator (a pure function of key and i). */
int li_fill_normal(void* out, int dtype, long long n, unsigned long long key, float mean, float std, cudaStream_t stream);

/* out[i] = an integer in [0, range) from (key, i). */
int li_fill_randint(int* out, long long n, unsigned long long key, int range, cudaStream_t stream);

/* ---- tcgen05_host.cu ---- */
/* 0, or the status a tcgen05 kernel left when one of its bounded waits ran out. */
int li_tcgen05_status();

/* Tests: clear the status word; make a bounded wait run out on purpose (one thread, a barrier nobody arrives on,
 * a limit in microseconds): the status then reads 99. */
void li_tcgen05_clear_status();

/* Progress marks of kernels launched with their debug flag (host memory, readable while they run). */
int li_tcgen05_progress(int* out, int n);
int li_tcgen05_wait_selftest(int limit_us, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
