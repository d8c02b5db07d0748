/* The fused decode step: a whole step of single tokens (every sequence one new token) of a pre-norm decoder of
 * attention + gated feed-forward layers as ONE persistent kernel.
 *
 * LitInfer runs a step as a loop of operator calls per layer (src/llaisys/models/qwen2.cpp:967-1047); launched as
 * separate kernels, a decode layer on this GPU is five dependent kernels of 5-14 us of which 3-4 us each are ramp-up
 * and drain, while its weights would stream in under 15 us.  Here one CTA per multiprocessor stays resident for the
 * whole step.  A producer warp streams the CTA's share of every weight matrix, layer after layer, through a ring of
 * shared-memory stages with bulk asynchronous copies (cp.async.bulk + mbarrier), never waiting for anything but a free
 * stage: weights depend on nothing, so the stream runs ahead across the phases and layers.  Eight consumer warps
 * multiply what has arrived (mma.sync m16n8k16, 16 weight rows x the step's tokens, as in gemv_bf16.cu) and run the
 * phases of a layer: q|k|v with rotary encoding and cache write, attention over the paged cache, output projection
 * into the residual stream, gate|up with SwiGLU, down projection into the stream; the RMSNorms ride on the products
 * (row_scale.cuh).  Between phases the CTAs meet at a grid-wide barrier (an arrival counter in global memory;
 * the kernel is launched cooperatively, so all CTAs are resident).  Every wait is bounded: a barrier or a stage that
 * does not come within the limit raises the status word (li_tcgen05_status) and the CTA leaves.
 *
 * The structures below are filled by the caller: the layers once per model (an array in device memory), the
 * step's arguments per launch (passed by value).  All pointers are device pointers.
 */
#pragma once

#include <cuda_runtime.h>

#define LI_DECODE_MAX_GROUPS 8

typedef struct LiDecodeLayer {
    const void* w_qkv;        /* bfloat16 [(heads + 2 kv_heads) * head_dim, hidden] */
    const float* b_qkv;       /* float [(heads + 2 kv_heads) * head_dim] or NULL */
    const void* w_o;          /* bfloat16 [hidden, heads * head_dim] */
    const void* w_gate_up;    /* bfloat16 [2 * intermediate, hidden], gate and up rows interleaved in groups of 8 */
    const void* w_down;       /* bfloat16 [hidden, intermediate] */
    const float* norm_ffn;    /* float [hidden]: weights of the norm before the feed-forward */
    const float* norm_next;   /* float [hidden]: weights of the norm that follows this layer (the next layer's first, or the final one) */
    void* kcache;             /* bfloat16 [pages, kv_heads, page_size, head_dim] */
    void* vcache;             /* bfloat16 [pages, kv_heads, head_dim, page_size] */
    const float* rope_denom;  /* float [head_dim / 2] */
    float eps_ffn, eps_next;  /* of the two norms above */
    float scale;              /* of the attention scores */
    int window;               /* keys a query sees, 0: all */
    int group;                /* which of the step's block tables / slot mappings this layer's cache uses */
    int num_pages;
    int write_cache;          /* 0: the layer reads a cache another layer wrote in this step */
    int reserved;
} LiDecodeLayer;

typedef struct LiDecodeStep {
    const LiDecodeLayer* layers;
    int num_layers;
    int M;                    /* tokens of the step = sequences, 1..16 */
    int hidden, heads, kv_heads, head_dim, intermediate, vocab, page_size, max_blocks;
    const void* embedding;    /* bfloat16 [vocab, hidden] */
    const float* norm_first;  /* float [hidden]: the first layer's first norm */
    float eps_first;
    int rows;                 /* logit rows wanted, 0..M */
    const int* token_ids;     /* [M] */
    const int* positions;     /* [M] */
    const int* ctx_lens;      /* [M] keys each sequence sees, its new token included */
    const int* old_lens;      /* [M] keys cached before this step, or NULL (ctx_lens - 1) */
    const int* logit_rows;    /* [rows] tokens whose logits are wanted */
    const int* slot_mapping[LI_DECODE_MAX_GROUPS];   /* per cache group: [M] */
    const int* block_table[LI_DECODE_MAX_GROUPS];    /* per cache group: [M, max_blocks] */
    const void* lm_head;      /* bfloat16 [vocab, hidden] */
    float* logits;            /* float [rows, vocab] */
    /* scratch, device memory owned by the caller; see li_decode_step_scratch for the sizes */
    float* x32;               /* [M, hidden] the residual stream */
    void* h_a;                /* bfloat16 [M, hidden]: input of q|k|v (and of the lm_head) with the norm's weights applied */
    void* h_b;                /* bfloat16 [M, hidden]: input of gate|up likewise */
    float* ssq_a;             /* [M, hidden / 16] partial sums of squares behind h_a */
    float* ssq_b;             /* [M, hidden / 16] behind h_b */
    void* qkv;                /* bfloat16 [M, (heads + 2 kv_heads) * head_dim] */
    void* attn;               /* bfloat16 [M, heads * head_dim] */
    void* act;                /* bfloat16 [M, intermediate] */
    float* attn_part;         /* [M, heads, splits, head_dim + 2] */
    unsigned* attn_counters;  /* [M * kv_heads], zero between launches */
    unsigned* barrier;        /* [1], zero at launch: li_decode_step clears it */
    int splits;               /* splits of 256 keys the partial sums hold */
    int stage_k;              /* columns of a weight row per stage of the ring (a multiple of 32) */
    int stages;               /* stages of the ring */
    int balance;              /* bit 1: progress marks and barrier time stamps in the mapped status area (debugging) */
    int x_cols;               /* columns of the shared buffer for a product's activations (a multiple of 64), 0: none */
} LiDecodeStep;

#ifdef __cplusplus
extern "C" {
#endif

/* 0 if a step of these sizes can run fused, else non-zero with the reason in li_last_error(). */
int li_decode_step_accepts(int M, int hidden, int heads, int kv_heads, int head_dim, int intermediate, int vocab, int page_size);

/* The shared-memory plan for these sizes: columns per stage and stages of the weight ring, columns of the buffer for a
 * product's activations (0: none fits), bytes of scratch beside them. */
int li_decode_step_plan(int M, int hidden, int heads, int kv_heads, int head_dim, int splits, int* stage_k, int* stages, int* x_cols,
    int* scratch_bytes);

/* Runs the step on `stream`: clears the barrier word, launches the kernel cooperatively. */
int li_decode_step(const LiDecodeStep* step, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
