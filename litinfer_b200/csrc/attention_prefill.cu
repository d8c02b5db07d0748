#include "common.cuh"
bool li_attention_prefill_accepts(int nh, int nkv, int dh, int page_size) { return false; }
int li_attention_prefill(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                         const int* q_start, const int* ctx_lens, int T, int S, int nh, int nkv, int dh, int page_size,
                         int num_pages, float scale, int window, int max_q_len, cudaStream_t stream) { return li_fail("not built"); }
