#include "common.cuh"
bool li_attention_decode_accepts(int nh, int nkv, int dh, int page_size) { return false; }
int li_attention_decode(const void* qkv, void* out, const void* kcache, const void* vcache, const int* block_table, int max_blocks,
                        const int* ctx_lens, int S, int nh, int nkv, int dh, int page_size, int num_pages, float scale, int window,
                        int max_ctx_len, cudaStream_t stream) { return li_fail("not built"); }
