// What the q|k|v product of a prefill step needs to finish its own rows: rotary position encoding of q and k from a
// table of cosines and sines that is made once per step (the angles are float32: float(pos) / denom[j], as in rope.cu),
// keys into the paged cache, values into it transposed.  head_dim = rotary_dim = 128 (a tile of 256 columns is two heads).
#pragma once

#include "common.cuh"

struct RopeEpilogue {
    const float* cos_sin = nullptr;      // [tokens, 64, 2]: cos and sin of pos / denom[j]
    const int* slot_mapping = nullptr;   // [tokens]
    bf16* kcache = nullptr;              // [pages, nkv, page_size, 128]
    bf16* vcache = nullptr;              // [pages, nkv, 128, page_size]
    int nh = 0, nkv = 0, page_size = 0, num_pages = 0, write = 0;
};
