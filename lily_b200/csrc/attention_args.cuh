// Arguments shared by the attention kernels (CUDA-core and tensor-core files).
#pragma once

namespace lily {

struct AttnArgs {
    const void* q;            // [tokens, nq, d]
    const void* kv;           // layer base
    void* out;                // [tokens, nq, d]
    const int* block_table;   // [requests, bt_stride]
    int bt_stride;
    const int* cu_seqlens;    // prefill: [requests + 1] offsets of each request's new tokens
    const int* prefix_lens;   // prefill: [requests] cached positions before the new tokens
    const int* tile_req;      // prefill: [tiles]
    const int* tile_start;    // prefill: [tiles] offset of the tile in its request's new tokens
    const int* seq_lens;      // decode: [requests] positions after this step
    float* part_o;            // decode: [requests, nq, splits, d]
    float* part_ml;           // decode: [requests, nq, splits, 2]
    int splits;
    int nq, nkv, d, page_size, window;
    float scale;
};

}  // namespace lily
