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
    // decode, tensor-core kernel only: the qkv product as it leaves the projection (this kernel then norms and
    // rotates its own query heads, and the block whose key range holds the new position does the same for the
    // key, and writes key and value to the cache, before it reads them).  Null: `q` holds finished queries.
    const void* qkv;          // [planes][requests, (nq + 2 nkv) d]: float32 partial sums, or bfloat16 with one plane
    int qkv_planes, qkv_f32;
    size_t qkv_stride;        // elements between planes
    const void* q_gain;       // [d] per-head RMSNorm gains (both or none), float32 or bfloat16
    const void* k_gain;
    int gain_f32;
    float eps;
    const float* cos_t;       // [positions, rd / 2] (both or none)
    const float* sin_t;
    int rd;                   // rotary width
    int write_kv;             // 0: the cache already holds this position (a layer that reads another layer's cache)
    int stages;               // decode, tensor-core kernel: key/value tiles a block keeps in shared memory (0: the default, 2;
                              // 3: two blocks a SM instead of three, each with two tiles in flight; head sizes up to 128)
};

}  // namespace lily
