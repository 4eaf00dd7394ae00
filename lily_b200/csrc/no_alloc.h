// An entry point of the kernel library that allocates nothing.  It has no counterpart in
// CodeMan62/lily; it exists for callers of this library that must not allocate device memory.
//
// Who they are: a host program that hands the whole device to its own pool at start-up (weights
// and the KV cache sized from what is free, as this engine's own runner does with
// mem_fraction_static) has nothing left for a later cudaMalloc, which may then fail or stall the
// device while it is served; and hosts that load this library as a plug-in often forbid
// allocation calls from extension code once their serving loop runs.  Such callers cannot use
// lily_attention_decode_simt / lily_attention_decode_mma with splits > 1, because those need a
// scratch buffer that somebody has to allocate.
//
// lily_attention_decode_static runs the same split-key decode attention (the tensor-core kernels
// for bfloat16 with head sizes 64, 128, 192, 256; the CUDA-core kernels otherwise) and merges the
// splits, with the partial results kept in an array that is part of the library image:
// LILY_STATIC_SCRATCH_FLOATS float32 (8 MiB), held by every GPU that loads the library until the
// process exits.  The caller passes inputs and outputs only.
//
//  * Limit: requests * nq * splits * (d + 2) <= LILY_STATIC_SCRATCH_FLOATS when splits > 1
//    (lily_attention_decode_static_fits tells); larger sizes are refused with an error, not
//    truncated.  splits == 1 needs no scratch and is never refused for size.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and keeps it; make that first call before any stream capture begins.
//  * All calls share the one array and it keeps what the last call left.  Nothing in it has to
//    start at zero: every split writes its own (max, sum, output) before the merge reads them.
//    Two calls that overlap on the GPU (different streams, or several host threads) race on it:
//    order them on one stream.
//  * It calls no cudaMalloc, cudaFree or allocating library routine.
//
// Arguments are those of lily_attention_decode_simt (attention_simt.cu) without the scratch pointer:
// q, out [requests, nq * d]; kv one layer of the cache [pages, 2, kv_heads, page_size, d];
// block_table int32 [requests, bt_stride]; seq_lens int32 [requests]; dtype 0 float32, 1 bfloat16.
// Returns 0, or non-zero with the message in lily_last_error().
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#define LILY_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)

#ifdef __cplusplus
extern "C" {
#endif

int lily_attention_decode_static(const void* q, const void* kv, void* out, const int* block_table, int bt_stride,
                                 const int* seq_lens, int requests, int splits, int nq, int nkv, int d,
                                 int page_size, int window, float scale, int dtype, cudaStream_t stream);

// 1 when a call with these sizes fits the static scratch (always 1 for splits <= 1).
int lily_attention_decode_static_fits(int requests, int splits, int nq, int d);

#ifdef __cplusplus
}
#endif
