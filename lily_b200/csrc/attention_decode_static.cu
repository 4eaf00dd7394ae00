// Split-key decode attention whose scratch is a static device array: see no_alloc.h, which
// declares the entry point, says for whom it is, and states its limit and its rules of use.
#include "no_alloc.h"

#include "common.cuh"

// The existing launchers this entry point drives (attention_simt.cu, attention_mma.cu).
extern "C" int lily_attention_decode_simt(const void*, const void*, void*, const int*, int, const int*, float*, int, int,
                                          int, int, int, int, int, float, int, cudaStream_t);
extern "C" int lily_attention_decode_mma(const void*, const void*, void*, const int*, int, const int*, float*, int, int,
                                         int, int, int, int, int, float, int, cudaStream_t);
extern "C" int lily_attention_mma_supports(int);

// Partial (output, max, sum) of every split of the last call.  In host code this name is only a
// handle for cudaGetSymbolAddress; the kernels are given the address that call returns.
static __device__ __align__(256) float g_static_scratch[LILY_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};

// The array's address on the current device, looked up once per device.
int scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        lily::set_error("attention_decode_static: cannot tell the current device (%s)", cudaGetErrorString(e));
        return 2;
    }
    if (g_scratch_address[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            lily::set_error("attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                            cudaGetErrorString(e));
            return 2;
        }
        g_scratch_address[dev] = p;
    }
    *out = g_scratch_address[dev];
    return 0;
}

size_t scratch_floats(int requests, int splits, int nq, int d) {
    return splits > 1 ? (size_t)requests * nq * splits * ((size_t)d + 2) : 0;
}
}  // namespace

LILY_API int lily_attention_decode_static_fits(int requests, int splits, int nq, int d) {
    if (requests < 0 || splits < 0 || nq < 0 || d < 0) return 0;
    return scratch_floats(requests, splits, nq, d) <= (size_t)LILY_STATIC_SCRATCH_FLOATS ? 1 : 0;
}

LILY_API int lily_attention_decode_static(const void* q, const void* kv, void* out, const int* block_table,
                                          int bt_stride, const int* seq_lens, int requests, int splits, int nq,
                                          int nkv, int d, int page_size, int window, float scale, int dtype,
                                          cudaStream_t stream) {
    if (requests == 0) return 0;
    LILY_REQUIRE(requests > 0 && splits >= 1 && nq > 0 && nkv > 0 && d > 0,
                 "attention_decode_static: bad sizes requests=%d splits=%d nq=%d nkv=%d d=%d", requests, splits, nq, nkv, d);
    const size_t need = scratch_floats(requests, splits, nq, d);
    LILY_REQUIRE(need <= (size_t)LILY_STATIC_SCRATCH_FLOATS,
                 "attention_decode_static: requests=%d x nq=%d x splits=%d x (d=%d + 2) = %zu float32 of scratch, "
                 "the static array holds %u; use fewer splits or a smaller batch",
                 requests, nq, splits, d, need, (unsigned)LILY_STATIC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (need > 0) {
        const int rc = scratch_for_current_device(&scratch);
        if (rc) return rc;
    }
    if (dtype == lily::kBF16 && lily_attention_mma_supports(d)) {
        // merges the splits itself: inside a cluster, or by the combine kernel behind it
        return lily_attention_decode_mma(q, kv, out, block_table, bt_stride, seq_lens, scratch, requests, splits, nq, nkv,
                                         d, page_size, window, scale, 0, stream);
    }
    return lily_attention_decode_simt(q, kv, out, block_table, bt_stride, seq_lens, scratch, requests, splits, nq, nkv,
                                      d, page_size, window, scale, dtype, stream);
}
