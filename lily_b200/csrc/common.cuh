// Shared helpers of the sm_100a kernels: element types, reductions, error reporting.
//
// Every launcher is an `extern "C"` function that takes raw device pointers, sizes and a
// stream, checks what it can on the host, launches, and returns 0 or an error code;
// `lily_last_error()` gives the message of the last failure on the calling thread.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#define LILY_API extern "C" __attribute__((visibility("default")))

namespace lily {

enum DType : int { kF32 = 0, kBF16 = 1 };

void set_error(const char* fmt, ...);

#define LILY_REQUIRE(cond, ...)              \
    do {                                     \
        if (!(cond)) {                       \
            ::lily::set_error(__VA_ARGS__);  \
            return 1;                        \
        }                                    \
    } while (0)

#define LILY_CHECK_LAUNCH(name)                                                       \
    do {                                                                              \
        cudaError_t e__ = cudaGetLastError();                                         \
        if (e__ != cudaSuccess) {                                                     \
            ::lily::set_error("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
            return 2;                                                                 \
        }                                                                             \
    } while (0)

// Programmatic dependent launch: a kernel launched with `launch_pdl` may start while the kernel
// before it in the stream is still draining; it must call pdl_wait() before it touches anything
// that kernel wrote (what comes before the call overlaps with the predecessor's tail), and
// pdl_launch_dependents() once the kernel after it may begin the same way.  Both are no-ops in a
// kernel launched the ordinary way.  LILY_B200_PDL=0 in the environment launches everything the
// ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// How a short kernel between two long ones enters: the kernel after it may start at once, and
// stream in what depends on no one (weights, cached keys of earlier steps), while this kernel still
// waits for its own predecessor.  Every kernel waits before it reads or writes anything that
// another kernel of the step writes, and a kernel only completes after its wait, so the order of
// the step's writes is kept along the chain however early the launches are.
__device__ __forceinline__ void pdl_enter_small() {
    pdl_launch_dependents();
    pdl_wait();
}

bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Streaming multiprocessors of the current device (148 on a B200), asked once.
inline int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    return sms;
}

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace lily
