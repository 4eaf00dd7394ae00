// Memory-bound kernels of the step: embedding rows, fused residual-add + RMSNorm,
// SiLU*mul, and the fused per-head (bias +) RMSNorm + rotary + cache write.
//
// The residual stream is float32 in both precisions; activations (`T`) are float or
// bfloat16; norm gains (`W`) are float or bfloat16 (a gain stored in 32-bit stays so).
// Variances, rsqrt, rotation angles and the residual sum are float32.
//
// Formulas: RMSNorm lily/layers/layernorm.py:37-44 (and its CUDA twin
// lily/csrc/small_fused.cu:45-85), rotate-half rotary lily/layers/rotary.py:18-20,70-87
// (small_fused.cu:124-142), SiLU*mul lily/models/llama.py:45, cache write
// lily/mem_cache/memory_pool.py:137-143, embedding lily/layers/vocab_embedding.py:37-39.
#include "common.cuh"

#include <cstdarg>

namespace lily {

static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// ---------------------------------------------------------------------------- embedding

template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int hidden, int vocab) {
    const int n = blockIdx.x;
    int id = ids[n];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);   // the host has checked the range
    const T* src = table + (size_t)id * hidden;
    float* dst = out + (size_t)n * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(src[i]);
}

// ---------------------------------------------------------------------------- add + RMSNorm

// One block per output row m.  src = rows ? rows[m] : m.
//   v = resid[src] (+ delta[src]);  if write_residual: resid[src] = v
//   out[m] = v * rsqrt(mean(v^2) + eps) * weight
template <typename T, typename W>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const W* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps, int write_residual,
                                   int stash) {
    extern __shared__ float smem[];
    float* red = smem;             // 33 floats
    float* row = smem + 40;        // hidden floats when stash
    const int m = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[m] : m) * hidden;
    float ssq = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = resid[src + i];
        if (delta) v += to_float(delta[src + i]);
        if (write_residual && delta) resid[src + i] = v;
        if (stash) row[i] = v;
        ssq += v * v;
    }
    const float total = block_sum(ssq, red);
    const float inv = rsqrtf(total / (float)hidden + eps);
    T* dst = out + (size_t)m * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v;
        if (stash) {
            v = row[i];
        } else {
            v = resid[src + i];
            if (delta && !write_residual) v += to_float(delta[src + i]);
        }
        dst[i] = from_float<T>((v * inv) * to_float(weight[i]));
    }
}

// ---------------------------------------------------------------------------- SiLU * mul

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t n = idx / inter;
        const int i = (int)(idx - n * inter);
        const float g = to_float(gate_up[n * 2 * inter + i]);
        const float u = to_float(gate_up[n * 2 * inter + inter + i]);
        out[idx] = from_float<T>((g / (1.f + expf(-g))) * u);
    }
}

// ---------------------------------------------------------------------------- q/k norm + rotary + cache write

// grid (tokens, ceil(heads / 4)), block (32, 4): one warp per (token, head) of the fused
// projection [q heads | k heads | v heads].  q heads go to q_out, k and v heads into the
// token's place in its page.
template <typename T, typename W>
__global__ void qk_norm_rope_write_kernel(const T* __restrict__ qkv, const W* __restrict__ q_gain,
                                          const W* __restrict__ k_gain, float eps,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          const int* __restrict__ positions, const int* __restrict__ token_req,
                                          const int* __restrict__ block_table, int bt_stride,
                                          T* __restrict__ kv_layer, T* __restrict__ q_out,
                                          int nq, int nkv, int d, int rd, int page_size, int write_kv) {
    const int n = blockIdx.x;
    const int head = blockIdx.y * blockDim.y + threadIdx.y;
    const int nheads = write_kv ? nq + 2 * nkv : nq;
    if (head >= nheads) return;
    const int lane = threadIdx.x;
    const int pos = positions[n];
    const T* src = qkv + (size_t)n * (nq + 2 * nkv) * d + (size_t)head * d;
    T* dst;
    const W* gain = nullptr;
    bool rotate = true;
    if (head < nq) {
        dst = q_out + ((size_t)n * nq + head) * d;
        gain = q_gain;
    } else {
        const int is_v = head >= nq + nkv;
        const int kvh = head - nq - (is_v ? nkv : 0);
        const int page = block_table[(size_t)token_req[n] * bt_stride + pos / page_size];
        dst = kv_layer + ((((size_t)page * 2 + is_v) * nkv + kvh) * page_size + (pos % page_size)) * d;
        gain = is_v ? nullptr : k_gain;
        rotate = !is_v;
    }
    float inv = 1.f;
    if (gain) {
        float ssq = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float x = to_float(src[i]);
            ssq += x * x;
        }
        ssq = warp_sum(ssq);
        inv = rsqrtf(ssq / (float)d + eps);
    }
    if (!rotate) {
        for (int i = lane; i < d; i += 32) dst[i] = src[i];
        return;
    }
    const int half = rd >> 1;
    const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* s = sin_t ? sin_t + (size_t)pos * half : nullptr;
    for (int i = lane; i < half; i += 32) {
        float x1 = to_float(src[i]), x2 = to_float(src[i + half]);
        if (gain) {
            x1 = (x1 * inv) * to_float(gain[i]);
            x2 = (x2 * inv) * to_float(gain[i + half]);
        }
        float o1 = x1, o2 = x2;
        if (c) {
            const float cc = c[i], ss = s[i];
            o1 = x1 * cc - x2 * ss;
            o2 = x2 * cc + x1 * ss;
        }
        dst[i] = from_float<T>(o1);
        dst[i + half] = from_float<T>(o2);
    }
    for (int i = rd + lane; i < d; i += 32) {
        float x = to_float(src[i]);
        if (gain) x = (x * inv) * to_float(gain[i]);
        dst[i] = from_float<T>(x);
    }
}

// ---------------------------------------------------------------------------- casts

template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ in, B* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_float<B>(to_float(in[i]));
}

}  // namespace lily

using namespace lily;

LILY_API const char* lily_last_error() { return g_error; }

LILY_API int lily_embed(const void* table, int table_dtype, const int* ids, float* out, int tokens, int hidden,
                        int vocab, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(hidden > 0 && vocab > 0, "embed: bad sizes hidden=%d vocab=%d", hidden, vocab);
    if (table_dtype == kBF16)
        embed_kernel<<<tokens, 256, 0, stream>>>((const __nv_bfloat16*)table, ids, out, hidden, vocab);
    else
        embed_kernel<<<tokens, 256, 0, stream>>>((const float*)table, ids, out, hidden, vocab);
    LILY_CHECK_LAUNCH("embed");
    return 0;
}

template <typename T, typename W>
static int launch_add_rmsnorm(float* resid, const void* delta, const void* weight, void* out, const int* rows,
                              int out_rows, int hidden, float eps, int write_residual, cudaStream_t stream) {
    const int stash = hidden <= 11264;   // 40 + hidden floats stay within 48 KB
    const size_t smem = (40 + (stash ? hidden : 0)) * sizeof(float);
    const int threads = hidden >= 2048 ? 512 : 256;
    add_rmsnorm_kernel<T, W><<<out_rows, threads, smem, stream>>>(resid, (const T*)delta, (const W*)weight, (T*)out,
                                                               rows, hidden, eps, write_residual, stash);
    return 0;
}

LILY_API int lily_add_rmsnorm(float* resid, const void* delta, const void* weight, void* out, const int* rows,
                              int out_rows, int hidden, float eps, int write_residual, int act_dtype,
                              int weight_dtype, cudaStream_t stream) {
    if (out_rows == 0) return 0;
    LILY_REQUIRE(hidden > 0, "add_rmsnorm: hidden=%d", hidden);
    LILY_REQUIRE(!(rows && write_residual && delta), "add_rmsnorm: gathered rows cannot write the residual back");
    if (act_dtype == kBF16 && weight_dtype == kBF16)
        launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, weight, out, rows, out_rows, hidden, eps, write_residual, stream);
    else if (act_dtype == kBF16)
        launch_add_rmsnorm<__nv_bfloat16, float>(resid, delta, weight, out, rows, out_rows, hidden, eps, write_residual, stream);
    else if (weight_dtype == kBF16)
        launch_add_rmsnorm<float, __nv_bfloat16>(resid, delta, weight, out, rows, out_rows, hidden, eps, write_residual, stream);
    else
        launch_add_rmsnorm<float, float>(resid, delta, weight, out, rows, out_rows, hidden, eps, write_residual, stream);
    LILY_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

LILY_API int lily_silu_mul(const void* gate_up, void* out, int tokens, int inter, int act_dtype, cudaStream_t stream) {
    const size_t total = (size_t)tokens * inter;
    if (total == 0) return 0;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (act_dtype == kBF16)
        silu_mul_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
    else
        silu_mul_kernel<<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
    LILY_CHECK_LAUNCH("silu_mul");
    return 0;
}

LILY_API int lily_qk_norm_rope_write(const void* qkv, const void* q_gain, const void* k_gain, float eps,
                                     const float* cos_t, const float* sin_t, const int* positions,
                                     const int* token_req, const int* block_table, int bt_stride, void* kv_layer,
                                     void* q_out, int tokens, int nq, int nkv, int d, int rd, int page_size,
                                     int write_kv, int act_dtype, int gain_dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(d > 0 && rd >= 0 && rd <= d && rd % 2 == 0, "qk_norm_rope_write: rotary_dim %d does not fit head_dim %d", rd, d);
    LILY_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "qk_norm_rope_write: q and k gains come together");
    LILY_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "qk_norm_rope_write: cos and sin tables come together");
    const int nheads = write_kv ? nq + 2 * nkv : nq;
    dim3 grid(tokens, (nheads + 3) / 4), block(32, 4);
#define LAUNCH(T, W)                                                                                              \
    qk_norm_rope_write_kernel<T, W><<<grid, block, 0, stream>>>((const T*)qkv, (const W*)q_gain, (const W*)k_gain, eps, \
        cos_t, sin_t, positions, token_req, block_table, bt_stride, (T*)kv_layer, (T*)q_out, nq, nkv, d,          \
        cos_t ? rd : 0, page_size, write_kv)
    if (act_dtype == kBF16 && gain_dtype == kBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (act_dtype == kBF16) LAUNCH(__nv_bfloat16, float);
    else if (gain_dtype == kBF16) LAUNCH(float, __nv_bfloat16);
    else LAUNCH(float, float);
#undef LAUNCH
    LILY_CHECK_LAUNCH("qk_norm_rope_write");
    return 0;
}

LILY_API int lily_cast(const void* in, int in_dtype, void* out, int out_dtype, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (in_dtype == kBF16 && out_dtype == kF32)
        cast_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, n);
    else if (in_dtype == kF32 && out_dtype == kBF16)
        cast_kernel<<<blocks, 256, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, n);
    else
        LILY_REQUIRE(false, "cast: unsupported pair %d -> %d", in_dtype, out_dtype);
    LILY_CHECK_LAUNCH("cast");
    return 0;
}
