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

#include <cooperative_groups.h>

#include <cstdarg>
#include <cstdlib>

namespace cg = cooperative_groups;

namespace lily {

static thread_local char g_error[512] = "";
bool pdl_enabled() {
    static const bool on = [] {
        const char* v = getenv("LILY_B200_PDL");
        return !(v && v[0] == '0');
    }();
    return on;
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// Four consecutive elements at a time (the element index is a multiple of 4 and the base pointers
// are 16-byte aligned, which the launchers check before they pick the VEC = 4 kernels).
__device__ __forceinline__ float4 load4(const float* p, size_t i) { return *reinterpret_cast<const float4*>(p + i); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p, size_t i) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p + i);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, size_t i, float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, size_t i, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p + i) = raw;
}

__device__ __forceinline__ float2 load2(const float* p, size_t i) { return *reinterpret_cast<const float2*>(p + i); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p, size_t i) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + i));
}
__device__ __forceinline__ void store2(float* p, size_t i, float2 v) { *reinterpret_cast<float2*>(p + i) = v; }
__device__ __forceinline__ void store2(__nv_bfloat16* p, size_t i, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p + i) = __floats2bfloat162_rn(v.x, v.y);
}

// A kernel input that may arrive as `splits` float32 partial sums (the slices of a split-k
// product, `stride` elements apart) to be added up in order while it is read.
template <typename IN>
struct Summed {
    const IN* p;
    int splits;
    size_t stride;
    __device__ __forceinline__ float operator()(size_t i) const {
        float v = to_float(p[i]);
        for (int s = 1; s < splits; ++s) v += to_float(p[i + (size_t)s * stride]);
        return v;
    }
    __device__ __forceinline__ float4 four(size_t i) const {
        float4 v = load4(p, i);
        for (int s = 1; s < splits; ++s) {
            const float4 t = load4(p, i + (size_t)s * stride);
            v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
        }
        return v;
    }
    __device__ __forceinline__ float2 two(size_t i) const {
        float2 v = load2(p, i);
        for (int s = 1; s < splits; ++s) {
            const float2 t = load2(p, i + (size_t)s * stride);
            v.x += t.x; v.y += t.y;
        }
        return v;
    }
    __device__ __forceinline__ explicit operator bool() const { return p != nullptr; }
};

// ---------------------------------------------------------------------------- embedding

// An id below zero names a request slot: the token is the one the sampler stored for that slot
// after the step before (`future`), so that a step can be launched before the host has seen it.
template <typename T, int VEC>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ future,
                             float* __restrict__ out, int hidden, int vocab, float scale) {
    pdl_enter_small();
    const int n = blockIdx.x;
    int id = ids[n];
    if (id < 0 && future != nullptr) id = future[-id - 1];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);   // the host has checked the range of what it knew
    const T* src = table + (size_t)id * hidden;
    float* dst = out + (size_t)n * hidden;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float4 v = load4(src, i);
            v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
            store4(dst, i, v);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(src[i]) * scale;
    }
}

// logits[i] = cap * tanh(scale * logits[i] / cap) (cap > 0), else scale * logits[i]; in place, float32.
__global__ void logit_transform_kernel(float* __restrict__ logits, size_t n, float scale, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = logits[i] * scale;
        logits[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
    }
}

// future[slot of row i] = tokens[i]: row i of the step's logits belongs to token logit_rows[i], that
// token to request token_req[.], that request to slot slots[.].
__global__ void scatter_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ logit_rows,
                                      const int* __restrict__ token_req, const int* __restrict__ slots,
                                      int* __restrict__ future, int n, int max_slots) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int slot = slots[token_req[logit_rows[i]]];
    if (slot >= 0 && slot < max_slots) future[slot] = tokens[i];
}

// ---------------------------------------------------------------------------- add + RMSNorm

// One block per output row m.  src = rows ? rows[m] : m.
//   v = resid[src] (+ delta[src]);  if write_residual: resid[src] = v
//   out[m] = v * rsqrt(mean(v^2) + eps) * weight
template <typename T, typename W, typename IN, int VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const Summed<IN> delta,
                                   const W* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps, int write_residual,
                                   int stash) {
    extern __shared__ __align__(16) float smem[];
    pdl_enter_small();
    float* red = smem;             // 33 floats
    float* row = smem + 40;        // hidden floats when stash
    const int m = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[m] : m) * hidden;
    float ssq = 0.f;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float4 v = load4(resid, src + i);
            if (delta) {
                const float4 dl = delta.four(src + i);
                v.x += dl.x; v.y += dl.y; v.z += dl.z; v.w += dl.w;
                if (write_residual) store4(resid, src + i, v);
            }
            if (stash) store4(row, i, v);
            ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = resid[src + i];
            if (delta) v += delta(src + i);
            if (write_residual && delta) resid[src + i] = v;
            if (stash) row[i] = v;
            ssq += v * v;
        }
    }
    const float total = block_sum(ssq, red);
    const float inv = rsqrtf(total / (float)hidden + eps);
    T* dst = out + (size_t)m * hidden;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float4 v;
            if (stash) {
                v = load4(row, i);
            } else {
                v = load4(resid, src + i);
                if (delta && !write_residual) {
                    const float4 dl = delta.four(src + i);
                    v.x += dl.x; v.y += dl.y; v.z += dl.z; v.w += dl.w;
                }
            }
            const float4 g = load4(weight, i);
            store4(dst, i, make_float4((v.x * inv) * g.x, (v.y * inv) * g.y, (v.z * inv) * g.z, (v.w * inv) * g.w));
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v;
            if (stash) {
                v = row[i];
            } else {
                v = resid[src + i];
                if (delta && !write_residual) v += delta(src + i);
            }
            dst[i] = from_float<T>((v * inv) * to_float(weight[i]));
        }
    }
}

// The same for a few rows (decode): a thread-block cluster of CL blocks shares one row, each block
// takes hidden / CL columns (four per thread) and the blocks exchange their sums of squares
// through distributed shared memory, so that 8 rows keep 64 SMs busy instead of 8.
// grid (CL, rows), cluster (CL, 1, 1); hidden % (4 * CL) == 0; block = hidden / (4 * CL) threads.
template <typename T, typename W, typename IN, int CL>
__global__ void add_rmsnorm_cluster_kernel(float* __restrict__ resid, const Summed<IN> delta,
                                           const W* __restrict__ weight, T* __restrict__ out,
                                           const int* __restrict__ rows, int hidden, float eps, int write_residual) {
    __shared__ float red[40];
    __shared__ float share[CL];                                      // every block's sum of squares, sent by its owner
    cg::cluster_group cluster = cg::this_cluster();
    pdl_enter_small();
    const int m = blockIdx.y;
    const size_t src = (size_t)(rows ? rows[m] : m) * hidden;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;       // this thread's four columns
    float4 v = load4(resid, src + i);
    if (delta) {
        const float4 dl = delta.four(src + i);
        v.x += dl.x; v.y += dl.y; v.z += dl.z; v.w += dl.w;
        if (write_residual) store4(resid, src + i, v);
    }
    const float4 g = load4(weight, i);
    const float mine = block_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w, red);
    // each block tells every block of the cluster its sum; after the one barrier nobody touches another block's
    // shared memory again, so a block may leave as soon as it is done
    if (threadIdx.x < CL) cluster.map_shared_rank(&share[0], threadIdx.x)[blockIdx.x] = mine;
    cluster.sync();
    float total = 0.f;
#pragma unroll
    for (int r = 0; r < CL; ++r) total += share[r];                  // same order in every block
    const float inv = rsqrtf(total / (float)hidden + eps);
    store4(out + (size_t)m * hidden, i, make_float4((v.x * inv) * g.x, (v.y * inv) * g.y, (v.z * inv) * g.z, (v.w * inv) * g.w));
}

// ---------------------------------------------------------------------------- SiLU * mul

__device__ __forceinline__ float silu_times(float g, float u) { return (g / (1.f + expf(-g))) * u; }

// The gate and up columns of one token alternate in runs of `block`: [gate block | up block | gate
// block | ...]; block == inter is the plain [all gate | all up] order.
template <typename T, typename IN, int VEC>
__global__ void silu_mul_kernel(const Summed<IN> gate_up, T* __restrict__ out, int inter, int block, size_t total) {
    pdl_enter_small();
    const size_t step = (size_t)gridDim.x * blockDim.x * VEC;
    for (size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC; idx < total; idx += step) {
        const size_t n = idx / inter;
        const int i = (int)(idx - n * inter);
        const size_t at = n * 2 * inter + (size_t)(i / block) * 2 * block + (i % block);
        if (VEC == 4) {
            const float4 g = gate_up.four(at), u = gate_up.four(at + block);
            store4(out, idx, make_float4(silu_times(g.x, u.x), silu_times(g.y, u.y), silu_times(g.z, u.z), silu_times(g.w, u.w)));
        } else {
            out[idx] = from_float<T>(silu_times(gate_up(at), gate_up(at + block)));
        }
    }
}

// The same for a bfloat16 product in one piece (no partial sums) whose runs are multiples of eight: 16-byte loads
// and stores, eight outputs a thread and turn, the exponential and the quotient in their fast forms (as the fused
// gate/up kernels compute them; the result is rounded to bfloat16 either way).  2,048 x 12,288 outputs: 44 -> 25 us, 0.92 of HBM.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter,
                                       int block, size_t total) {
    pdl_enter_small();
    const size_t step = (size_t)gridDim.x * blockDim.x * 8;
    for (size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; idx < total; idx += step) {
        const size_t n = idx / inter;
        const int i = (int)(idx - n * inter);
        const size_t at = n * 2 * inter + (size_t)(i / block) * 2 * block + (i % block);
        const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + at), uv = *reinterpret_cast<const uint4*>(gate_up + at + block);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            o2[j] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + idx) = ov;
    }
}

// ---------------------------------------------------------------------------- q/k norm + rotary + cache write

// grid (tokens, ceil(heads / 4)), block (32, 4): one warp per (token, head) of the fused
// projection [q heads | k heads | v heads].  q heads go to q_out, k and v heads into the
// token's place in its page.
template <typename T, typename W, typename IN, int VEC>
__global__ void qk_norm_rope_write_kernel(const Summed<IN> qkv, const W* __restrict__ q_gain,
                                          const W* __restrict__ k_gain, float eps,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          const int* __restrict__ positions, const int* __restrict__ token_req,
                                          const int* __restrict__ block_table, int bt_stride,
                                          T* __restrict__ kv_layer, T* __restrict__ q_out,
                                          int nq, int nkv, int d, int rd, int page_size, int write_kv) {
    pdl_enter_small();
    const int n = blockIdx.x;
    const int head = blockIdx.y * blockDim.y + threadIdx.y;
    const int nheads = write_kv ? nq + 2 * nkv : nq;
    if (head >= nheads) return;
    const int lane = threadIdx.x;
    const int pos = positions[n];
    const size_t src = (size_t)n * (nq + 2 * nkv) * d + (size_t)head * d;
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
    if (VEC == 2) {
        // two neighbouring features per lane and step (d, the rotary width and its half are even)
        if (gain) {
            float ssq = 0.f;
            for (int i = 2 * lane; i < d; i += 64) {
                const float2 x = qkv.two(src + i);
                ssq += x.x * x.x + x.y * x.y;
            }
            inv = rsqrtf(warp_sum(ssq) / (float)d + eps);
        }
        if (!rotate) {
            for (int i = 2 * lane; i < d; i += 64) store2(dst, i, qkv.two(src + i));
            return;
        }
        const int half = rd >> 1;
        for (int i = 2 * lane; i < half; i += 64) {
            float2 x1 = qkv.two(src + i), x2 = qkv.two(src + i + half);
            if (gain) {
                const float2 g1 = load2(gain, i), g2 = load2(gain, i + half);
                x1 = make_float2((x1.x * inv) * g1.x, (x1.y * inv) * g1.y);
                x2 = make_float2((x2.x * inv) * g2.x, (x2.y * inv) * g2.y);
            }
            float2 o1 = x1, o2 = x2;
            if (cos_t) {
                const float2 cc = load2(cos_t, (size_t)pos * half + i), ss = load2(sin_t, (size_t)pos * half + i);
                o1 = make_float2(x1.x * cc.x - x2.x * ss.x, x1.y * cc.y - x2.y * ss.y);
                o2 = make_float2(x2.x * cc.x + x1.x * ss.x, x2.y * cc.y + x1.y * ss.y);
            }
            store2(dst, i, o1);
            store2(dst, i + half, o2);
        }
        for (int i = rd + 2 * lane; i < d; i += 64) {
            float2 x = qkv.two(src + i);
            if (gain) {
                const float2 gg = load2(gain, i);
                x = make_float2((x.x * inv) * gg.x, (x.y * inv) * gg.y);
            }
            store2(dst, i, x);
        }
        return;
    }
    if (gain) {
        float ssq = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float x = qkv(src + i);
            ssq += x * x;
        }
        ssq = warp_sum(ssq);
        inv = rsqrtf(ssq / (float)d + eps);
    }
    if (!rotate) {
        for (int i = lane; i < d; i += 32) dst[i] = from_float<T>(qkv(src + i));
        return;
    }
    const int half = rd >> 1;
    const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* s = sin_t ? sin_t + (size_t)pos * half : nullptr;
    for (int i = lane; i < half; i += 32) {
        float x1 = qkv(src + i), x2 = qkv(src + i + half);
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
        float x = qkv(src + i);
        if (gain) x = (x * inv) * to_float(gain[i]);
        dst[i] = from_float<T>(x);
    }
}

// The same work for bfloat16 in and out with 16-byte accesses, for many tokens: G = head_dim / 16
// threads share a head (G a power of two, at most 32), each holding eight features of the first
// half and the matching eight of the second, so the rotation needs no exchange and the norm's
// sum of squares takes log2(G) shuffles.  The whole head is rotated (rotary width == head_dim).
// grid (tokens, ceil(heads / (128 / G))), block 128.
template <typename W>
__global__ void qk_norm_rope_write_wide_kernel(const __nv_bfloat16* __restrict__ qkv, const W* __restrict__ q_gain,
                                               const W* __restrict__ k_gain, float eps,
                                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                               const int* __restrict__ positions, const int* __restrict__ token_req,
                                               const int* __restrict__ block_table, int bt_stride,
                                               __nv_bfloat16* __restrict__ kv_layer, __nv_bfloat16* __restrict__ q_out,
                                               int nq, int nkv, int d, int group, int page_size, int write_kv) {
    pdl_enter_small();
    const int n = blockIdx.x;
    const int per_block = blockDim.x / group;
    const int head = blockIdx.y * per_block + threadIdx.x / group;
    const int j = threadIdx.x % group;
    const int nheads = write_kv ? nq + 2 * nkv : nq;
    const bool valid = head < nheads;
    const int half = d >> 1;
    const int pos = positions[n];
    __nv_bfloat16* dst = nullptr;
    const W* gain = nullptr;
    bool rotate = true;
    float a[8], b[8];
    uint4 ra = make_uint4(0, 0, 0, 0), rb = ra;
    if (valid) {
        const __nv_bfloat16* src = qkv + ((size_t)n * (nq + 2 * nkv) + head) * d;
        ra = *reinterpret_cast<const uint4*>(src + 8 * j);
        rb = *reinterpret_cast<const uint4*>(src + half + 8 * j);
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
    }
    if (valid && !rotate) {
        *reinterpret_cast<uint4*>(dst + 8 * j) = ra;
        *reinterpret_cast<uint4*>(dst + half + 8 * j) = rb;
    }
    {
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&rb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
            a[2 * i] = fa.x; a[2 * i + 1] = fa.y;
            b[2 * i] = fb.x; b[2 * i + 1] = fb.y;
        }
    }
    float ssq = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ssq += a[i] * a[i] + b[i] * b[i];
    for (int o = group >> 1; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    if (!valid || !rotate) return;
    if (gain) {
        const float inv = rsqrtf(ssq / (float)d + eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            a[i] = (a[i] * inv) * to_float(gain[8 * j + i]);
            b[i] = (b[i] * inv) * to_float(gain[half + 8 * j + i]);
        }
    }
    if (cos_t) {
        const float4* c4 = reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + 8 * j);
        const float4* s4 = reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + 8 * j);
        const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x1 = a[i], x2 = b[i];
            a[i] = x1 * c[i] - x2 * s[i];
            b[i] = x2 * c[i] + x1 * s[i];
        }
    }
    uint4 oa, ob;
    __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
    __nv_bfloat162* qb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        qa[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
        qb[i] = __floats2bfloat162_rn(b[2 * i], b[2 * i + 1]);
    }
    *reinterpret_cast<uint4*>(dst + 8 * j) = oa;
    *reinterpret_cast<uint4*>(dst + half + 8 * j) = ob;
}

// ---------------------------------------------------------------------------- casts

template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ in, B* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_float<B>(to_float(in[i]));
}

}  // namespace lily

using namespace lily;

static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

LILY_API const char* lily_last_error() { return g_error; }

// Streaming multiprocessors of the current device.
LILY_API int lily_sm_count() { return sm_count(); }

LILY_API int lily_logit_transform(float* logits, size_t n, float scale, float cap, cudaStream_t stream) {
    if (n == 0) return 0;
    const size_t blocks = (n + 255) / 256;
    logit_transform_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, stream>>>(logits, n, scale, cap);
    LILY_CHECK_LAUNCH("logit_transform");
    return 0;
}

LILY_API int lily_embed(const void* table, int table_dtype, const int* ids, const int* future, float* out, int tokens,
                        int hidden, int vocab, float scale, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(hidden > 0 && vocab > 0, "embed: bad sizes hidden=%d vocab=%d", hidden, vocab);
    const bool vec = hidden % 4 == 0 && aligned16(table) && aligned16(out);
    if (table_dtype == kBF16) {
        if (vec) launch_pdl(embed_kernel<__nv_bfloat16, 4>, dim3(tokens), dim3(256), 0, stream, (const __nv_bfloat16*)table, ids, future, out, hidden, vocab, scale);
        else launch_pdl(embed_kernel<__nv_bfloat16, 1>, dim3(tokens), dim3(256), 0, stream, (const __nv_bfloat16*)table, ids, future, out, hidden, vocab, scale);
    } else {
        if (vec) launch_pdl(embed_kernel<float, 4>, dim3(tokens), dim3(256), 0, stream, (const float*)table, ids, future, out, hidden, vocab, scale);
        else launch_pdl(embed_kernel<float, 1>, dim3(tokens), dim3(256), 0, stream, (const float*)table, ids, future, out, hidden, vocab, scale);
    }
    LILY_CHECK_LAUNCH("embed");
    return 0;
}

LILY_API int lily_scatter_tokens(const int* tokens, const int* logit_rows, const int* token_req, const int* slots,
                                 int* future, int n, int max_slots, cudaStream_t stream) {
    if (n == 0) return 0;
    LILY_REQUIRE(n > 0 && max_slots > 0, "scatter_tokens: n=%d max_slots=%d", n, max_slots);
    scatter_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, logit_rows, token_req, slots, future, n, max_slots);
    LILY_CHECK_LAUNCH("scatter_tokens");
    return 0;
}

// `in_dtype` is the dtype of the summed input (delta, gate_up, qkv): the activation dtype with one
// split, or float32 partial sums with `splits` slices `stride` elements apart.
template <typename T, typename W, typename IN>
static void launch_add_rmsnorm(float* resid, const void* delta, int splits, size_t stride, const void* weight, void* out,
                               const int* rows, int out_rows, int hidden, float eps, int write_residual,
                               cudaStream_t stream) {
    const int stash = hidden <= 11264;   // 40 + hidden floats stay within 48 KB
    const size_t smem = (40 + (stash ? hidden : 0)) * sizeof(float);
    const bool vec = hidden % 4 == 0 && stride % 4 == 0 && aligned16(resid) && aligned16(delta) && aligned16(weight) && aligned16(out);
    const int per = vec ? 4 : 1;
    const int threads = hidden >= 2048 * per ? 512 : (hidden >= 1024 * per ? 256 : 128);
    const Summed<IN> d{(const IN*)delta, splits, stride};
    constexpr int CL = 8;
    if (vec && out_rows <= 64 && hidden % (4 * CL) == 0 && hidden / (4 * CL) >= 32 && hidden / (4 * CL) <= 1024) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(CL, out_rows);
        cfg.blockDim = dim3(hidden / (4 * CL));
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        cudaLaunchKernelEx(&cfg, add_rmsnorm_cluster_kernel<T, W, IN, CL>, resid, d, (const W*)weight, (T*)out, rows, hidden, eps,
                           write_residual);
        return;
    }
    if (vec)
        launch_pdl(add_rmsnorm_kernel<T, W, IN, 4>, dim3(out_rows), dim3(threads), smem, stream, resid, d, (const W*)weight, (T*)out, rows, hidden, eps, write_residual, stash);
    else
        launch_pdl(add_rmsnorm_kernel<T, W, IN, 1>, dim3(out_rows), dim3(threads), smem, stream, resid, d, (const W*)weight, (T*)out, rows, hidden, eps, write_residual, stash);
}

static int check_summed(const char* name, int act_dtype, int in_dtype, int splits) {
    LILY_REQUIRE(splits >= 1, "%s: %d splits", name, splits);
    LILY_REQUIRE(in_dtype == act_dtype || in_dtype == kF32, "%s: the input is the activation dtype or float32 partial sums", name);
    LILY_REQUIRE(splits == 1 || in_dtype == kF32, "%s: only float32 partial sums come in several splits", name);
    return 0;
}

LILY_API int lily_add_rmsnorm(float* resid, const void* delta, const void* weight, void* out, const int* rows,
                              int out_rows, int hidden, float eps, int write_residual, int act_dtype,
                              int weight_dtype, int delta_dtype, int delta_splits, size_t delta_stride,
                              cudaStream_t stream) {
    if (out_rows == 0) return 0;
    LILY_REQUIRE(hidden > 0, "add_rmsnorm: hidden=%d", hidden);
    LILY_REQUIRE(!(rows && write_residual && delta), "add_rmsnorm: gathered rows cannot write the residual back");
    if (check_summed("add_rmsnorm", act_dtype, delta_dtype, delta_splits)) return 1;
#define GO(T, W, IN) launch_add_rmsnorm<T, W, IN>(resid, delta, delta_splits, delta_stride, weight, out, rows, out_rows, hidden, eps, write_residual, stream)
    const bool wb = weight_dtype == kBF16, ib = delta_dtype == kBF16;
    if (act_dtype == kBF16) {
        if (wb && ib) GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
        else if (wb) GO(__nv_bfloat16, __nv_bfloat16, float);
        else if (ib) GO(__nv_bfloat16, float, __nv_bfloat16);
        else GO(__nv_bfloat16, float, float);
    } else {
        if (wb) GO(float, __nv_bfloat16, float);
        else GO(float, float, float);
    }
#undef GO
    LILY_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

LILY_API int lily_silu_mul(const void* gate_up, void* out, int tokens, int inter, int block, int act_dtype,
                           int in_dtype, int splits, size_t stride, cudaStream_t stream) {
    const size_t total = (size_t)tokens * inter;
    if (total == 0) return 0;
    LILY_REQUIRE(block > 0 && inter % block == 0, "silu_mul: gate/up runs of %d do not tile %d columns", block, inter);
    if (check_summed("silu_mul", act_dtype, in_dtype, splits)) return 1;
    const bool vec = block % 4 == 0 && stride % 4 == 0 && aligned16(gate_up) && aligned16(out);
    const size_t work = vec ? total / 4 : total;
    const int blocks = (int)((work + 255) / 256 < sm_count() * 16 ? (work + 255) / 256 : sm_count() * 16);
#define GO(T, IN, V) launch_pdl(silu_mul_kernel<T, IN, V>, dim3(blocks), dim3(256), 0, stream, Summed<IN>{(const IN*)gate_up, splits, stride}, (T*)out, inter, block, total)
    if (act_dtype == kBF16 && in_dtype == kBF16 && splits == 1 && block % 8 == 0 && aligned16(gate_up) && aligned16(out)) {
        const size_t work8 = total / 8;
        const int blocks8 = (int)((work8 + 255) / 256 < (size_t)sm_count() * 16 ? (work8 + 255) / 256 : (size_t)sm_count() * 16);
        launch_pdl(silu_mul_bf16x8_kernel, dim3(blocks8), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block, total);
    } else if (act_dtype == kBF16 && in_dtype == kBF16) { if (vec) GO(__nv_bfloat16, __nv_bfloat16, 4); else GO(__nv_bfloat16, __nv_bfloat16, 1); }
    else if (act_dtype == kBF16) { if (vec) GO(__nv_bfloat16, float, 4); else GO(__nv_bfloat16, float, 1); }
    else { if (vec) GO(float, float, 4); else GO(float, float, 1); }
#undef GO
    LILY_CHECK_LAUNCH("silu_mul");
    return 0;
}

LILY_API int lily_qk_norm_rope_write(const void* qkv, const void* q_gain, const void* k_gain, float eps,
                                     const float* cos_t, const float* sin_t, const int* positions,
                                     const int* token_req, const int* block_table, int bt_stride, void* kv_layer,
                                     void* q_out, int tokens, int nq, int nkv, int d, int rd, int page_size,
                                     int write_kv, int act_dtype, int gain_dtype, int in_dtype, int splits,
                                     size_t stride, cudaStream_t stream) {
    if (tokens == 0) return 0;
    LILY_REQUIRE(d > 0 && rd >= 0 && rd <= d && rd % 2 == 0, "qk_norm_rope_write: rotary_dim %d does not fit head_dim %d", rd, d);
    LILY_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "qk_norm_rope_write: q and k gains come together");
    LILY_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "qk_norm_rope_write: cos and sin tables come together");
    if (check_summed("qk_norm_rope_write", act_dtype, in_dtype, splits)) return 1;
    const int nheads = write_kv ? nq + 2 * nkv : nq;
    dim3 grid(tokens, (nheads + 3) / 4), block(32, 4);
    const int rot = cos_t ? rd : 0;
    const bool vec = d % 2 == 0 && rot % 4 == 0 && stride % 2 == 0 && aligned16(qkv) && aligned16(kv_layer) &&
                     aligned16(q_out) && aligned16(q_gain) && aligned16(k_gain) && aligned16(cos_t) && aligned16(sin_t);
#define LAUNCH_V(T, W, IN, V)                                                                                     \
    launch_pdl(qk_norm_rope_write_kernel<T, W, IN, V>, grid, block, 0, stream, Summed<IN>{(const IN*)qkv, splits, stride}, \
        (const W*)q_gain, (const W*)k_gain, eps, cos_t, sin_t, positions, token_req, block_table, bt_stride,      \
        (T*)kv_layer, (T*)q_out, nq, nkv, d, rot, page_size, write_kv)
#define LAUNCH(T, W, IN) do { if (vec) LAUNCH_V(T, W, IN, 2); else LAUNCH_V(T, W, IN, 1); } while (0)
    const bool gb = gain_dtype == kBF16, ib = in_dtype == kBF16;
    const int group = d / 16;
    if (act_dtype == kBF16 && ib && splits == 1 && d % 16 == 0 && group <= 32 && (group & (group - 1)) == 0 &&
        (rot == d || rot == 0) && aligned16(qkv) && aligned16(kv_layer) && aligned16(q_out) && aligned16(q_gain) &&
        aligned16(k_gain) && aligned16(cos_t) && aligned16(sin_t)) {
        const int per_block = 128 / group;
        dim3 wgrid(tokens, (nheads + per_block - 1) / per_block);
        if (gb)
            launch_pdl(qk_norm_rope_write_wide_kernel<__nv_bfloat16>, wgrid, dim3(128), 0, stream, (const __nv_bfloat16*)qkv,
                       (const __nv_bfloat16*)q_gain, (const __nv_bfloat16*)k_gain, eps, cos_t, sin_t, positions, token_req,
                       block_table, bt_stride, (__nv_bfloat16*)kv_layer, (__nv_bfloat16*)q_out, nq, nkv, d, group, page_size, write_kv);
        else
            launch_pdl(qk_norm_rope_write_wide_kernel<float>, wgrid, dim3(128), 0, stream, (const __nv_bfloat16*)qkv,
                       (const float*)q_gain, (const float*)k_gain, eps, cos_t, sin_t, positions, token_req,
                       block_table, bt_stride, (__nv_bfloat16*)kv_layer, (__nv_bfloat16*)q_out, nq, nkv, d, group, page_size, write_kv);
        LILY_CHECK_LAUNCH("qk_norm_rope_write");
        return 0;
    }
    if (act_dtype == kBF16) {
        if (gb && ib) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
        else if (gb) LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
        else if (ib) LAUNCH(__nv_bfloat16, float, __nv_bfloat16);
        else LAUNCH(__nv_bfloat16, float, float);
    } else {
        if (gb) LAUNCH(float, __nv_bfloat16, float);
        else LAUNCH(float, float, float);
    }
#undef LAUNCH
#undef LAUNCH_V
    LILY_CHECK_LAUNCH("qk_norm_rope_write");
    return 0;
}

LILY_API int lily_cast(const void* in, int in_dtype, void* out, int out_dtype, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 < sm_count() * 16 ? (n + 255) / 256 : sm_count() * 16);
    if (in_dtype == kBF16 && out_dtype == kF32)
        cast_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, n);
    else if (in_dtype == kF32 && out_dtype == kBF16)
        cast_kernel<<<blocks, 256, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, n);
    else
        LILY_REQUIRE(false, "cast: unsupported pair %d -> %d", in_dtype, out_dtype);
    LILY_CHECK_LAUNCH("cast");
    return 0;
}
