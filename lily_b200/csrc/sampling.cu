// Sampling over float32 logits [rows, vocab]: penalties and bias, argmax, and temperature
// sampling with top-k, top-p and min-p, one block per row, no sort.
//
// Order of operations as in lily/layers/sampler.py:1-12,64-116: (1) repetition, frequency and
// presence penalties and the additive bias on the logits; (2) argmax for a greedy row;
// (3) x = logit / max(T, 1e-5); (4) keep the top_k largest, softmax over them, keep the sorted
// prefix whose mass before each member is < top_p, drop what is below min_p * max, renormalise;
// (5) draw.  The draw is the engine's own: the first token in vocabulary order whose cumulative
// probability exceeds u, u in [0, 1) supplied per row by the host from a counter-based generator
// keyed by (seed, request, step), so a request's tokens do not depend on what else is in the batch
// (the reference gets the same from per-request torch generators, lily/scheduler/scheduler.py:237).
//
// The k-th largest value and the top-p cut are found by radix selection over the order-preserving
// bit pattern of x (4 passes of 8 bits); masses are summed in 2^-40 fixed point so that every
// sum is independent of the order in which threads add.
#include "common.cuh"

namespace lily {

constexpr int STHREADS = 1024;
constexpr double FIXED_ONE = 1099511627776.0;   // 2^40

__device__ __forceinline__ unsigned ordered_key(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long to_fixed(float e) {
    return (unsigned long long)((double)e * FIXED_ONE);
}

struct ArgBest {
    float v;
    int i;
};
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ ArgBest block_argmax(const float* row, int vocab, float tdiv, ArgBest* scratch) {
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgBest{row[i] / tdiv, i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    if (warp == 0) {
        ArgBest t = lane < nwarp ? scratch[lane] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgBest other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
            t = better(t, other);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__global__ void __launch_bounds__(STHREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ ArgBest scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const ArgBest b = block_argmax(logits + (size_t)blockIdx.x * vocab, vocab, 1.f, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = b.i < vocab ? b.i : 0;
}

// Large vocabularies: a row is cut into `chunks` ranges, one block each, whose best (value, index)
// go to `partial`; argmax_merge_kernel then picks the best of a row (ties go to the lower index).
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, float* __restrict__ partial_v, int* __restrict__ partial_i,
                      int vocab, int chunks) {
    __shared__ ArgBest scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x, c = blockIdx.y;
    const int per = (vocab + chunks - 1) / chunks;
    const int lo = c * per, hi = min(vocab, lo + per);
    const float* src = logits + (size_t)row * vocab;
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) best = better(best, ArgBest{src[i], i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    if (warp == 0) {
        ArgBest t = lane < (int)(blockDim.x >> 5) ? scratch[lane] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgBest other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
            t = better(t, other);
        }
        if (lane == 0) {
            partial_v[row * chunks + c] = t.v;
            partial_i[row * chunks + c] = t.i;
        }
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ partial_v, const int* __restrict__ partial_i,
                                    int* __restrict__ out, int vocab, int chunks) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x, lane = threadIdx.x;
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int c = lane; c < chunks; c += 32) best = better(best, ArgBest{partial_v[row * chunks + c], partial_i[row * chunks + c]});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (lane == 0) out[row] = best.i < vocab ? best.i : 0;
}

// One entry per (row, token) that some request has seen or biases.
__global__ void penalties_kernel(float* __restrict__ logits, const int* __restrict__ entry_row,
                                 const int* __restrict__ entry_token, const int* __restrict__ entry_count,
                                 const float* __restrict__ entry_bias, const float* __restrict__ repetition,
                                 const float* __restrict__ frequency, const float* __restrict__ presence,
                                 int entries, int vocab) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= entries) return;
    const int r = entry_row[e], t = entry_token[e], c = entry_count[e];
    if (t < 0 || t >= vocab) return;
    float v = logits[(size_t)r * vocab + t];
    if (c > 0) {
        const float rep = repetition[r];
        if (rep != 1.f) v = v > 0.f ? v / rep : v * rep;
        v -= (float)c * frequency[r];
        v -= presence[r];
    }
    v += entry_bias[e];
    logits[(size_t)r * vocab + t] = v;
}

// Radix selection over ordered keys among elements with key >= floor_key.
//   by count: the k-th largest key.
//   by mass:  the smallest key whose mass of strictly larger keys is < limit.
template <bool BY_MASS>
__device__ unsigned radix_select(const float* row, int vocab, float tdiv, float mx, unsigned floor_key,
                                 unsigned long long limit, unsigned* cnt, unsigned long long* mass,
                                 unsigned* pick) {
    unsigned prefix = 0, prefix_mask = 0;
    unsigned long long above = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            cnt[b] = 0;
            mass[b] = 0;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float x = row[i] / tdiv;
            const unsigned key = ordered_key(x);
            if (key < floor_key || (key & prefix_mask) != prefix) continue;
            const unsigned bin = (key >> shift) & 255u;
            atomicAdd(&cnt[bin], 1u);
            if (BY_MASS) atomicAdd(&mass[bin], to_fixed(expf(x - mx)));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long run = above, chosen_above = above;
            int chosen = -1;
            for (int b = 255; b >= 0; --b) {
                if (!cnt[b]) continue;
                if (BY_MASS) {
                    // the lowest non-empty bin with less than `limit` of mass strictly above it
                    if (run >= limit && chosen >= 0) break;
                    chosen = b;
                    chosen_above = run;
                    run += mass[b];
                } else {
                    // the bin that holds the limit-th largest key
                    chosen = b;
                    chosen_above = run;
                    if (run + cnt[b] >= limit) break;
                    run += cnt[b];
                }
            }
            pick[1] = (unsigned)(chosen_above >> 32);
            pick[2] = (unsigned)chosen_above;
            pick[0] = (unsigned)(chosen < 0 ? 0 : chosen);
        }
        __syncthreads();
        prefix |= pick[0] << shift;
        prefix_mask |= 255u << shift;
        above = ((unsigned long long)pick[1] << 32) | pick[2];
        __syncthreads();
    }
    return prefix;
}

__global__ void __launch_bounds__(STHREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, int* __restrict__ out_token, float* __restrict__ out_logprob,
              int vocab) {
    __shared__ ArgBest abest[33];
    __shared__ float fred[33];
    __shared__ unsigned cnt[256];
    __shared__ unsigned long long mass[256];
    __shared__ unsigned pick[4];
    __shared__ unsigned long long chunk_sum[STHREADS];
    __shared__ unsigned long long total_s;
    __shared__ int last_kept_s;

    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const float temp = temperature[r];
    const int k = top_k[r];
    const bool greedy = temp == 0.f || k == 1;

    if (greedy) {
        const ArgBest b = block_argmax(row, vocab, 1.f, abest);
        float s = 0.f;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) s += expf(row[i] - b.v);
        s = block_sum(s, fred);
        if (threadIdx.x == 0) {
            out_token[r] = b.i < vocab ? b.i : 0;
            if (out_logprob) out_logprob[r] = -logf(s);
        }
        return;
    }

    const float tdiv = fmaxf(temp, 1e-5f);   // the divisor: x = logit / max(T, 1e-5)
    const ArgBest top = block_argmax(row, vocab, tdiv, abest);
    const float mx = top.v;

    unsigned floor_key = 0;
    if (k > 0 && k < vocab)
        floor_key = radix_select<false>(row, vocab, tdiv, mx, 0u, (unsigned long long)k, cnt, mass, pick);

    const float p = top_p[r];
    if (p < 1.f) {
        // mass of the top-k survivors, then the cut
        unsigned long long z = 0;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float x = row[i] / tdiv;
            if (ordered_key(x) >= floor_key) z += to_fixed(expf(x - mx));
        }
        if (threadIdx.x == 0) total_s = 0;
        __syncthreads();
        atomicAdd(&total_s, z);
        __syncthreads();
        const unsigned long long limit = (unsigned long long)((double)p * (double)total_s);
        const unsigned cut = radix_select<true>(row, vocab, tdiv, mx, floor_key, limit > 0 ? limit : 1ull, cnt, mass, pick);
        floor_key = max(floor_key, cut);
    }
    const float mp = min_p[r];

    // kept mass per contiguous chunk of the vocabulary, then the draw in vocabulary order
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * chunk, hi = min(vocab, lo + chunk);
    unsigned long long mine = 0;
    int my_last = -1;
    for (int i = lo; i < hi; ++i) {
        const float x = row[i] / tdiv;
        const float e = expf(x - mx);
        if (ordered_key(x) >= floor_key && e >= mp) {
            mine += to_fixed(e);
            my_last = i;
        }
    }
    chunk_sum[threadIdx.x] = mine;
    if (threadIdx.x == 0) { total_s = 0; last_kept_s = -1; }
    __syncthreads();
    atomicAdd(&total_s, mine);
    atomicMax(&last_kept_s, my_last);
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long total = total_s;
        unsigned long long target = (unsigned long long)((double)uniform[r] * (double)total);
        if (target >= total) target = total ? total - 1 : 0;
        unsigned long long run = 0;
        int t = 0;
        for (; t < (int)blockDim.x - 1; ++t) {
            if (run + chunk_sum[t] > target) break;
            run += chunk_sum[t];
        }
        int token = last_kept_s < 0 ? top.i : last_kept_s;
        float chosen_e = 0.f;
        const int clo = t * chunk, chi = min(vocab, clo + chunk);
        for (int i = clo; i < chi; ++i) {
            const float x = row[i] / tdiv;
            const float e = expf(x - mx);
            if (ordered_key(x) >= floor_key && e >= mp) {
                run += to_fixed(e);
                if (run > target) { token = i; chosen_e = e; break; }
            }
        }
        if (chosen_e == 0.f) chosen_e = expf(row[token] / tdiv - mx);
        out_token[r] = token;
        if (out_logprob) out_logprob[r] = logf(chosen_e) - logf((float)((double)total / FIXED_ONE));
    }
}

}  // namespace lily

using namespace lily;

// Ranges a row is cut into (1: the single-block kernel); the caller provides scratch of
// rows * chunks floats and as many ints when it is more than 1.
LILY_API int lily_argmax_chunks(int rows, int vocab) {
    if (vocab < 16384) return 1;
    int chunks = (148 * 4 + rows - 1) / (rows > 0 ? rows : 1);
    const int most = vocab / 2048;
    chunks = chunks > most ? most : chunks;
    return chunks < 1 ? 1 : (chunks > 256 ? 256 : chunks);
}

LILY_API int lily_argmax(const float* logits, int* out, float* partial_v, int* partial_i, int rows, int vocab,
                         cudaStream_t stream) {
    if (rows == 0) return 0;
    LILY_REQUIRE(vocab > 0, "argmax: vocab=%d", vocab);
    const int chunks = lily_argmax_chunks(rows, vocab);
    if (chunks <= 1 || partial_v == nullptr || partial_i == nullptr) {
        launch_pdl(argmax_kernel, dim3(rows), dim3(STHREADS), 0, stream, logits, out, vocab);
    } else {
        launch_pdl(argmax_partial_kernel, dim3(rows, chunks), dim3(256), 0, stream, logits, partial_v, partial_i, vocab, chunks);
        launch_pdl(argmax_merge_kernel, dim3(rows), dim3(32), 0, stream, (const float*)partial_v, (const int*)partial_i, out, vocab, chunks);
    }
    LILY_CHECK_LAUNCH("argmax");
    return 0;
}

LILY_API int lily_apply_penalties(float* logits, const int* entry_row, const int* entry_token,
                                  const int* entry_count, const float* entry_bias, const float* repetition,
                                  const float* frequency, const float* presence, int entries, int vocab,
                                  cudaStream_t stream) {
    if (entries == 0) return 0;
    penalties_kernel<<<(entries + 255) / 256, 256, 0, stream>>>(logits, entry_row, entry_token, entry_count, entry_bias,
                                                                repetition, frequency, presence, entries, vocab);
    LILY_CHECK_LAUNCH("apply_penalties");
    return 0;
}

LILY_API int lily_sample(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                         const float* min_p, const float* uniform, int* out_token, float* out_logprob, int rows,
                         int vocab, cudaStream_t stream) {
    if (rows == 0) return 0;
    LILY_REQUIRE(vocab > 0, "sample: vocab=%d", vocab);
    sample_kernel<<<rows, STHREADS, 0, stream>>>(logits, temperature, top_k, top_p, min_p, uniform, out_token,
                                                 out_logprob, vocab);
    LILY_CHECK_LAUNCH("sample");
    return 0;
}
