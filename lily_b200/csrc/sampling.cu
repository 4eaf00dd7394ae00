// Sampling over float32 logits [rows, vocab]: penalties and bias, argmax, and temperature
// sampling with top-k, top-p and min-p, one block (small vocabularies) or a cluster of eight blocks
// per row, no sort.
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

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

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

// ---- temperature sampling: a thread-block cluster per row -----------------------------------------
//
// A row of a large vocabulary is cut into CL contiguous slices, one block of the cluster each; what
// the blocks find out about their slices (best value, histograms, masses) they leave in their own
// shared memory, and after a cluster barrier every block reads all of them through distributed
// shared memory and combines them in rank order, so all blocks reach the same decision without a
// broadcast.  CL == 1 is the same code without a cluster (small vocabularies).

template <int CL>
struct RowShared {
    ArgBest best[33];
    float fsum[33];
    ArgBest cbest;                      // this block's best, for the others to read
    float csum;                         // ... its sum of exponentials (greedy log-probability)
    unsigned long long ctotal;          // ... its mass of top-k survivors
    unsigned cnt[2][256];               // histograms of the radix passes, double-buffered by pass
    unsigned long long mass[2][256];
    unsigned tcnt[256];                 // the cluster's totals of the current pass
    unsigned long long tmass[256];
    unsigned pick[4];
    unsigned long long wsum[32];        // kept mass of each warp's segment
    unsigned long long all_wsum[CL * 32];
};

template <int CL, typename T>
__device__ __forceinline__ const T* peer(cg::cluster_group& cluster, const T* mine, int rank) {
    if (CL == 1) return mine;
    return cluster.map_shared_rank(const_cast<T*>(mine), rank);
}
template <int CL>
__device__ __forceinline__ void cluster_barrier(cg::cluster_group& cluster) {
    if (CL == 1) __syncthreads();
    else cluster.sync();
}

// Radix selection over ordered keys among the row's elements with key >= floor_key.
//   by count: the k-th largest key.
//   by mass:  the smallest key whose mass of strictly larger keys is < limit.
// `pass` counts the radix passes of the kernel so far (it picks the histogram buffer).
// x of element i of the row: from the block's copy in shared memory when the slice fits there.
struct RowX {
    const float* row;
    const float* cached;    // x of [v0, v1), or null
    int v0;
    float tdiv;
    __device__ __forceinline__ float operator()(int i) const { return cached ? cached[i - v0] : row[i] / tdiv; }
};

template <int CL, bool BY_MASS>
__device__ unsigned radix_select(cg::cluster_group& cluster, RowShared<CL>& sh, const RowX& xs, int v0, int v1,
                                 float mx, unsigned floor_key, unsigned long long limit, int& pass) {
    unsigned prefix = 0, prefix_mask = 0;
    unsigned long long above = 0;
    const int lane = threadIdx.x & 31;
    for (int shift = 24; shift >= 0; shift -= 8, ++pass) {
        unsigned* cnt = sh.cnt[pass & 1];
        unsigned long long* mass = sh.mass[pass & 1];
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            cnt[b] = 0;
            mass[b] = 0;
        }
        __syncthreads();
        for (int base = v0; base < v1; base += blockDim.x) {
            const int i = base + threadIdx.x;
            bool act = false;
            unsigned bin = 0;
            unsigned long long m = 0;
            if (i < v1) {
                const float x = xs(i);
                const unsigned key = ordered_key(x);
                if (key >= floor_key && (key & prefix_mask) == prefix) {
                    act = true;
                    bin = (key >> shift) & 255u;
                    if (BY_MASS) m = to_fixed(expf(x - mx));
                }
            }
            if (shift == 24) {
                // On the first pass nearly every key falls into a handful of bins (sign and exponent): a
                // warp adds up what its lanes bring for the same bin before it touches shared memory.
                unsigned pending = __ballot_sync(0xffffffffu, act);
                while (pending) {
                    const int leader = __ffs(pending) - 1;
                    const unsigned b0 = __shfl_sync(0xffffffffu, bin, leader);
                    const bool mine = act && bin == b0;
                    const unsigned same = __ballot_sync(0xffffffffu, mine);
                    if (BY_MASS) {
                        unsigned long long v = mine ? m : 0ull;
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                        if (lane == leader) atomicAdd(&mass[b0], v);
                    }
                    if (lane == leader) atomicAdd(&cnt[b0], (unsigned)__popc(same));
                    pending &= ~same;
                }
            } else if (act) {
                atomicAdd(&cnt[bin], 1u);
                if (BY_MASS) atomicAdd(&mass[bin], m);
            }
        }
        cluster_barrier<CL>(cluster);                   // every block's histogram of this pass is complete
        for (int b = threadIdx.x; b < 256; b += blockDim.x) {
            unsigned c = 0;
            unsigned long long ms = 0;
            for (int rk = 0; rk < CL; ++rk) {
                c += peer<CL>(cluster, cnt, rk)[b];
                if (BY_MASS) ms += peer<CL>(cluster, mass, rk)[b];
            }
            sh.tcnt[b] = c;
            sh.tmass[b] = ms;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // Lane l owns bins [8 l, 8 l + 8).  w(b) = what bin b weighs (its count, or its mass); S(b) = above +
            // the weight of all higher bins.  By count the answer is the bin with S < limit <= S + w; by
            // mass the lowest non-empty bin with S < limit, or the highest non-empty bin when there is none.
            unsigned long long w[8], mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                w[j] = BY_MASS ? sh.tmass[8 * lane + j] : (unsigned long long)sh.tcnt[8 * lane + j];
                mine += w[j];
            }
            unsigned long long higher = mine;              // inclusive sum over lanes >= this one
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long up = __shfl_down_sync(0xffffffffu, higher, o);
                if (lane + o < 32) higher += up;
            }
            unsigned long long s_above = above + higher - mine;     // S of this lane's highest bin
            int found = -1, top_nonempty = -1;
            unsigned long long found_above = 0, top_above = 0;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                const int b = 8 * lane + j;
                if (sh.tcnt[b]) {
                    if (top_nonempty < 0) { top_nonempty = b; top_above = s_above; }
                    const bool ok = BY_MASS ? s_above < limit : (s_above < limit && limit <= s_above + w[j]);
                    if (ok && (BY_MASS || found < 0)) { found = b; found_above = s_above; }    // by mass: the lowest wins
                }
                s_above += w[j];
            }
            // across lanes: by mass the lowest found bin, by count the only one; else the highest non-empty bin
            unsigned has = __ballot_sync(0xffffffffu, found >= 0);
            int src;
            if (has) {
                src = BY_MASS ? __ffs(has) - 1 : 31 - __clz(has);
            } else {
                has = __ballot_sync(0xffffffffu, top_nonempty >= 0);
                src = has ? 31 - __clz(has) : 0;
                found = top_nonempty;
                found_above = top_above;
            }
            const int chosen = __shfl_sync(0xffffffffu, found, src);
            const unsigned long long chosen_above = __shfl_sync(0xffffffffu, found_above, src);
            if (lane == 0) {
                sh.pick[0] = (unsigned)(chosen < 0 ? 0 : chosen);
                sh.pick[1] = (unsigned)((chosen < 0 ? above : chosen_above) >> 32);
                sh.pick[2] = (unsigned)(chosen < 0 ? above : chosen_above);
            }
        }
        __syncthreads();
        prefix |= sh.pick[0] << shift;
        prefix_mask |= 255u << shift;
        above = ((unsigned long long)sh.pick[1] << 32) | sh.pick[2];
        __syncthreads();
    }
    return prefix;
}

template <int CL>
__global__ void __launch_bounds__(STHREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, int* __restrict__ out_token, float* __restrict__ out_logprob,
              int vocab, int cache_floats) {
    __shared__ RowShared<CL> sh;
    extern __shared__ __align__(16) float x_cache[];     // x of this block's slice when `cache_floats` holds it
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = CL == 1 ? 0 : (int)cluster.block_rank();
    const int r = blockIdx.y;
    const float* row = logits + (size_t)r * vocab;
    const int slice = ((vocab + CL - 1) / CL + 31) / 32 * 32;
    const int v0 = min(vocab, rank * slice), v1 = min(vocab, v0 + slice);
    const float temp = temperature[r];
    const int k = top_k[r];
    const bool greedy = temp == 0.f || k == 1;
    const float tdiv = greedy ? 1.f : fmaxf(temp, 1e-5f);   // the divisor: x = logit / max(T, 1e-5)

    // x = logit / divisor of this block's slice, once, into shared memory: every later pass reads it there
    const bool cached = v1 - v0 <= cache_floats;
    if (cached)
        for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) x_cache[i - v0] = row[i] / tdiv;
    __syncthreads();
    const RowX xs{row, cached ? x_cache : nullptr, v0, tdiv};

    // the row's best value (ties go to the lower index)
    {
        const ArgBest b = cached ? block_argmax(x_cache, v1 - v0, 1.f, sh.best) : block_argmax(row + v0, v1 - v0, tdiv, sh.best);
        if (threadIdx.x == 0) sh.cbest = ArgBest{b.v, b.i < v1 - v0 ? b.i + v0 : 0x7fffffff};
    }
    cluster_barrier<CL>(cluster);
    ArgBest top{-INFINITY, 0x7fffffff};
    for (int rk = 0; rk < CL; ++rk) top = better(top, *peer<CL>(cluster, &sh.cbest, rk));
    const float mx = top.v;

    if (greedy) {
        float s = 0.f;
        for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) s += expf(xs(i) - mx);
        s = block_sum(s, sh.fsum);
        if (threadIdx.x == 0) sh.csum = s;
        cluster_barrier<CL>(cluster);
        if (rank == 0 && threadIdx.x == 0) {
            float total = 0.f;
            for (int rk = 0; rk < CL; ++rk) total += *peer<CL>(cluster, &sh.csum, rk);
            out_token[r] = top.i < vocab ? top.i : 0;
            if (out_logprob) out_logprob[r] = -logf(total);
        }
        cluster_barrier<CL>(cluster);                   // nobody leaves while its shared memory may be read
        return;
    }

    int pass = 0;
    unsigned floor_key = 0;
    if (k > 0 && k < vocab)
        floor_key = radix_select<CL, false>(cluster, sh, xs, v0, v1, mx, 0u, (unsigned long long)k, pass);

    const float p = top_p[r];
    if (p < 1.f) {
        // mass of the top-k survivors, then the cut
        unsigned long long z = 0;
        for (int i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
            const float x = xs(i);
            if (ordered_key(x) >= floor_key) z += to_fixed(expf(x - mx));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
        if (threadIdx.x == 0) sh.ctotal = 0;
        __syncthreads();
        if ((threadIdx.x & 31) == 0) atomicAdd(&sh.ctotal, z);
        cluster_barrier<CL>(cluster);
        unsigned long long total = 0;
        for (int rk = 0; rk < CL; ++rk) total += *peer<CL>(cluster, &sh.ctotal, rk);
        const unsigned long long limit = (unsigned long long)((double)p * (double)total);
        const unsigned cut = radix_select<CL, true>(cluster, sh, xs, v0, v1, mx, floor_key, limit > 0 ? limit : 1ull, pass);
        floor_key = max(floor_key, cut);
    }
    const float mp = min_p[r];
    if (threadIdx.x < 32) sh.wsum[threadIdx.x] = 0;     // a block of fewer than 32 warps leaves the other slots empty
    __syncthreads();

    // kept mass of each warp's contiguous segment of the slice (lanes interleaved, so the reads
    // coalesce), then the draw in vocabulary order: the segment in which the running mass passes the
    // target is walked by its warp 32 tokens at a time with a prefix sum over the lanes
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int seg = ((v1 - v0 + nwarp - 1) / nwarp + 31) / 32 * 32;
    const int lo = min(v1, v0 + warp * seg), hi = min(v1, lo + seg);
    unsigned long long mine = 0;
    for (int i = lo + lane; i < hi; i += 32) {
        const float x = xs(i);
        const float e = expf(x - mx);
        if (ordered_key(x) >= floor_key && e >= mp) mine += to_fixed(e);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) sh.wsum[warp] = mine;
    cluster_barrier<CL>(cluster);
    for (int i = threadIdx.x; i < CL * 32; i += blockDim.x) sh.all_wsum[i] = peer<CL>(cluster, sh.wsum, i / 32)[i % 32];
    cluster_barrier<CL>(cluster);                       // the last read of another block's shared memory is behind us
    unsigned long long total = 0, before = 0;
    const int me = rank * 32 + warp;
    for (int w = 0; w < CL * 32; ++w) {
        if (w < me) before += sh.all_wsum[w];
        total += sh.all_wsum[w];
    }
    if (total == 0) {
        if (rank == 0 && threadIdx.x == 0) {    // nothing kept (cannot happen: the largest always is): the largest
            out_token[r] = top.i < vocab ? top.i : 0;
            if (out_logprob) out_logprob[r] = 0.f;
        }
        return;
    }
    unsigned long long target = (unsigned long long)((double)uniform[r] * (double)total);
    if (target >= total) target = total - 1;
    if (!(before <= target && target < before + mine)) return;       // the one warp whose segment holds the target stays
    unsigned long long run = before;
    for (int base = lo; base < hi; base += 32) {
        const int i = base + lane;
        float e = 0.f;
        unsigned long long v = 0;
        if (i < hi) {
            const float x = xs(i);
            e = expf(x - mx);
            if (ordered_key(x) >= floor_key && e >= mp) v = to_fixed(e);
        }
        unsigned long long incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, v != 0 && run + incl > target);
        if (hit) {
            if (lane == __ffs(hit) - 1) {
                out_token[r] = i;
                if (out_logprob) out_logprob[r] = logf(e) - logf((float)((double)total / FIXED_ONE));
            }
            return;
        }
        run += __shfl_sync(0xffffffffu, incl, 31);
    }
}

// The k most probable tokens of a row and their log-probabilities (log-softmax of the logits as they
// are, i.e. after penalties and before temperature: lily/layers/sampler.py:118-133).  One block per row:
// maximum and log-sum-exp, the k-th largest key by radix selection, then every token at or above it is
// appended to the row's list (ties may make it longer than k, up to `cap`; the host sorts and cuts).
constexpr int TOP_CAP = 128;

__global__ void __launch_bounds__(STHREADS)
top_logprobs_kernel(const float* __restrict__ logits, const int* __restrict__ k_per_row, int* __restrict__ out_token,
                    float* __restrict__ out_logprob, int* __restrict__ out_count, int vocab) {
    __shared__ RowShared<1> sh;
    __shared__ int count_s;
    cg::cluster_group cluster = cg::this_cluster();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    const int k = min(k_per_row[r], TOP_CAP);
    if (threadIdx.x == 0) count_s = 0;
    if (k <= 0) {
        if (threadIdx.x == 0) out_count[r] = 0;
        return;
    }
    const ArgBest top = block_argmax(row, vocab, 1.f, sh.best);
    float s = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) s += expf(row[i] - top.v);
    s = block_sum(s, sh.fsum);
    const float lse = top.v + logf(s);
    const RowX xs{row, nullptr, 0, 1.f};
    int pass = 0;
    const unsigned kth = k < vocab ? radix_select<1, false>(cluster, sh, xs, 0, vocab, top.v, 0u, (unsigned long long)k, pass) : 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i];
        if (ordered_key(x) >= kth) {
            const int at = atomicAdd(&count_s, 1);
            if (at < TOP_CAP) {
                out_token[(size_t)r * TOP_CAP + at] = i;
                out_logprob[(size_t)r * TOP_CAP + at] = x - lse;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) out_count[r] = min(count_s, TOP_CAP);
}

}  // namespace lily

using namespace lily;

// Ranges a row is cut into (1: the single-block kernel); the caller provides scratch of
// rows * chunks floats and as many ints when it is more than 1.
LILY_API int lily_argmax_chunks(int rows, int vocab) {
    if (vocab < 16384) return 1;
    int chunks = (sm_count() * 4 + rows - 1) / (rows > 0 ? rows : 1);
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
    constexpr int CL = 8;
    const bool clustered = vocab >= CL * 4096;
    const int slice = clustered ? ((vocab + CL - 1) / CL + 31) / 32 * 32 : (vocab + 31) / 32 * 32;
    // the slice's x values stay in shared memory when they fit beside the kernel's static 12 KB
    int cache_floats = slice * 4 <= 160 * 1024 ? slice : 0;
    static int granted[2] = {0, 0};
    if (cache_floats * 4 > granted[clustered]) {
        const cudaError_t e = clustered
            ? cudaFuncSetAttribute(sample_kernel<CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, cache_floats * 4)
            : cudaFuncSetAttribute(sample_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cache_floats * 4);
        if (e != cudaSuccess) {
            cudaGetLastError();
            cache_floats = 0;                           // the kernel reads the logits again in every pass instead
        } else {
            granted[clustered] = cache_floats * 4;
        }
    }
    if (clustered) {
        // a cluster of CL blocks per row
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(CL, rows);
        // more blocks than the device holds at once (a block of 1,024 threads has a SM to itself): half the threads,
        // so that two blocks share a SM and one computes while the other waits at a cluster barrier
        // (vocabulary 151,936, temperature only: 64 rows 139 -> 96 us, 256 rows 486 -> 339 us; with top-p 1904 -> 1442 us)
        cfg.blockDim = dim3((long)CL * rows > sm_count() ? STHREADS / 2 : STHREADS);
        cfg.dynamicSmemBytes = (size_t)cache_floats * 4;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, sample_kernel<CL>, logits, temperature, top_k, top_p, min_p, uniform, out_token, out_logprob, vocab,
                           cache_floats);
    } else {
        sample_kernel<1><<<dim3(1, rows), STHREADS, (size_t)cache_floats * 4, stream>>>(logits, temperature, top_k, top_p, min_p, uniform,
                                                                                       out_token, out_logprob, vocab, cache_floats);
    }
    LILY_CHECK_LAUNCH("sample");
    return 0;
}

LILY_API int lily_top_logprobs_cap() { return TOP_CAP; }

// out_token / out_logprob: [rows, lily_top_logprobs_cap()], out_count [rows]; k_per_row[r] <= 0 leaves row r empty.
LILY_API int lily_top_logprobs(const float* logits, const int* k_per_row, int* out_token, float* out_logprob, int* out_count,
                               int rows, int vocab, cudaStream_t stream) {
    if (rows == 0) return 0;
    LILY_REQUIRE(vocab > 0, "top_logprobs: vocab=%d", vocab);
    top_logprobs_kernel<<<rows, STHREADS, 0, stream>>>(logits, k_per_row, out_token, out_logprob, out_count, vocab);
    LILY_CHECK_LAUNCH("top_logprobs");
    return 0;
}
