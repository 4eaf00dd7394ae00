// Paged causal grouped-query attention in bfloat16 on the tensor cores (mma.sync m16n8k16,
// float32 accumulation), for head sizes that are multiples of 64 up to 256.  Other head sizes and
// the float32 path use attention_simt.cu; both read the same cache layout and take the same
// arguments, and both are tested against the same plain statement.
//
//  * prefill: grid (query tiles of 64 new tokens, query heads), 4 warps of 16 query rows each.
//  * decode:  grid (requests, kv heads x row chunks, splits).  The query heads that share a kv head
//    are the (up to 16) rows; the 4 warps take 16 keys each of every 64-key tile and keep their own
//    running (max, sum, output), merged through shared memory at the end.  The splits of one
//    (request, kv head) are merged either inside a thread-block cluster (1 x 1 x splits, up to 16
//    blocks: each block sends every other its share of the sums through distributed shared memory,
//    one cluster barrier, each finishes its share of the output; used while all clusters are resident
//    at once) or through scratch and the combine kernel of attention_simt.cu.
//    The queries come finished from `q`, or, in a step where every request brings one token, from
//    the qkv product itself: a warp per head sums the product's partial planes, applies the per-head
//    RMSNorm and the rotation, and the block whose key range holds the new position does the same
//    for the key, copies the value, and writes both to their page before it reads them.
//
// Key and value tiles of 64 positions are brought in with cp.async (16-byte pieces, any page
// size: each row's page is looked up in the block table), double buffered, into shared memory
// whose 16-byte pieces are XOR-swizzled by row so that ldmatrix reads without bank conflicts.
// Scores, the running maximum and sum, and the output accumulate in float32; probabilities are
// rounded to bfloat16 for p.v as in lily/layers/attention/triton_ops/extend_attention.py:110-112.
#include "attention_args.cuh"
#include "common.cuh"

#include <cooperative_groups.h>

namespace lily {
namespace mma {

namespace cg = cooperative_groups;

constexpr int BN = 64;        // keys per tile
constexpr int MAX_CLUSTER = 16;      // blocks of a cluster that merges the splits of a decode row
constexpr int THREADS = 128;
#ifndef LILY_DECODE_STAGES
// Two key/value stages.  Measured and not kept: three stages (the kernel alone gains 6 %, the step loses 2 %: the shared
// memory keeps the next product's blocks from becoming resident and streaming weights under it), and four stages for
// steps whose blocks have a SM each (one request over 16 key ranges: 15.1 -> 13.1 us alone, the step unchanged at 3.39 ms).
#define LILY_DECODE_STAGES 2
#endif
// Also measured and not kept: asking the lines of the next two or four tiles into L2 (prefetch.global.L2, a line a
// thread) while the block prepares its queries: the step of 8 requests went from 3.92 to 4.04 ms, of one from 3.30 to 3.43;
// and asking the weights of the product behind the attention into L2 (cp.async.bulk.prefetch.L2, each block its share)
// once a block's keys and values are in: 3.92 to 3.97 ms and 3.30 to 3.35 ms; and a final merge with a thread for each
// (four features, split) and shuffles over the splits instead of a loop: 3.90 to 3.94 ms and 3.28 to 3.32 ms.

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Built with -DLILY_DECODE_TIMING, thread 0 of each of the first 16 splits of (request 0, kv head 0) stamps the
// SM's cycle counter as it passes each phase of the decode kernel (lily_attention_decode_timing reads the stamps).
#ifdef LILY_DECODE_TIMING
__device__ unsigned long long g_decode_stamps[16][16];
__device__ unsigned long long g_decode_spans[4096][2];      // per block: the global timer (ns) at entry and at exit
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define DECODE_SPAN(which) do { const unsigned b__ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z); \
                                if (DECODE && threadIdx.x == 0 && b__ < 4096) g_decode_spans[b__][which] = global_ns(); } while (0)
#define DECODE_STAMP(slot) do { if (DECODE && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z < 16) \
                                    g_decode_stamps[blockIdx.z][slot] = (unsigned long long)clock64(); } while (0)
#else
#define DECODE_STAMP(slot) do {} while (0)
#define DECODE_SPAN(which) do {} while (0)
#endif

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;     // 0 source bytes: the 16 destination bytes are zero-filled
#if defined(LILY_ATTN_L2_256)
    asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
#else
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
#endif
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of the 16-byte piece `chunk` of row `row` in a tile whose rows hold D bfloat16.
template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * (D * 2) + ((((chunk ^ row) & 7) | (chunk & ~7)) << 4));
}

// Shared memory of one block: the key/value stages (reused for the merge of the four warps), then, when a
// cluster merges the splits (CLUSTER), what the other blocks of the cluster send: per split this block's share
// of the output sums, and per split and row (max, sum).
template <int D, int STAGES>
__host__ __device__ constexpr size_t stage_bytes(bool decode) {
    const size_t stages = 2 * (size_t)STAGES * BN * D * 2, merge = (size_t)(4 * 16 * D + 4 * 16 * 2) * sizeof(float);
    return decode && merge > stages ? merge : stages;
}
// Output sums a block of a cluster of `splits` blocks merges: its share of rows x D.
__host__ __device__ inline int cluster_share(int rows, int d, int splits) { return ((rows * d + splits - 1) / splits + 3) / 4 * 4; }

template <int D, bool DECODE, int STAGES, bool CLUSTER>
__global__ void __launch_bounds__(THREADS, D <= 128 ? 3 : 1)
attention_mma_kernel(const AttnArgs a, const int page_shift) {
    constexpr int CH = D / 8;                  // 16-byte pieces per row
    constexpr int KSTEPS = D / 16;
    constexpr int BM = DECODE ? 16 : 64;
    constexpr int NT = DECODE ? 2 : 8;         // score n-tiles (8 keys each) per warp and key tile
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* k_s = smem_raw;                                  // [STAGES][BN][D]
    unsigned char* v_s = k_s + STAGES * BN * D * 2;                 // [STAGES][BN][D]
    // the queries pass through the last key stage on their way to registers: that stage is first
    // filled after the barrier of the first loop iteration, when every warp has its fragments
    unsigned char* q_s = k_s + (STAGES - 1) * BN * D * 2;           // [BM][D], BM <= BN
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    DECODE_STAMP(0);
    DECODE_SPAN(0);
    // Prefill waits here for the kernel before it (which wrote q and this step's keys).  Decode
    // waits further down: the block table, the lengths and every cached key but the one of this
    // step were there before that kernel began, so the first key tiles stream in while it runs.
    if (!DECODE) {
        pdl_wait();
        pdl_launch_dependents();
    }
    const __nv_bfloat16* q = (const __nv_bfloat16*)a.q;
    const __nv_bfloat16* kv = (const __nv_bfloat16*)a.kv;
    const int group = a.nq / a.nkv;

    int req, kvh, kbeg, kend, nrows, head0 = 0, tok0 = 0, pos0 = 0;
    if (DECODE) {
        req = blockIdx.x;
        const int chunks = (group + 15) / 16;
        kvh = blockIdx.y / chunks;
        const int r0 = (blockIdx.y % chunks) * 16;
        const int seq = a.seq_lens[req];
        const int lo = (a.window > 0 && seq > a.window) ? seq - a.window : 0;
        int per = (seq - lo + a.splits - 1) / a.splits;
        per = (per + BN - 1) / BN * BN;
        kbeg = lo + blockIdx.z * per;
        kend = min(seq, kbeg + per);
        nrows = min(16, group - r0);
        head0 = kvh * group + r0;
        tok0 = req;
        pos0 = seq > 0 ? seq - 1 : 0;                        // an empty row (no position yet) reads table entry 0 at most
    } else {
        const int tile = gridDim.x - 1 - blockIdx.x;       // the tiles come ordered by the keys they see: longest first
        req = a.tile_req[tile];
        const int start = a.tile_start[tile];
        const int t0 = a.cu_seqlens[req], len = a.cu_seqlens[req + 1] - t0;
        const int prefix = a.prefix_lens[req];
        head0 = blockIdx.y;
        kvh = head0 / group;
        nrows = min(BM, len - start);
        tok0 = t0 + start;
        pos0 = prefix + start;
        kend = pos0 + nrows;
        kbeg = (a.window > 0 && pos0 + 1 > a.window) ? pos0 + 1 - a.window : 0;
    }

    const int* table = a.block_table + (size_t)req * a.bt_stride;
    const size_t head_stride = (size_t)a.page_size * D;
    const size_t page_stride = 2 * (size_t)a.nkv * head_stride;
    const int ntiles = kend > kbeg ? (kend - kbeg + BN - 1) / BN : 0;

    const __nv_bfloat16* kv_head = kv + (size_t)kvh * head_stride;
    const int page_mask = (1 << page_shift) - 1;
    auto load_tile = [&](int t, int buf) {
        const int kb = kbeg + t * BN;
        unsigned char* kd = k_s + buf * BN * D * 2;
        unsigned char* vd = v_s + buf * BN * D * 2;
#pragma unroll
        for (int i = tid; i < BN * CH; i += THREADS) {
            const int r = i / CH, ch = i % CH;
            const int kpos = kb + r;
            const bool ok = kpos < kend;
            const int page = ok ? table[kpos >> page_shift] : 0;
            const __nv_bfloat16* src = kv_head + (size_t)page * page_stride + (((ok ? kpos : 0) & page_mask) * D + ch * 8);
            const uint32_t off = swz<D>(r, ch);
            cp_async16(smem_u32(kd + off), src, ok);
            cp_async16(smem_u32(vd + off), src + (size_t)a.nkv * head_stride, ok);
        }
    };

    // the pipeline keeps STAGES - 1 tiles in flight; every iteration commits one group (maybe empty).
    // Decode: the tiles that end before this step's own key are asked for ahead of the wait.
    int early = 0;
    if (DECODE) {
#pragma unroll
        for (int st = 0; st < STAGES - 1; ++st) {
            if (st < ntiles && kbeg + (st + 1) * BN <= pos0 && early == st) {
                load_tile(st, st);
                cp_async_commit();
                ++early;
            }
        }
        DECODE_STAMP(1);
        pdl_wait();
        pdl_launch_dependents();
        DECODE_STAMP(2);
    }

    // ---- queries to shared memory (zero rows beyond nrows), then to A fragments -------------
    if (DECODE && a.qkv != nullptr) {
        // straight from the projection: a warp per head sums the planes, norms (lily/models/qwen3.py:27-29), rotates
        // (lily/layers/rotary.py:18-20, 70-87) and rounds to bfloat16 as the separate kernel does; the block whose
        // range holds this step's position also finishes the key and the value and writes them to their page
        for (int i = tid; i < (BM - nrows) * CH; i += THREADS)
            *reinterpret_cast<uint4*>(q_s + swz<D>(nrows + i / CH, i % CH)) = make_uint4(0, 0, 0, 0);
        const size_t width = (size_t)(a.nq + 2 * a.nkv) * D;
        auto in = [&](size_t idx) -> float {
            if (!a.qkv_f32) return __bfloat162float(((const __nv_bfloat16*)a.qkv)[idx]);
            const float* p = (const float*)a.qkv + idx;
            float sum = 0.f;
            for (int pl = 0; pl < a.qkv_planes; ++pl) sum += p[(size_t)pl * a.qkv_stride];
            return sum;
        };
        const int half = a.rd >> 1;
        const float* cs = a.cos_t ? a.cos_t + (size_t)pos0 * half : nullptr;
        const float* sn = a.sin_t ? a.sin_t + (size_t)pos0 * half : nullptr;
        const bool owner = a.write_kv && kbeg <= pos0 && pos0 < kend;
        const int jobs = nrows + (owner ? 2 : 0);                      // the query heads, then the key, then the value
        const bool whole = cs == nullptr || a.rd == D;                 // no rotation, or over the whole head
        constexpr int WARPS = THREADS / 32;
        auto head_of = [&](int job) { return job < nrows ? head0 + job : a.nq + (job == nrows + 1 ? a.nkv : 0) + kvh; };
        // where this step's key goes (the value lies nkv heads further)
        __nv_bfloat16* own_key = owner ? const_cast<__nv_bfloat16*>(kv_head) + (size_t)table[pos0 >> page_shift] * page_stride +
                                             (size_t)(pos0 & page_mask) * D : nullptr;
        if (whole && warp < jobs) {
            // A lane holds E neighbouring features; the feature half a head further is in lane ^ 16, same place.
            // Everything a warp reads is asked for before the first sum: gains, angles, and the planes (up to eight
            // each) of two heads at a time, so that the block with the key and the value (six heads over four
            // warps where four query heads share a kv head) waits for memory once and not twice.
            constexpr int E = D / 32;
            const int e0 = lane * E, t0 = e0 - (lane >= 16 ? D / 2 : 0);
            const size_t step = a.qkv_stride / 2;
            float gain_q[E], gain_k[E], cos_r[E], sin_r[E];
#pragma unroll
            for (int j = 0; j < E; ++j) {
                gain_q[j] = gain_k[j] = 1.f;
                if (a.q_gain) {
                    gain_q[j] = a.gain_f32 ? ((const float*)a.q_gain)[e0 + j] : __bfloat162float(((const __nv_bfloat16*)a.q_gain)[e0 + j]);
                    gain_k[j] = a.gain_f32 ? ((const float*)a.k_gain)[e0 + j] : __bfloat162float(((const __nv_bfloat16*)a.k_gain)[e0 + j]);
                }
                cos_r[j] = cs ? cs[t0 + j] : 1.f;
                sin_r[j] = cs ? sn[t0 + j] : 0.f;
            }
            auto ask = [&](int job, float2 (&v)[8][E / 2]) {
                const size_t src = (size_t)tok0 * width + (size_t)head_of(job) * D + e0;
                if (a.qkv_f32) {
                    const float2* p = reinterpret_cast<const float2*>((const float*)a.qkv + src);
#pragma unroll
                    for (int u = 0; u < 8; ++u)
#pragma unroll
                        for (int j = 0; j < E / 2; ++j) v[u][j] = u < a.qkv_planes ? p[(size_t)u * step + j] : make_float2(0.f, 0.f);
                } else {
                    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>((const __nv_bfloat16*)a.qkv + src);
#pragma unroll
                    for (int u = 0; u < 8; ++u)
#pragma unroll
                        for (int j = 0; j < E / 2; ++j) v[u][j] = u == 0 ? __bfloat1622float2(p[j]) : make_float2(0.f, 0.f);
                }
            };
            auto finish = [&](int job, const float2 (&v)[8][E / 2]) {
                const bool is_q = job < nrows, is_v = job == nrows + 1;
                float x[E];
#pragma unroll
                for (int j = 0; j < E; ++j) x[j] = 0.f;
#pragma unroll
                for (int u = 0; u < 8; ++u)                            // summed in the order of the planes
#pragma unroll
                    for (int j = 0; j < E / 2; ++j) {
                        x[2 * j] += v[u][j].x;
                        x[2 * j + 1] += v[u][j].y;
                    }
                if (a.qkv_f32 && a.qkv_planes > 8) {
                    const float2* p = reinterpret_cast<const float2*>((const float*)a.qkv + (size_t)tok0 * width + (size_t)head_of(job) * D + e0);
                    for (int pl = 8; pl < a.qkv_planes; ++pl)
#pragma unroll
                        for (int j = 0; j < E / 2; ++j) {
                            const float2 more = p[(size_t)pl * step + j];
                            x[2 * j] += more.x;
                            x[2 * j + 1] += more.y;
                        }
                }
                if (a.q_gain && !is_v) {
                    float ssq = 0.f;
#pragma unroll
                    for (int j = 0; j < E; ++j) ssq += x[j] * x[j];
                    const float inv = rsqrtf(warp_sum(ssq) / (float)D + a.eps);
#pragma unroll
                    for (int j = 0; j < E; ++j) x[j] = (x[j] * inv) * (is_q ? gain_q[j] : gain_k[j]);
                }
                if (cs && !is_v) {
#pragma unroll
                    for (int j = 0; j < E; ++j) {
                        const float other = __shfl_xor_sync(0xffffffffu, x[j], 16);
                        const float x1 = lane < 16 ? x[j] : other, x2 = lane < 16 ? other : x[j];
                        x[j] = lane < 16 ? x1 * cos_r[j] - x2 * sin_r[j] : x2 * cos_r[j] + x1 * sin_r[j];
                    }
                }
                __nv_bfloat16* cached = is_q ? nullptr : own_key + (is_v ? (size_t)a.nkv * head_stride : 0);
#pragma unroll
                for (int j = 0; j < E / 2; ++j) {
                    const uint32_t two = pack_bf16(x[2 * j], x[2 * j + 1]);
                    const int i = e0 + 2 * j;
                    if (is_q) *reinterpret_cast<uint32_t*>(q_s + swz<D>(job, i >> 3) + (i & 7) * 2) = two;
                    else *reinterpret_cast<uint32_t*>(cached + i) = two;
                }
            };
            for (int job = warp; job < jobs; job += 2 * WARPS) {
                float2 v0[8][E / 2], v1[8][E / 2];
                const bool second = job + WARPS < jobs;
                ask(job, v0);
                if (second) ask(job + WARPS, v1);
                finish(job, v0);
                if (second) finish(job + WARPS, v1);
            }
        } else if (!whole)
        for (int job = warp; job < jobs; job += WARPS) {
            const bool is_q = job < nrows, is_v = job == nrows + 1;
            const size_t src = (size_t)tok0 * width + (size_t)head_of(job) * D;
            const void* gain = is_q ? a.q_gain : (is_v ? nullptr : a.k_gain);
            __nv_bfloat16* cached = is_q ? nullptr : own_key + (is_v ? (size_t)a.nkv * head_stride : 0);
            auto gain_at = [&](int i) -> float {
                return a.gain_f32 ? ((const float*)gain)[i] : __bfloat162float(((const __nv_bfloat16*)gain)[i]);
            };
            auto put = [&](int i, float v) {
                const __nv_bfloat16 b = __float2bfloat16_rn(v);
                if (is_q) *reinterpret_cast<__nv_bfloat16*>(q_s + swz<D>(job, i >> 3) + (i & 7) * 2) = b;
                else cached[i] = b;
            };
            if (is_v) {
                for (int i = lane; i < D; i += 32) put(i, in(src + i));
                continue;
            }
            float inv = 1.f;
            if (gain) {
                float ssq = 0.f;
                for (int i = lane; i < D; i += 32) {
                    const float x = in(src + i);
                    ssq += x * x;
                }
                inv = rsqrtf(warp_sum(ssq) / (float)D + a.eps);
            }
            for (int i = lane; i < half; i += 32) {
                float x1 = in(src + i), x2 = in(src + i + half);
                if (gain) {
                    x1 = (x1 * inv) * gain_at(i);
                    x2 = (x2 * inv) * gain_at(i + half);
                }
                float o1 = x1, o2 = x2;
                if (cs) {
                    const float cc = cs[i], ss = sn[i];
                    o1 = x1 * cc - x2 * ss;
                    o2 = x2 * cc + x1 * ss;
                }
                put(i, o1);
                put(i + half, o2);
            }
            for (int i = a.rd + lane; i < D; i += 32) {
                float x = in(src + i);
                if (gain) x = (x * inv) * gain_at(i);
                put(i, x);
            }
        }
        if (owner) __threadfence();                // the key and the value are in place before this block's copies read them
    } else
    for (int i = tid; i < BM * CH; i += THREADS) {
        const int r = i / CH, ch = i % CH;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (r < nrows) {
            const size_t tok = DECODE ? (size_t)tok0 : (size_t)tok0 + r;
            const int head = DECODE ? head0 + r : head0;
            val = *reinterpret_cast<const uint4*>(q + (tok * a.nq + head) * D + ch * 8);
        }
        *reinterpret_cast<uint4*>(q_s + swz<D>(r, ch)) = val;
    }
    __syncthreads();
    DECODE_STAMP(3);
    uint32_t qf[KSTEPS][4];
    {
        const int rbase = DECODE ? 0 : warp * 16;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk)
            ldmatrix_x4(smem_u32(q_s + swz<D>(rbase + (lane & 15), kk * 2 + (lane >> 4))), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
    const int row_lo = DECODE ? g : warp * 16 + g;      // this thread's two rows within the block
    const int row_hi = row_lo + 8;
    const int qpos_lo = DECODE ? pos0 : pos0 + row_lo, qpos_hi = DECODE ? pos0 : pos0 + row_hi;

    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st >= early) {
            if (st < ntiles) load_tile(st, st);
            cp_async_commit();
        }
    }
    const float sl2 = a.scale * 1.4426950408889634f;       // scores are kept in units of log2(e)

    for (int t = 0; t < ntiles; ++t) {
        const int buf = t % STAGES;
        cp_async_wait<STAGES - 2>();
        __syncthreads();                                    // tile t has landed; tile t-1's readers are done
        if (t == 0) DECODE_STAMP(4);
        if (t + STAGES - 1 < ntiles) load_tile(t + STAGES - 1, (t + STAGES - 1) % STAGES);
        cp_async_commit();
        const unsigned char* kt = k_s + buf * BN * D * 2;
        const unsigned char* vt = v_s + buf * BN * D * 2;
        const int kb = kbeg + t * BN;
        const int key0 = DECODE ? warp * 16 : 0;            // first key of this warp's share of the tile

        // ---- s = q . k^T -------------------------------------------------------------------
        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
            for (int jp = 0; jp < NT / 2; ++jp) {
                uint32_t b0, b1, b2, b3;
                const int krow = key0 + jp * 16 + (lane & 7) + ((lane >> 4) << 3);
                ldmatrix_x4(smem_u32(kt + swz<D>(krow, kk * 2 + ((lane >> 3) & 1))), b0, b1, b2, b3);
                mma_bf16(s[2 * jp], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
                mma_bf16(s[2 * jp + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
            }
        }

        // ---- mask (boundary tiles only), running maximum and sum ----------------------------------
        const int q_first = DECODE ? pos0 : pos0 + warp * 16, q_last = DECODE ? pos0 : q_first + 15;
        const bool need_mask = kb + BN > kend || kb + BN - 1 > q_first || (a.window > 0 && kb <= q_last - a.window);
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
        if (need_mask) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int kpos = kb + key0 + j * 8 + 2 * c + (e & 1);
                    const int qpos = (e < 2) ? qpos_lo : qpos_hi;
                    const bool seen = kpos < kend && kpos <= qpos && (a.window <= 0 || kpos > qpos - a.window);
                    if (!seen) s[j][e] = -INFINITY;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            mx_lo = fmaxf(mx_lo, fmaxf(s[j][0], s[j][1]));
            mx_hi = fmaxf(mx_hi, fmaxf(s[j][2], s[j][3]));
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        // running maxima are kept in scaled (log2) units: scale > 0, so the order is the same
        const float mn_lo = fmaxf(m_lo, mx_lo * sl2), mn_hi = fmaxf(m_hi, mx_hi * sl2);
        const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo, base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float al_lo = exp2f(m_lo - base_lo), al_hi = exp2f(m_hi - base_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            s[j][0] = exp2f(fmaf(s[j][0], sl2, -base_lo));
            s[j][1] = exp2f(fmaf(s[j][1], sl2, -base_lo));
            s[j][2] = exp2f(fmaf(s[j][2], sl2, -base_hi));
            s[j][3] = exp2f(fmaf(s[j][3], sl2, -base_hi));
            sum_lo += s[j][0] + s[j][1];
            sum_hi += s[j][2] + s[j][3];
        }
        l_lo = l_lo * al_lo + sum_lo;                       // per-thread partial sums; reduced at the end
        l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            o[j][0] *= al_lo;
            o[j][1] *= al_lo;
            o[j][2] *= al_hi;
            o[j][3] *= al_hi;
        }

        // ---- o += p . v -------------------------------------------------------------------------
#pragma unroll
        for (int kb16 = 0; kb16 < NT / 2; ++kb16) {
            const uint32_t a0 = pack_bf16(s[2 * kb16][0], s[2 * kb16][1]);
            const uint32_t a1 = pack_bf16(s[2 * kb16][2], s[2 * kb16][3]);
            const uint32_t a2 = pack_bf16(s[2 * kb16 + 1][0], s[2 * kb16 + 1][1]);
            const uint32_t a3 = pack_bf16(s[2 * kb16 + 1][2], s[2 * kb16 + 1][3]);
            const int vrow = key0 + kb16 * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
            for (int jp = 0; jp < D / 16; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(smem_u32(vt + swz<D>(vrow, jp * 2 + (lane >> 4))), b0, b1, b2, b3);
                mma_bf16(o[2 * jp], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[2 * jp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
    }

    DECODE_STAMP(5);
    // sums over the four threads that share a row
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    if (!DECODE) {
        __nv_bfloat16* out = (__nv_bfloat16*)a.out;
        const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            const int col = j * 8 + 2 * c;
            if (row_lo < nrows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(tok0 + row_lo) * a.nq + head0) * D + col) =
                    pack_bf16(o[j][0] * inv_lo, o[j][1] * inv_lo);
            if (row_hi < nrows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(tok0 + row_hi) * a.nq + head0) * D + col) =
                    pack_bf16(o[j][2] * inv_hi, o[j][3] * inv_hi);
        }
        return;
    }

    // ---- decode: merge the four warps' partial results through shared memory ---------------------
    __syncthreads();                                        // every warp is done with the key/value tiles
    float* mo = reinterpret_cast<float*>(k_s);              // [4 warps][16 rows][D]
    float* mml = mo + 4 * 16 * D;                           // [4 warps][16 rows][2]
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        const int col = j * 8 + 2 * c;
        mo[(warp * 16 + row_lo) * D + col] = o[j][0];
        mo[(warp * 16 + row_lo) * D + col + 1] = o[j][1];
        mo[(warp * 16 + row_hi) * D + col] = o[j][2];
        mo[(warp * 16 + row_hi) * D + col + 1] = o[j][3];
    }
    if (c == 0) {
        mml[(warp * 16 + row_lo) * 2] = m_lo;
        mml[(warp * 16 + row_lo) * 2 + 1] = l_lo;
        mml[(warp * 16 + row_hi) * 2] = m_hi;
        mml[(warp * 16 + row_hi) * 2 + 1] = l_hi;
    }
    __syncthreads();
    DECODE_STAMP(6);
    const float ln2 = 0.6931471805599453f;
    // CLUSTER: the blocks of the cluster hold the splits of one (request, kv head); each sends every other its
    // share of the merged sums through distributed shared memory, and after one cluster barrier each block
    // finishes its share of the output, so that neither scratch in global memory nor a combine kernel is needed.
    // Sums travel and are merged four neighbouring features at a time (shares are multiples of four).
    cg::cluster_group cluster = cg::this_cluster();
    const int splits = a.splits, me = blockIdx.z;
    const int share = cluster_share(min(16, group), D, splits);
    float* recv_o = reinterpret_cast<float*>(smem_raw + stage_bytes<D, STAGES>(true));     // [splits][share]
    float* recv_ml = recv_o + (size_t)splits * share;                                        // [splits][16][2]
    for (int i4 = tid; i4 < nrows * (D / 4); i4 += THREADS) {
        const int r = i4 / (D / 4), col = (i4 % (D / 4)) * 4, i = r * D + col;
        float mw[4], mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            mw[w] = mml[(w * 16 + r) * 2];
            mx = fmaxf(mx, mw[w]);
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float den = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            if (mw[w] > -INFINITY) {
                const float f = exp2f(mw[w] - mx);
                const float4 v = *reinterpret_cast<const float4*>(mo + (w * 16 + r) * D + col);
                acc.x += v.x * f;
                acc.y += v.y * f;
                acc.z += v.z * f;
                acc.w += v.w * f;
                den += mml[(w * 16 + r) * 2 + 1] * f;
            }
        }
        const int head = head0 + r;
        if (CLUSTER) {
            const int owner = i / share;
            *reinterpret_cast<float4*>(cluster.map_shared_rank(recv_o, owner) + me * share + (i - owner * share)) = acc;
            if (col / 4 < splits)                          // group p of four columns tells block p the row's (max, sum)
                *reinterpret_cast<float2*>(cluster.map_shared_rank(recv_ml, col / 4) + (me * 16 + r) * 2) = make_float2(mx, den);
        } else if (a.splits > 1) {
            const size_t base = ((size_t)tok0 * a.nq + head) * a.splits + blockIdx.z;
            *reinterpret_cast<float4*>(a.part_o + base * D + col) = acc;
            if (col == 0) {
                a.part_ml[base * 2] = mx * ln2;             // back to natural-log units for the combine kernel
                a.part_ml[base * 2 + 1] = den;
            }
        } else {
            const float inv = den > 0.f ? 1.f / den : 0.f;
            *reinterpret_cast<uint2*>((__nv_bfloat16*)a.out + ((size_t)tok0 * a.nq + head) * D + col) =
                make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        }
    }
    DECODE_STAMP(7);
    if (CLUSTER) {
        cluster.sync();                                     // every block's sums have arrived; nobody is written to after this
        DECODE_STAMP(8);
        for (int slot = tid * 4; slot < share; slot += THREADS * 4) {
            const int i = me * share + slot;
            if (i >= nrows * D) break;
            const int r = i / D, col = i % D;
            float mx = -INFINITY;
            for (int sp = 0; sp < splits; ++sp) mx = fmaxf(mx, recv_ml[(sp * 16 + r) * 2]);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float den = 0.f;
            for (int sp = 0; sp < splits; ++sp) {           // in the order of the splits, whichever block merges
                const float2 ml = *reinterpret_cast<const float2*>(recv_ml + (sp * 16 + r) * 2);
                if (ml.x > -INFINITY) {
                    const float f = exp2f(ml.x - mx);
                    const float4 v = *reinterpret_cast<const float4*>(recv_o + sp * share + slot);
                    acc.x += v.x * f;
                    acc.y += v.y * f;
                    acc.z += v.z * f;
                    acc.w += v.w * f;
                    den += ml.y * f;
                }
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
            *reinterpret_cast<uint2*>((__nv_bfloat16*)a.out + ((size_t)tok0 * a.nq + head0 + r) * D + col) =
                make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        }
    }
    DECODE_STAMP(9);
    DECODE_SPAN(1);
}

// Raises the kernel's dynamic shared memory limit to `bytes` if it is lower (never lowers it).
template <int D, int STAGES>
static bool cluster_smem(size_t bytes) {
    static size_t granted = 0;
    if (bytes > granted) {
        if (cudaFuncSetAttribute(attention_mma_kernel<D, true, STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)bytes) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        granted = bytes;
    }
    return true;
}

// How many clusters of `splits` blocks of the decode kernel the device holds at once (asked once per head
// size, cluster size and shared-memory size, which grows with the query heads of a kv head; 0: such a cluster
// cannot be placed).
template <int D, int STAGES>
static int cluster_capacity(int splits, size_t smem) {
    static int known[MAX_CLUSTER + 1] = {};                     // 0 not asked, -1 none, else the count
    static size_t known_smem[MAX_CLUSTER + 1] = {};             // the shared memory the answer was given for
    if (known[splits] == 0 || known_smem[splits] != smem) {
        known_smem[splits] = smem;
        int clusters = 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, splits);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = splits;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        // more than 8 blocks a cluster is a size the device has to allow explicitly
        const bool ok = cluster_smem<D, STAGES>(smem) &&
                        (splits <= 8 || cudaFuncSetAttribute(attention_mma_kernel<D, true, STAGES, true>,
                                                             cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) &&
                        cudaOccupancyMaxActiveClusters(&clusters, attention_mma_kernel<D, true, STAGES, true>, &cfg) == cudaSuccess &&
                        clusters > 0;
        if (!ok) cudaGetLastError();
        known[splits] = ok ? clusters : -1;
    }
    return known[splits] > 0 ? known[splits] : 0;
}

// LILY_B200_DECODE_CLUSTER=0 keeps the splits on scratch and the combine kernel.
static bool cluster_enabled() {
    static const bool on = [] {
        const char* v = getenv("LILY_B200_DECODE_CLUSTER");
        return !(v && v[0] == '0');
    }();
    return on;
}

// Returns 0 on success, and in `merged` whether the kernel itself merged the splits into `out`.
template <int D, bool DECODE, int STAGES>
static int launch(const AttnArgs& a, dim3 grid, int page_shift, cudaStream_t stream, bool* merged) {
    size_t smem = stage_bytes<D, STAGES>(DECODE);
    // clusters pay when all of them are resident at once; over several rounds of blocks their placement costs
    // more than the combine kernel (measured: 32 requests x 8 kv heads x 7 splits 116 against 103 us)
    if (DECODE && STAGES == (D <= 128 ? LILY_DECODE_STAGES : 2) && a.splits >= 2 && a.splits <= MAX_CLUSTER && cluster_enabled()) {
        const int rows = a.nq / a.nkv < 16 ? a.nq / a.nkv : 16;
        const size_t with_recv = smem + ((size_t)a.splits * cluster_share(rows, D, a.splits) + (size_t)a.splits * 16 * 2) * sizeof(float);
        if ((long)grid.x * grid.y <= cluster_capacity<D, DECODE ? STAGES : 2>(a.splits, with_recv)) {
            auto kern = attention_mma_kernel<D, true, DECODE ? STAGES : 2, true>;
            if (!cluster_smem<D, DECODE ? STAGES : 2>(with_recv)) {
                set_error("attention_mma: cannot get %zu bytes of shared memory", with_recv);
                return 2;
            }
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = grid;
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = with_recv;
            cfg.stream = stream;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = a.splits;
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = pdl_enabled() ? 2 : 1;
            cudaLaunchKernelEx(&cfg, kern, a, page_shift);
            *merged = true;
            return 0;
        }
    }
    auto kern = attention_mma_kernel<D, DECODE, STAGES, false>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error("attention_mma: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return 2;
        }
        configured = true;
    }
    launch_pdl(kern, grid, dim3(THREADS), smem, stream, a, page_shift);
    *merged = false;
    return 0;
}

template <bool DECODE>
static int dispatch(const AttnArgs& a, dim3 grid, cudaStream_t stream, bool* merged) {
    int page_shift = 0;
    while ((1 << page_shift) < a.page_size) ++page_shift;
    if ((1 << page_shift) != a.page_size) {
        set_error("attention_mma: page_size %d is not a power of two", a.page_size);
        return 1;
    }
    constexpr int ST = DECODE ? LILY_DECODE_STAGES : 2;
    if (DECODE && a.stages != 0 && a.stages != ST) {
        // a third stage: 96 KB a block at head size 128, so two blocks a SM, each with two tiles on their way while it
        // works on a third.  Measured on a B200 (8 kv heads of 4 query heads, head size 128, one range a row, us, two
        // stages / three): 32 rows of 4,096 keys 109 / 82 (and 96 in 7 ranges with the combine kernel), 64 rows 181 in
        // 4 ranges / 168, 32 rows of 1,024 keys 31.6 / 24.2, 64 rows 58.7 / 48.0; 20 rows of 4,096 keys 89.5 / 78.9
        // (61.0 in two ranges of two stages: too few blocks for three stages).  Four stages, one block a SM: slower
        // everywhere (32 rows of 4,096 keys 122 us).
        if (a.stages != 3 || a.d > 128) {
            set_error("attention_mma: %d key/value stages at head size %d (2 everywhere, 3 up to head size 128)", a.stages, a.d);
            return 1;
        }
        if (a.d == 64) return launch<64, DECODE, DECODE ? 3 : 2>(a, grid, page_shift, stream, merged);
        return launch<128, DECODE, DECODE ? 3 : 2>(a, grid, page_shift, stream, merged);
    }
    switch (a.d) {
        case 64: return launch<64, DECODE, ST>(a, grid, page_shift, stream, merged);
        case 128: return launch<128, DECODE, ST>(a, grid, page_shift, stream, merged);
        case 192: return launch<192, DECODE, 2>(a, grid, page_shift, stream, merged);
        case 256: return launch<256, DECODE, 2>(a, grid, page_shift, stream, merged);
    }
    set_error("attention_mma: head_dim %d is not one of 64, 128, 192, 256", a.d);
    return 1;
}

}  // namespace mma
}  // namespace lily

using namespace lily;

// 1 when the tensor-core kernels take this head size (bfloat16 only); the caller uses the
// CUDA-core kernels otherwise.
LILY_API int lily_attention_mma_supports(int d) { return d == 64 || d == 128 || d == 192 || d == 256; }
LILY_API int lily_attention_prefill_mma_rows() { return 64; }

#ifdef LILY_DECODE_TIMING
// The cycle stamps of the last decode launch: [split (the first 16)][phase] (16 x 16 numbers).  Phases: 0 entry, 1 early tiles asked
// for, 2 the kernel before has finished, 3 queries in shared memory, 4 first tile landed, 5 all tiles done, 6 the
// four warps' results in shared memory, 7 sent to the cluster (or written), 8 the cluster's barrier passed, 9 exit.
LILY_API int lily_attention_decode_timing(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, mma::g_decode_stamps, sizeof(unsigned long long) * 256) == cudaSuccess ? 0 : 1;
}
// Entry and exit times (ns) of the first `blocks` blocks (x fastest, then y, then z) of the last decode launch.
LILY_API int lily_attention_decode_spans(unsigned long long* out, int blocks) {
    return cudaMemcpyFromSymbol(out, mma::g_decode_spans, sizeof(unsigned long long) * 2 * (blocks < 4096 ? blocks : 4096)) == cudaSuccess ? 0 : 1;
}
#endif

LILY_API int lily_attention_prefill_mma(const void* q, const void* kv, void* out, const int* block_table,
                                        int bt_stride, const int* cu_seqlens, const int* prefix_lens,
                                        const int* tile_req, const int* tile_start, int tiles, int nq, int nkv,
                                        int d, int page_size, int window, float scale, cudaStream_t stream) {
    if (tiles == 0) return 0;
    LILY_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_prefill: %d query heads over %d kv heads", nq, nkv);
    LILY_REQUIRE(nq <= 65535 && page_size > 0, "attention_prefill: nq=%d page_size=%d", nq, page_size);
    AttnArgs a{};
    a.q = q; a.kv = kv; a.out = out; a.block_table = block_table; a.bt_stride = bt_stride;
    a.cu_seqlens = cu_seqlens; a.prefix_lens = prefix_lens; a.tile_req = tile_req; a.tile_start = tile_start;
    a.splits = 1; a.nq = nq; a.nkv = nkv; a.d = d; a.page_size = page_size; a.window = window; a.scale = scale;
    bool merged = false;
    int rc = mma::dispatch<false>(a, dim3(tiles, nq), stream, &merged);
    if (rc) return rc;
    LILY_CHECK_LAUNCH("attention_prefill_mma");
    return 0;
}

extern "C" int lily_attention_combine(const float*, void*, int, int, int, int, int, cudaStream_t);

// Clusters of `splits` blocks of the decode kernel that the device holds at once for this head size and
// group size (0: none, or more splits than a cluster takes): with at most that many (request, kv head) pairs
// the kernel merges the splits inside clusters.
LILY_API int lily_attention_decode_mma_clusters(int d, int splits, int group) {
    if (splits < 2 || splits > mma::MAX_CLUSTER || !mma::cluster_enabled()) return 0;
    const int rows = group < 16 ? group : 16;
    const size_t recv = ((size_t)splits * mma::cluster_share(rows, d, splits) + (size_t)splits * 16 * 2) * sizeof(float);
    switch (d) {
        case 64: return mma::cluster_capacity<64, LILY_DECODE_STAGES>(splits, mma::stage_bytes<64, LILY_DECODE_STAGES>(true) + recv);
        case 128: return mma::cluster_capacity<128, LILY_DECODE_STAGES>(splits, mma::stage_bytes<128, LILY_DECODE_STAGES>(true) + recv);
        case 192: return mma::cluster_capacity<192, 2>(splits, mma::stage_bytes<192, 2>(true) + recv);
        case 256: return mma::cluster_capacity<256, 2>(splits, mma::stage_bytes<256, 2>(true) + recv);
    }
    return 0;
}

static int decode_mma(AttnArgs& a, const void* q, const void* kv, void* out, const int* block_table, int bt_stride,
                      const int* seq_lens, float* scratch, int requests, int splits, int nq, int nkv, int d, int page_size,
                      int window, float scale, int stages, cudaStream_t stream) {
    if (requests == 0) return 0;
    a.stages = stages;
    LILY_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_decode: %d query heads over %d kv heads", nq, nkv);
    LILY_REQUIRE(splits >= 1 && splits <= 65535 && page_size > 0, "attention_decode: splits=%d page_size=%d", splits, page_size);
    LILY_REQUIRE(splits == 1 || scratch != nullptr, "attention_decode: splits need scratch");
    const int group = nq / nkv, chunks = (group + 15) / 16;
    LILY_REQUIRE(nkv * chunks <= 65535, "attention_decode: %d kv heads", nkv);
    a.q = q; a.kv = kv; a.out = out; a.block_table = block_table; a.bt_stride = bt_stride; a.seq_lens = seq_lens;
    a.splits = splits; a.nq = nq; a.nkv = nkv; a.d = d; a.page_size = page_size; a.window = window; a.scale = scale;
    a.part_o = scratch;
    a.part_ml = scratch ? scratch + (size_t)requests * nq * splits * d : nullptr;
    bool merged = false;
    int rc = mma::dispatch<true>(a, dim3(requests, nkv * chunks, splits), stream, &merged);
    if (rc) return rc;
    LILY_CHECK_LAUNCH("attention_decode_mma");
    if (splits > 1 && !merged) return lily_attention_combine(scratch, out, requests, nq, d, splits, kBF16, stream);
    return 0;
}

// One query token per request over its cached keys, the keys cut into `splits` ranges.  With 2 to 16 splits (and all
// clusters resident at once) the blocks of a (request, kv head) form a cluster and merge their results through
// distributed shared memory; else the partial results go to `scratch` in the layout of attention_simt.cu
// ([requests, nq, splits, d] outputs, then [requests, nq, splits, 2] (max, sum)) and the combine kernel is launched behind.
// `stages`: 0, or the key/value tiles a block holds (3, up to head size 128: two blocks a SM, no clusters).
LILY_API int lily_attention_decode_mma(const void* q, const void* kv, void* out, const int* block_table,
                                       int bt_stride, const int* seq_lens, float* scratch, int requests, int splits,
                                       int nq, int nkv, int d, int page_size, int window, float scale, int stages,
                                       cudaStream_t stream) {
    AttnArgs a{};
    return decode_mma(a, q, kv, out, block_table, bt_stride, seq_lens, scratch, requests, splits, nq, nkv, d, page_size,
                      window, scale, stages, stream);
}

// The same from the qkv product itself ([planes][requests, (nq + 2 nkv) d], float32 partial sums or bfloat16 with
// one plane): the kernel norms and rotates its query heads (gains and tables optional, as in
// lily_qk_norm_rope_write) and, unless write_kv is 0, writes this step's key and value to the cache before it
// reads them, so that no kernel runs between the projection and the attention.
LILY_API int lily_attention_decode_mma_fused(const void* qkv, int qkv_planes, size_t qkv_stride, int qkv_dtype,
                                             const void* q_gain, const void* k_gain, int gain_dtype, float eps,
                                             const float* cos_t, const float* sin_t, int rd, int write_kv,
                                             void* kv, void* out, const int* block_table, int bt_stride,
                                             const int* seq_lens, float* scratch, int requests, int splits, int nq,
                                             int nkv, int d, int page_size, int window, float scale, int stages,
                                             cudaStream_t stream) {
    LILY_REQUIRE(qkv != nullptr && qkv_planes >= 1 && (qkv_dtype == kF32 || qkv_planes == 1),
                 "attention_decode_fused: %d planes of dtype %d", qkv_planes, qkv_dtype);
    LILY_REQUIRE(rd >= 0 && rd <= d && rd % 2 == 0, "attention_decode_fused: rotary_dim %d does not fit head_dim %d", rd, d);
    LILY_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "attention_decode_fused: q and k gains come together");
    LILY_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "attention_decode_fused: cos and sin tables come together");
    AttnArgs a{};
    a.qkv = qkv; a.qkv_planes = qkv_planes; a.qkv_stride = qkv_stride; a.qkv_f32 = qkv_dtype == kF32;
    a.q_gain = q_gain; a.k_gain = k_gain; a.gain_f32 = gain_dtype == kF32; a.eps = eps;
    a.cos_t = cos_t; a.sin_t = sin_t; a.rd = cos_t ? rd : 0; a.write_kv = write_kv;
    return decode_mma(a, nullptr, kv, out, block_table, bt_stride, seq_lens, scratch, requests, splits, nq, nkv, d,
                      page_size, window, scale, stages, stream);
}
