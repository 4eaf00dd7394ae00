// Paged causal grouped-query attention on CUDA cores, any head size up to 256, float32
// accumulation: the kernels of the 32-bit path, and of bfloat16 where no tensor-core kernel
// takes the shape.
//
// Cache layout of one layer: [pages, 2 (keys, values), kv_heads, page_size, head_dim]; a
// request's block table gives the page of each run of page_size positions.
//
//  * prefill: grid (query tiles, query heads).  A tile is up to 32 consecutive new tokens of one
//    request; their keys are the request's cached prefix and the new tokens up to each query
//    (all written to the cache before this kernel runs).
//  * decode: grid (requests, kv heads x row chunks, splits).  One new token per request; the
//    query heads that share a kv head are the rows; the keys are cut into `splits` ranges whose
//    partial (max, sum, output) go to scratch and are merged by the combine kernel.
//
// Scores q.k * scale, keys visible when key position <= query position (and > query position -
// window when a window is given), softmax and p.v in float32: the formulas of
// lily/layers/attention/torch_native_backend.py:31-37,52-77; the split over keys follows
// lily/layers/attention/triton_ops/decode_attention.py:21-157, the prefix + new tokens form
// lily/layers/attention/triton_ops/extend_attention.py:17-169.
#include "attention_args.cuh"
#include "common.cuh"

namespace lily {

constexpr int ROWS = 32;      // query rows per block
constexpr int KEYS = 32;      // keys per tile (one per lane)
constexpr int WARPS = 4;
constexpr int RPW = ROWS / WARPS;


template <typename T, int DCH, bool DECODE>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const AttnArgs a) {
    extern __shared__ float smem[];
    const int d = a.d;
    float* Qs = smem;                          // [ROWS][d]
    float* Ks = Qs + ROWS * d;                 // [KEYS][d + 1]
    float* Vs = Ks + KEYS * (d + 1);           // [KEYS][d]
    float* Ps = Vs + KEYS * d;                 // [WARPS][RPW][KEYS]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* q = (const T*)a.q;
    const T* kv = (const T*)a.kv;
    T* out = (T*)a.out;
    const int group = a.nq / a.nkv;

    int req, kvh, kbeg, kend, nrows;
    int row_tok[RPW], row_head[RPW], row_pos[RPW];
    bool row_ok[RPW];
    if (DECODE) {
        req = blockIdx.x;
        const int chunks = (group + ROWS - 1) / ROWS;
        kvh = blockIdx.y / chunks;
        const int r0 = (blockIdx.y % chunks) * ROWS;
        const int seq = a.seq_lens[req];
        const int lo = (a.window > 0 && seq > a.window) ? seq - a.window : 0;
        int per = (seq - lo + a.splits - 1) / a.splits;
        per = (per + KEYS - 1) / KEYS * KEYS;
        kbeg = lo + blockIdx.z * per;
        kend = min(seq, kbeg + per);
        nrows = min(ROWS, group - r0);
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = i * WARPS + warp;            // interleaved: few rows still use every warp
            row_ok[i] = r < nrows;
            row_tok[i] = req;
            row_head[i] = kvh * group + r0 + r;
            row_pos[i] = seq - 1;
        }
    } else {
        const int tile = blockIdx.x;
        req = a.tile_req[tile];
        const int start = a.tile_start[tile];
        const int tok0 = a.cu_seqlens[req], len = a.cu_seqlens[req + 1] - tok0;
        const int prefix = a.prefix_lens[req];
        const int head = blockIdx.y;
        kvh = head / group;
        nrows = min(ROWS, len - start);
        kend = prefix + start + nrows;
        kbeg = (a.window > 0 && prefix + start + 1 > a.window) ? prefix + start + 1 - a.window : 0;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp * RPW + i;
            row_ok[i] = r < nrows;
            row_tok[i] = tok0 + start + r;
            row_head[i] = head;
            row_pos[i] = prefix + start + r;
        }
    }

    // stage the queries (float32)
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = DECODE ? i * WARPS + warp : warp * RPW + i;
        const T* src = q + ((size_t)row_tok[i] * a.nq + row_head[i]) * d;
        for (int c = lane; c < d; c += 32) Qs[r * d + c] = row_ok[i] ? to_float(src[c]) : 0.f;
    }

    float m[RPW], l[RPW], acc[RPW][DCH];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < DCH; ++c) acc[i][c] = 0.f;
    }

    const int* table = a.block_table + (size_t)req * a.bt_stride;
    const size_t head_stride = (size_t)a.page_size * d;            // one head's tile in a page
    const size_t page_stride = 2 * (size_t)a.nkv * head_stride;

    for (int kb = kbeg; kb < kend; kb += KEYS) {
        __syncthreads();
        // load the key and value tiles: KEYS rows of d, a warp per row at a time
        for (int j = warp; j < KEYS; j += WARPS) {
            const int kpos = kb + j;
            if (kpos < kend) {
                const int page = table[kpos / a.page_size];
                const T* ksrc = kv + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)(kpos % a.page_size) * d;
                const T* vsrc = ksrc + (size_t)a.nkv * head_stride;
                for (int c = lane; c < d; c += 32) {
                    Ks[j * (d + 1) + c] = to_float(ksrc[c]);
                    Vs[j * d + c] = to_float(vsrc[c]);
                }
            } else {
                for (int c = lane; c < d; c += 32) {
                    Ks[j * (d + 1) + c] = 0.f;
                    Vs[j * d + c] = 0.f;
                }
            }
        }
        __syncthreads();

        // scores: lane j holds key kb + j for each of the warp's rows
        float s[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) s[i] = 0.f;
        const float* krow = Ks + lane * (d + 1);
        for (int c = 0; c < d; ++c) {
            const float kval = krow[c];
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const int r = DECODE ? i * WARPS + warp : warp * RPW + i;
                s[i] = fmaf(Qs[r * d + c], kval, s[i]);
            }
        }
        const int kpos = kb + lane;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const bool seen = row_ok[i] && kpos < kend && kpos <= row_pos[i] &&
                              (a.window <= 0 || kpos > row_pos[i] - a.window);
            const float sv = seen ? s[i] * a.scale : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(sv));
            float p = 0.f, alpha = 1.f;
            if (m_new > -INFINITY) {
                alpha = expf(m[i] - m_new);
                p = expf(sv - m_new);
            }
            l[i] = l[i] * alpha + warp_sum(p);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < DCH; ++c) acc[i][c] *= alpha;
            Ps[(warp * RPW + i) * KEYS + lane] = p;
        }
        __syncwarp();
        // p.v: lane owns output columns lane, lane + 32, ...
        for (int j = 0; j < KEYS; ++j) {
            float v[DCH];
#pragma unroll
            for (int c = 0; c < DCH; ++c) {
                const int col = lane + 32 * c;
                v[c] = col < d ? Vs[j * d + col] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const float p = Ps[(warp * RPW + i) * KEYS + j];
#pragma unroll
                for (int c = 0; c < DCH; ++c) acc[i][c] = fmaf(p, v[c], acc[i][c]);
            }
        }
        __syncwarp();
    }

#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        if (!row_ok[i]) continue;
        if (DECODE && a.splits > 1) {
            const size_t base = ((size_t)row_tok[i] * a.nq + row_head[i]) * a.splits + blockIdx.z;
#pragma unroll
            for (int c = 0; c < DCH; ++c) {
                const int col = lane + 32 * c;
                if (col < d) a.part_o[base * d + col] = acc[i][c];
            }
            if (lane == 0) {
                a.part_ml[base * 2] = m[i];
                a.part_ml[base * 2 + 1] = l[i];
            }
        } else {
            const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
            T* dst = out + ((size_t)row_tok[i] * a.nq + row_head[i]) * d;
#pragma unroll
            for (int c = 0; c < DCH; ++c) {
                const int col = lane + 32 * c;
                if (col < d) dst[col] = from_float<T>(acc[i][c] * inv);
            }
        }
    }
}

// Merges the partial results of the splits: grid (requests, query heads), threads over d.  With 9 to 256 splits the
// block has four rows of threads and first brings every split's (max, sum) into shared memory, one a thread, and
// forms the weights exp(m - max) there; each row of threads then sums every fourth split, loads that do not wait for
// one another, and the first row adds the four partial sums up, in a fixed order.  (With dozens of splits the plain
// loops are a chain of trips to L2: 22 us for 55 splits.)  Fewer splits (where the staging costs more than it saves:
// a step of 64 requests with 4 splits each 10.44 -> 10.53 ms) and more take the plain loops, a column in the order of
// the splits.
constexpr int COMBINE_STAGED = 256, COMBINE_ROWS = 4, COMBINE_D = 256;
static bool combine_staged(int splits, int d) { return splits > 8 && splits <= COMBINE_STAGED && d <= COMBINE_D; }

template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         T* __restrict__ out, int nq, int d, int splits) {
    __shared__ float w_s[COMBINE_STAGED], l_s[COMBINE_STAGED];
    __shared__ float red[32];
    __shared__ float sums[COMBINE_ROWS - 1][COMBINE_D];
    pdl_enter_small();
    const size_t base = ((size_t)blockIdx.x * nq + blockIdx.y) * splits;
    if (blockDim.y > 1) {                                   // the launcher's choice: combine_staged(splits, d)
        const int tid = threadIdx.y * blockDim.x + threadIdx.x, threads = blockDim.x * blockDim.y;
        float mx = -INFINITY;
        for (int s = tid; s < splits; s += threads) {
            const float2 ml = *reinterpret_cast<const float2*>(part_ml + (base + s) * 2);
            w_s[s] = ml.x;
            l_s[s] = ml.y;
            mx = fmaxf(mx, ml.x);
        }
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if ((tid & 31) == 0) red[tid >> 5] = mx;
        __syncthreads();
        mx = red[0];
        for (int w = 1; w < (threads + 31) / 32; ++w) mx = fmaxf(mx, red[w]);
        for (int s = tid; s < splits; s += threads) w_s[s] = w_s[s] > -INFINITY ? expf(w_s[s] - mx) : 0.f;
        __syncthreads();
        const int rows = blockDim.y, row = threadIdx.y;
        float part[COMBINE_D / 128];                          // blockDim.x is 128: a thread has up to two columns
#pragma unroll
        for (int j = 0; j < COMBINE_D / 128; ++j) {
            const int c = threadIdx.x + j * 128;
            float o = 0.f;
            if (c < d) {
#pragma unroll 4
                for (int s = row; s < splits; s += rows) {
                    const float v = part_o[(base + s) * d + c];
                    if (w_s[s] != 0.f) o += v * w_s[s];        // a split without keys has weight 0 whatever it left
                }
                if (row > 0) sums[row - 1][c] = o;
            }
            part[j] = o;
        }
        __syncthreads();
        if (row == 0) {
            float denom = 0.f;
            for (int s = 0; s < splits; ++s) denom += l_s[s] * w_s[s];
            const float inv = denom > 0.f ? 1.f / denom : 0.f;
#pragma unroll
            for (int j = 0; j < COMBINE_D / 128; ++j) {
                const int c = threadIdx.x + j * 128;
                if (c < d) {
                    float o = part[j];
                    for (int r = 1; r < rows; ++r) o += sums[r - 1][c];
                    out[((size_t)blockIdx.x * nq + blockIdx.y) * d + c] = from_float<T>(o * inv);
                }
            }
        }
        return;
    }
    float mx = -INFINITY;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_ml[(base + s) * 2]);
    float denom = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = part_ml[(base + s) * 2];
        if (ms > -INFINITY) denom += part_ml[(base + s) * 2 + 1] * expf(ms - mx);
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = part_ml[(base + s) * 2];
            if (ms > -INFINITY) o += part_o[(base + s) * d + c] * expf(ms - mx);
        }
        out[((size_t)blockIdx.x * nq + blockIdx.y) * d + c] = from_float<T>(o * inv);
    }
}

static size_t smem_bytes(int d) { return sizeof(float) * ((size_t)ROWS * d + KEYS * (d + 1) + KEYS * d + ROWS * KEYS); }

template <typename T, bool DECODE>
static int launch(const AttnArgs& a, dim3 grid, cudaStream_t stream) {
    const int dch = (a.d + 31) / 32;
    const size_t smem = smem_bytes(a.d);
#define CASE(N)                                                                                          \
    case N: {                                                                                            \
        auto kern = attention_simt_kernel<T, N, DECODE>;                                                 \
        static size_t granted = 48 * 1024;      /* set once per size, never while a graph is captured */  \
        if (smem > granted) {                                                                            \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) { set_error("attention: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); return 2; } \
            granted = smem;                                                                              \
        }                                                                                                \
        kern<<<grid, WARPS * 32, smem, stream>>>(a);                                                     \
        break;                                                                                           \
    }
    switch (dch) {
        CASE(1) CASE(2) CASE(3) CASE(4) CASE(5) CASE(6) CASE(7) CASE(8)
        default:
            set_error("attention: head_dim %d is beyond the 256 this kernel takes", a.d);
            return 1;
    }
#undef CASE
    return 0;
}

static int check_common(const char* name, int nq, int nkv, int d, int page_size) {
    LILY_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "%s: %d query heads do not group over %d kv heads", name, nq, nkv);
    LILY_REQUIRE(d > 0 && d <= 256, "%s: head_dim %d is outside 1..256", name, d);
    LILY_REQUIRE(page_size > 0, "%s: page_size %d", name, page_size);
    return 0;
}

}  // namespace lily

using namespace lily;

LILY_API int lily_attention_prefill_simt(const void* q, const void* kv, void* out, const int* block_table,
                                         int bt_stride, const int* cu_seqlens, const int* prefix_lens,
                                         const int* tile_req, const int* tile_start, int tiles, int nq, int nkv,
                                         int d, int page_size, int window, float scale, int dtype,
                                         cudaStream_t stream) {
    if (tiles == 0) return 0;
    if (check_common("attention_prefill", nq, nkv, d, page_size)) return 1;
    LILY_REQUIRE(nq <= 65535, "attention_prefill: %d query heads", nq);
    AttnArgs a{};
    a.q = q; a.kv = kv; a.out = out; a.block_table = block_table; a.bt_stride = bt_stride;
    a.cu_seqlens = cu_seqlens; a.prefix_lens = prefix_lens; a.tile_req = tile_req; a.tile_start = tile_start;
    a.splits = 1; a.nq = nq; a.nkv = nkv; a.d = d; a.page_size = page_size; a.window = window; a.scale = scale;
    dim3 grid(tiles, nq);
    int rc = dtype == kBF16 ? launch<__nv_bfloat16, false>(a, grid, stream) : launch<float, false>(a, grid, stream);
    if (rc) return rc;
    LILY_CHECK_LAUNCH("attention_prefill");
    return 0;
}

// Merges the partial results that a split-key decode kernel left in `scratch`
// ([requests, nq, splits, d] outputs, then [requests, nq, splits, 2] (max, sum)).
LILY_API int lily_attention_combine(const float* scratch, void* out, int requests, int nq, int d, int splits,
                                    int dtype, cudaStream_t stream) {
    if (requests == 0 || splits <= 1) return 0;
    const float* part_o = scratch;
    const float* part_ml = scratch + (size_t)requests * nq * splits * d;
    dim3 cgrid(requests, nq), cblock(128, combine_staged(splits, d) ? COMBINE_ROWS : 1);
    if (dtype == kBF16)
        launch_pdl(attention_combine_kernel<__nv_bfloat16>, cgrid, cblock, 0, stream, (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, nq, d, splits);
    else
        launch_pdl(attention_combine_kernel<float>, cgrid, cblock, 0, stream, (const float*)part_o, (const float*)part_ml, (float*)out, nq, d, splits);
    LILY_CHECK_LAUNCH("attention_combine");
    return 0;
}

// Rows of a prefill tile: the host cuts each request's new tokens into tiles of this many.
LILY_API int lily_attention_prefill_simt_rows() { return ROWS; }

LILY_API size_t lily_attention_decode_scratch_floats(int requests, int nq, int d, int splits) {
    return splits > 1 ? (size_t)requests * nq * splits * (d + 2) : 0;
}

LILY_API int lily_attention_decode_simt(const void* q, const void* kv, void* out, const int* block_table,
                                        int bt_stride, const int* seq_lens, float* scratch, int requests,
                                        int splits, int nq, int nkv, int d, int page_size, int window,
                                        float scale, int dtype, cudaStream_t stream) {
    if (requests == 0) return 0;
    if (check_common("attention_decode", nq, nkv, d, page_size)) return 1;
    LILY_REQUIRE(splits >= 1 && splits <= 65535, "attention_decode: %d splits", splits);
    LILY_REQUIRE(splits == 1 || scratch != nullptr, "attention_decode: splits need scratch");
    const int group = nq / nkv, chunks = (group + ROWS - 1) / ROWS;
    AttnArgs a{};
    a.q = q; a.kv = kv; a.out = out; a.block_table = block_table; a.bt_stride = bt_stride;
    a.seq_lens = seq_lens; a.splits = splits; a.nq = nq; a.nkv = nkv; a.d = d; a.page_size = page_size;
    a.window = window; a.scale = scale;
    a.part_o = scratch;
    a.part_ml = scratch ? scratch + (size_t)requests * nq * splits * d : nullptr;
    dim3 grid(requests, nkv * chunks, splits);
    LILY_REQUIRE(grid.y <= 65535, "attention_decode: %d kv heads", nkv);
    int rc = dtype == kBF16 ? launch<__nv_bfloat16, true>(a, grid, stream) : launch<float, true>(a, grid, stream);
    if (rc) return rc;
    LILY_CHECK_LAUNCH("attention_decode");
    if (splits > 1) {
        dim3 cgrid(requests, nq), cblock(128, combine_staged(splits, d) ? COMBINE_ROWS : 1);
        if (dtype == kBF16)
            launch_pdl(attention_combine_kernel<__nv_bfloat16>, cgrid, cblock, 0, stream, (const float*)a.part_o, (const float*)a.part_ml, (__nv_bfloat16*)out, nq, d, splits);
        else
            launch_pdl(attention_combine_kernel<float>, cgrid, cblock, 0, stream, (const float*)a.part_o, (const float*)a.part_ml, (float*)out, nq, d, splits);
        LILY_CHECK_LAUNCH("attention_combine");
    }
    return 0;
}
