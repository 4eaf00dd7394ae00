// Weight-streaming matrix product for a few tokens (decode): parts[s][m][n] = sum over the s-th
// slice of k of x[m][k] * w[n][k], bfloat16 in, float32 out, M <= 64 tokens.
//
// At these sizes the product is bound by reading w once from HBM, so the kernel is built around
// that stream.  The weight rows are the 16-row side of mma.sync m16n8k16 and the tokens the
// 8-column side (as in lily/csrc/bf16_skinny.cu:1-6,45-96 of the reference).  Each warp owns 16 * MT
// weight rows and runs a pipeline of its own: STAGES tiles of [rows][64 k] are in flight with
// cp.async (16-byte pieces, 128 contiguous bytes per row and instruction) into the warp's private,
// XOR-swizzled ring in shared memory, and ldmatrix feeds the tensor cores from the oldest tile.
// Warps never wait for one another in the loop (no block barrier): with about 100 KB of loads in
// flight per SM the stream runs near HBM speed whatever the arithmetic does.  x is staged once per
// block in shared memory.
//
// The k range is cut into `ksplit` slices over blockIdx.y so that enough blocks stream at once to
// fill the device; each slice writes its own float32 partial sums and the kernel that consumes the
// product (norm, rotation, SiLU*mul) adds the slices up while it reads them, in a fixed order.
// Requires K % 64 == 0; N and M are free (M <= 64).
#include "common.cuh"

#include <cstdlib>

namespace lily {
namespace skinny {

constexpr int KB = 64;            // granule of k: K must be a multiple of it, slices are counted in it

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    // the hint lets L2 fetch the 256-byte line pair: a warp comes back for the other half of the pair with its next
    // tile, and DRAM serves longer bursts (measured on a B200: 8 x 4096 x 12288 in 17.8 us with the hint, 19.0 without)
    asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: 8-token tiles (M <= 8 * NT).  MT: 16-row tiles of w per warp.  WARPS per block.  KT: k per
// tile (64: 128 contiguous bytes of each row per copy round).  XSMEM: the block's slice of x is staged in shared
// memory; without it (a slice too long to fit beside the rings of two blocks a SM: deep products of wide models, or
// 9 to 16 tokens) every lane reads its own fragments of x from global memory, one tile of k ahead: x is small and
// stays in the caches, and all shared memory goes to the rings.
template <int NT, int MT, int WARPS, int STAGES, int KT, bool XSMEM>
__global__ void __launch_bounds__(WARPS * 32)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   float* __restrict__ parts, int M, int N, int K, int blocks_per_slice) {
    static_assert(XSMEM || (KT == 64 && NT <= 2), "x from global memory: tiles of 64 k, up to 16 tokens");
    constexpr int ROWS = 16 * MT;                     // weight rows per warp
    constexpr int PIECES = KT / 8;                    // 16-byte pieces per row of a tile
    constexpr int PITCH = KT * 2;                     // bytes per row of a tile
    constexpr int TILE = ROWS * PITCH;                // bytes of one warp tile
    constexpr int COPIES = ROWS * PIECES / 32;        // cp.async per lane and tile
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    unsigned char* ring = smem + (size_t)warp * STAGES * TILE;        // this warp's tiles
    unsigned char* xs = smem + (size_t)WARPS * STAGES * TILE;         // [NT * 8][slice k], 16-byte pieces swizzled
    const int kblocks = K / KT;                       // tiles along k (blocks_per_slice counts tiles too)
    const int kb0 = blockIdx.y * blocks_per_slice;
    const int nkb = max(0, min(blocks_per_slice, kblocks - kb0));
    const int row0 = (blockIdx.x * WARPS + warp) * ROWS;

    // copy i of this lane moves piece (32 i + lane) % PIECES of row (32 i + lane) / PIECES: a warp-wide
    // copy covers whole rows of the tile (4 rows of 128 bytes, or one row of 512); rows beyond N repeat the last row
    const __nv_bfloat16* src[COPIES];
    uint32_t dst[COPIES];
#pragma unroll
    for (int i = 0; i < COPIES; ++i) {
        const int r = (32 * i + lane) / PIECES, piece = (32 * i + lane) % PIECES;
        src[i] = w + (size_t)min(row0 + r, N - 1) * K + (size_t)kb0 * KT + piece * 8;
        dst[i] = (uint32_t)(r * PITCH + (((piece & ~7) | ((piece ^ r) & 7)) << 4));
    }
    auto issue = [&](int kb) {
        const uint32_t base = smem_u32(ring + (kb % STAGES) * TILE);
#pragma unroll
        for (int i = 0; i < COPIES; ++i) cp_async16(base + dst[i], src[i] + (size_t)kb * KT);
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {            // the weight stream starts before x is staged
        if (s < nkb) issue(s);
        cp_async_commit();
    }

    // x comes from the kernel before this one; the weights above do not, so their stream is
    // already running while that kernel drains
    pdl_wait();
    pdl_launch_dependents();

    // stage this slice of x: rows beyond M are zero
    const int chunks = nkb * PIECES;
    if (XSMEM) {
        for (int i = tid; i < NT * 8 * chunks; i += WARPS * 32) {
            const int r = i / chunks, ch = i % chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < M) v = *reinterpret_cast<const uint4*>(x + (size_t)r * K + (size_t)kb0 * KT + ch * 8);
            *reinterpret_cast<uint4*>(xs + ((size_t)r * chunks + (ch ^ (r & 7))) * 16) = v;
        }
        __syncthreads();
    }
    // without XSMEM: a lane's fragments of x for 64 k and token tile nt: token 8 nt + g, for each of the four k16
    // steps the pairs at 2c and 2c + 8
    constexpr int XT = XSMEM ? 1 : NT;
    uint32_t xf[XT][8], xnext[XT][8];
    auto load_x = [&](int kb, uint32_t (&f)[XT][8]) {
#pragma unroll
        for (int nt = 0; nt < XT; ++nt) {
            const int tok = nt * 8 + g;
            const uint32_t* p = reinterpret_cast<const uint32_t*>(x + (size_t)min(tok, M - 1) * K + (size_t)(kb0 + kb) * KT + 2 * c);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                f[nt][2 * kk] = tok < M ? __ldg(p + kk * 8) : 0u;
                f[nt][2 * kk + 1] = tok < M ? __ldg(p + kk * 8 + 4) : 0u;
            }
        }
    };
    if (!XSMEM && nkb > 0) load_x(0, xnext);

    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;

    for (int kb = 0; kb < nkb; ++kb) {
        cp_async_wait<STAGES - 2>();                  // this lane's pieces of tile kb have landed
        __syncwarp();                                 // ... and every lane's; the warp is done with tile kb - 1
        if (kb + STAGES - 1 < nkb) issue(kb + STAGES - 1);
        cp_async_commit();
        const uint32_t tile = smem_u32(ring + (kb % STAGES) * TILE);
        if (!XSMEM) {
#pragma unroll
            for (int nt = 0; nt < XT; ++nt)
#pragma unroll
                for (int j = 0; j < 8; ++j) xf[nt][j] = xnext[nt][j];
            if (kb + 1 < nkb) load_x(kb + 1, xnext);
        }
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            uint32_t a[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int r = mt * 16 + (lane & 15), ch = kk * 2 + (lane >> 4);
                ldmatrix_x4(tile + r * PITCH + (((ch & ~7) | ((ch ^ r) & 7)) << 4), a[mt][0], a[mt][1], a[mt][2], a[mt][3]);
            }
#pragma unroll
            for (int np = 0; np < (NT + 1) / 2; ++np) {
                // two token tiles at once: (tokens 0-7, k lo), (0-7, k hi), (8-15, k lo), (8-15, k hi)
                uint32_t b0, b1, b2, b3;
                const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int ch = kb * PIECES + kk * 2 + ((lane >> 3) & 1);
                const int rr = NT == 1 ? (lane & 7) : r;              // one tile only: both halves read tokens 0-7
                if (XSMEM) {
                    ldmatrix_x4(smem_u32(xs + ((size_t)rr * chunks + (ch ^ (rr & 7))) * 16), b0, b1, b2, b3);
                } else {
                    b0 = xf[2 * np < XT ? 2 * np : 0][2 * (kk & 3)];
                    b1 = xf[2 * np < XT ? 2 * np : 0][2 * (kk & 3) + 1];
                    b2 = xf[2 * np + 1 < XT ? 2 * np + 1 : 0][2 * (kk & 3)];
                    b3 = xf[2 * np + 1 < XT ? 2 * np + 1 : 0][2 * (kk & 3) + 1];
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    mma_bf16(acc[mt][2 * np], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
                    if (2 * np + 1 < NT) mma_bf16(acc[mt][2 * np + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
                }
            }
        }
    }

    float* out = parts + (size_t)blockIdx.y * M * N;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = row0 + mt * 16 + g + (e >> 1) * 8;
                const int tok = nt * 8 + 2 * c + (e & 1);
                if (row < N && tok < M) out[(size_t)tok * N + row] = acc[mt][nt][e];
            }
}

struct Shape {
    int nt, mt, warps, stages, kt;
};
// Measured and not kept: tiles of 256 k (512 contiguous bytes of a row per copy round) were no faster than
// tiles of 64 k and cost shared memory that x's slice needs; one 256-row block per SM over the whole k for a
// wide product (8 x 24576 x 4096) took 41.9 us against the library's 35.6 us.
static Shape shape_for(int M) {
    if (M <= 8) return {1, 1, 8, 5, 64};
    if (M <= 16) return {2, 1, 8, 4, 64};       // four stages: 16 rows of x of a ninth of the down product's k fit beside them
                                                // (9 to 16 tokens, Qwen3-8B sizes: the step 2 % shorter than with the library's down product)
    if (M <= 32) return {4, 2, 4, 5, 64};
    return {8, 2, 4, 5, 64};
}
static size_t smem_bytes(const Shape& s, int tiles_per_slice) {
    return (size_t)s.warps * s.stages * 16 * s.mt * s.kt * 2 + (size_t)s.nt * 8 * tiles_per_slice * s.kt * 2;
}

// Two blocks a SM: what a block may take of the SM's shared memory.
constexpr size_t kHalfSm = 112 * 1024;
static size_t ring_bytes(const Shape& s) { return (size_t)s.warps * s.stages * 16 * s.mt * s.kt * 2; }
// Whether the lanes read x from global memory: a slice of x that does not fit beside the rings, and few enough
// tokens that the lanes' own loads of x (4 bytes each, a token's row per group of four lanes) cost less than they
// save.  Measured against the library, us: K = 25600, N = 5120: 41.6 / 51.4 at 1 token, 45.0 / 49.3 at 2, 48.0 / 51.1 at
// 4, 52.6 / 48.2 at 8; K = 8192, N = 10240: 28.4 / 34.3 at 1, 33.4 / 35.3 at 4, 37.3 / 34.2 at 8; K = 28672, N = 8192:
// 74.5 / 79.7 at 1, 82.0 / 77.4 at 2; 16 tokens: twice the library's time everywhere.
static bool x_from_global(const Shape& s, int tiles_per_slice, int M, int K) {
    return s.nt <= 2 && smem_bytes(s, tiles_per_slice) > kHalfSm && (long long)M * K <= 2 * 25600;
}

template <int NT, int MT, int WARPS, int STAGES, int KT, bool XSMEM>
static int launch_form(const __nv_bfloat16* x, const __nv_bfloat16* w, float* parts, int M, int N, int K, int ksplit,
                       cudaStream_t stream) {
    const int tiles = K / KT;
    const int per = (tiles + ksplit - 1) / ksplit;
    const Shape sh{NT, MT, WARPS, STAGES, KT};
    const size_t smem = XSMEM ? smem_bytes(sh, per) : ring_bytes(sh);
    auto kern = skinny_gemm_kernel<NT, MT, WARPS, STAGES, KT, XSMEM>;
    static size_t granted = 48 * 1024;
    if (smem > granted) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error("skinny_gemm: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return 2;
        }
        granted = smem;
    }
    dim3 grid((N + WARPS * 16 * MT - 1) / (WARPS * 16 * MT), ksplit);
    launch_pdl(kern, grid, dim3(WARPS * 32), smem, stream, x, w, parts, M, N, K, per);
    return 0;
}

template <int NT, int MT, int WARPS, int STAGES, int KT>
static int launch(const __nv_bfloat16* x, const __nv_bfloat16* w, float* parts, int M, int N, int K, int ksplit,
                  cudaStream_t stream) {
    if constexpr (NT <= 2 && KT == 64) {
        const int tiles = K / KT;
        if (x_from_global(Shape{NT, MT, WARPS, STAGES, KT}, (tiles + ksplit - 1) / ksplit, M, K))
            return launch_form<NT, MT, WARPS, STAGES, KT, false>(x, w, parts, M, N, K, ksplit, stream);
    }
    return launch_form<NT, MT, WARPS, STAGES, KT, true>(x, w, parts, M, N, K, ksplit, stream);
}


// ---------------------------------------------------------------------------- gate/up product with SiLU*mul
//
// out[m][o] = silu(x[m] . gate[o]) * (x[m] . up[o]) for up to 8 tokens, the fused gate/up matrix streamed once.
//
// The fused matrix holds runs of `run` gate rows followed by the `run` up rows of the same outputs.  A warp owns 8
// outputs: the 16-row side of its mma tile is their 8 gate rows followed by their 8 up rows, so that a lane ends up
// with the gate and the up sum of the same (output, token) in its own accumulator and forms SiLU*mul in registers.
//
// The work is cut into units of (block of 8 * WARPS outputs, 64 k).  The units, row block after row block, are dealt
// out in equal contiguous stretches to a grid that is resident all at once (one block a SM), so every
// block streams the same number of bytes whatever the matrix's height: no ragged second round of blocks.  A stretch
// ends where it ends, usually in the middle of a row block's k range; a row block is therefore finished by two or
// three blocks.  Each leaves its partial sums in scratch and counts itself in; the one that counts in last adds all
// the partial sums up, in the order of their k ranges and not of their arrival, applies SiLU*mul and writes bfloat16.
// Nobody waits for anybody (no spinning), and the counter goes back to zero for the next launch.
template <int WARPS, int STAGES, bool XSMEM, int KT>
__global__ void __launch_bounds__(WARPS * 32)
skinny_swiglu_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     __nv_bfloat16* __restrict__ out, float* __restrict__ scratch, int* __restrict__ counters,
                     int M, int I, int K, int run, int row_blocks, int max_seg, int x_slots) {
    static_assert(!XSMEM || KT == 64, "x is staged in shared memory in blocks of 64 k");
    constexpr int PIECES = KT / 8, PITCH = KT * 2, TILE = 16 * PITCH, COPIES = KT / 16, OUTS = 8 * WARPS;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_arrived;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    unsigned char* ring = smem + (size_t)warp * STAGES * TILE;
    unsigned char* xs = smem + (size_t)WARPS * STAGES * TILE;          // [8 tokens][x_slots * 8 pieces], pieces swizzled
    const int kblocks = K / KT;
    const long long units = (long long)row_blocks * kblocks;
    const long long G = gridDim.x;
    const long long u0 = (long long)blockIdx.x * units / G, u1 = (long long)(blockIdx.x + 1) * units / G;
    const int n = (int)(u1 - u0);
    if (n <= 0) {                                       // more blocks than units: nothing to do, but keep the chain going
        pdl_wait();
        pdl_launch_dependents();
        return;
    }
    const bool x_by_unit = n <= kblocks;                // x is staged per unit of the stretch, else for every k block once
    const int chunks = x_slots * 8;

    // the weight stream: copy i of a lane moves piece (32 i + lane) % PIECES of tile row (32 i + lane) / PIECES
    int issue_rb = (int)(u0 / kblocks), issue_kb = (int)(u0 % kblocks), issued = 0;
    const __nv_bfloat16* src[COPIES];
    uint32_t dst[COPIES];
    auto rows_of = [&](int rb) {
#pragma unroll
        for (int i = 0; i < COPIES; ++i) {
            const int r = (32 * i + lane) / PIECES, piece = (32 * i + lane) % PIECES;
            const int o = min(rb * OUTS + warp * 8 + (r & 7), I - 1);
            const size_t row = (size_t)(o / run) * 2 * run + (o % run) + (size_t)(r >> 3) * run;
            src[i] = w + row * K + piece * 8;
            dst[i] = (uint32_t)(r * PITCH + (((piece & ~7) | ((piece ^ r) & 7)) << 4));
        }
    };
    rows_of(issue_rb);
    auto issue = [&]() {                                // the next unit of the stretch
        const uint32_t base = smem_u32(ring + (issued % STAGES) * TILE);
#pragma unroll
        for (int i = 0; i < COPIES; ++i) cp_async16(base + dst[i], src[i] + (size_t)issue_kb * KT);
        ++issued;
        if (++issue_kb == kblocks) {
            issue_kb = 0;
            rows_of(++issue_rb);
        }
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {              // the weights depend on no kernel: they start before the wait
        if (issued < n) issue();
        cp_async_commit();
    }
    pdl_wait();
    pdl_launch_dependents();

    // x of the k blocks this stretch meets; rows beyond M are zero.  (Without XSMEM the lanes read their share of
    // x from global memory, 64 k ahead: x is small and stays in the caches, and all shared memory goes to the rings.)
    const int first_kb = (int)(u0 % kblocks);
    const int staged = XSMEM ? (x_by_unit ? n : kblocks) : 0;
    for (int i = tid; i < 8 * staged * 8; i += WARPS * 32) {
        const int r = i / (staged * 8), rest = i % (staged * 8), slot = rest / 8, piece = rest % 8;
        const int kb = x_by_unit ? (first_kb + slot) % kblocks : slot;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < M) v = *reinterpret_cast<const uint4*>(x + (size_t)r * K + (size_t)kb * KT + piece * 8);
        const int ch = slot * 8 + piece;
        *reinterpret_cast<uint4*>(xs + ((size_t)r * chunks + (ch ^ (r & 7))) * 16) = v;
    }
    if (XSMEM) __syncthreads();

    // a lane's share of x for 64 k: token g, for each of the four k16 steps the pairs at 2c and 2c + 8
    const __nv_bfloat16* xrow = x + (size_t)min(g, M - 1) * K + 2 * c;
    uint32_t xf[8], xnext[8];
    auto load_x = [&](size_t k0, uint32_t (&f)[8]) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const uint32_t* p = reinterpret_cast<const uint32_t*>(xrow + k0 + kk * 16);
            f[2 * kk] = g < M ? __ldg(p) : 0u;
            f[2 * kk + 1] = g < M ? __ldg(p + 4) : 0u;
        }
    };
    if (!XSMEM) load_x((size_t)first_kb * KT, xnext);

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int rb = (int)(u0 / kblocks), kb = first_kb;
    for (int i = 0; i < n; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        if (issued < n) issue();
        cp_async_commit();
        const uint32_t tile = smem_u32(ring + (i % STAGES) * TILE);
        const int slot = x_by_unit ? i : kb;
#pragma unroll
        for (int q = 0; q < KT / 64; ++q) {             // 64 k at a time
            if (!XSMEM) {
#pragma unroll
                for (int j = 0; j < 8; ++j) xf[j] = xnext[j];
                // the next 64 k: of this unit, or the first of the next unit
                if (q + 1 < KT / 64) load_x((size_t)kb * KT + (q + 1) * 64, xnext);
                else if (i + 1 < n) load_x((size_t)(kb + 1 == kblocks ? 0 : kb + 1) * KT, xnext);
            }
#pragma unroll
            for (int kq = 0; kq < 4; ++kq) {
                const int kk = q * 4 + kq;
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                const int r = lane & 15, ch = kk * 2 + (lane >> 4);
                ldmatrix_x4(tile + r * PITCH + (((ch & ~7) | ((ch ^ r) & 7)) << 4), a0, a1, a2, a3);
                if (XSMEM) {
                    const int rr = lane & 7, xch = slot * 8 + kk * 2 + ((lane >> 3) & 1);
                    ldmatrix_x4(smem_u32(xs + ((size_t)rr * chunks + (xch ^ (rr & 7))) * 16), b0, b1, b2, b3);
                } else {
                    b0 = xf[2 * kq];
                    b1 = xf[2 * kq + 1];
                }
                mma_bf16(acc, a0, a1, a2, a3, b0, b1);
            }
        }
        const bool row_block_ends = kb == kblocks - 1;
        if (row_block_ends || i == n - 1) {
            // which blocks share this row block: block b holds unit u when b = ceil((u + 1) G / units) - 1
            const long long lo = (long long)rb * kblocks, hi = lo + kblocks - 1;
            const int b_first = (int)(((lo + 1) * G + units - 1) / units - 1);
            const int b_last = (int)(((hi + 1) * G + units - 1) / units - 1);
            const int nseg = b_last - b_first + 1, myseg = (int)blockIdx.x - b_first;
            bool finish = nseg == 1;
            if (!finish) {
                float4* mine = reinterpret_cast<float4*>(scratch) + ((size_t)rb * max_seg + myseg) * (WARPS * 32) + tid;
                *mine = make_float4(acc[0], acc[1], acc[2], acc[3]);
                __threadfence();
                __syncthreads();
                if (tid == 0) s_arrived = atomicAdd(&counters[rb], 1);
                __syncthreads();
                finish = s_arrived == nseg - 1;
                if (finish) {
                    __threadfence();
                    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                    const float4* all = reinterpret_cast<const float4*>(scratch) + (size_t)rb * max_seg * (WARPS * 32) + tid;
                    for (int s = 0; s < nseg; ++s) {            // in the order of the k ranges, whoever came last
                        const float4 v = __ldcg(all + (size_t)s * (WARPS * 32));
                        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
                    }
                    if (tid == 0) counters[rb] = 0;             // ready for the next launch
                }
                __syncthreads();                                // s_arrived is free again
            }
            if (finish) {
                // acc[0], acc[1]: gate sums of output o for tokens 2c, 2c + 1; acc[2], acc[3]: the up sums
                const int o = rb * OUTS + warp * 8 + g;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int tok = 2 * c + e;
                    const float gate = acc[e], up = acc[2 + e];
                    if (o < I && tok < M) out[(size_t)tok * I + o] = __float2bfloat16_rn(gate / (1.f + __expf(-gate)) * up);
                }
            }
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        }
        if (++kb == kblocks) {
            kb = 0;
            ++rb;
        }
    }
}

struct SwigluPlan {
    int grid, row_blocks, max_seg, x_slots;
    bool xsmem;
    size_t smem, scratch_floats;
};

// One block of 16 warps a SM, five tiles of 16 rows x 64 k in each warp's ring (160 KB, 128 KB of it in flight).
// Measured on a B200, 8 x 24576 x 4096: 38.0 us; eight warps and two blocks a SM 41.3; deeper rings (up to 192 KB in
// flight, x read from global memory to make room) 40.0 to 41.7; tiles of 128 and 256 k 40.5 to 40.7.
constexpr int SWIGLU_WARPS = 16, SWIGLU_STAGES = 5, SWIGLU_KT = 64;

// The grid and the scratch for a shape, or grid 0 when the kernel does not take it.  x of a block's stretch is
// staged in shared memory beside the rings when it fits (the faster form), else the lanes read it from global memory.
static SwigluPlan swiglu_plan(int M, int I, int K, int run) {
    SwigluPlan p = {};
    if (M < 1 || M > 8 || K < SWIGLU_KT || K % SWIGLU_KT != 0 || I < 8 || run < 8 || run % 8 != 0 || I % run != 0) return p;
    static const bool x_global = [] {
        const char* v = getenv("LILY_B200_SWIGLU_X");          // "global": never stage x in shared memory (for tests)
        return v && v[0] == 'g';
    }();
    const int outs = 8 * SWIGLU_WARPS, kblocks = K / SWIGLU_KT;
    p.row_blocks = (I + outs - 1) / outs;
    const long long units = (long long)p.row_blocks * kblocks;
    long long grid = sm_count();
    if (grid > units) grid = units;
    p.grid = (int)grid;
    const long long longest = (units + grid - 1) / grid, shortest = units / grid;
    const size_t rings = (size_t)SWIGLU_WARPS * SWIGLU_STAGES * 16 * SWIGLU_KT * 2;
    p.x_slots = (int)(longest <= kblocks ? longest : kblocks);
    p.xsmem = !x_global && rings + (size_t)8 * p.x_slots * 128 <= (size_t)226 * 1024;
    if (!p.xsmem) p.x_slots = 0;
    p.max_seg = (int)(kblocks / (shortest > 0 ? shortest : 1) + 2);
    p.smem = rings + (size_t)8 * p.x_slots * 128;
    p.scratch_floats = (size_t)p.row_blocks * p.max_seg * SWIGLU_WARPS * 32 * 4;
    return p;
}

template <bool XSMEM>
static int launch_swiglu(const SwigluPlan& p, const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* out,
                         float* scratch, int* counters, int M, int I, int K, int run, cudaStream_t stream) {
    auto kern = skinny_swiglu_kernel<SWIGLU_WARPS, SWIGLU_STAGES, XSMEM, SWIGLU_KT>;
    static size_t granted = 48 * 1024;
    if (p.smem > granted) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess) {
            set_error("skinny_swiglu: cannot get %zu bytes of shared memory: %s", p.smem, cudaGetErrorString(e));
            return 2;
        }
        granted = p.smem;
    }
    launch_pdl(kern, dim3(p.grid), dim3(SWIGLU_WARPS * 32), p.smem, stream, x, w, out, scratch, counters, M, I, K, run,
               p.row_blocks, p.max_seg, p.x_slots);
    return 0;
}

}  // namespace skinny
}  // namespace lily

using namespace lily;

LILY_API int lily_skinny_gemm_max_rows() { return 64; }

// Slices of k for this shape, or 0 when the library product is the better choice.  All blocks
// must run at once (two per SM): a second, partly filled wave of blocks costs as much as a full
// one.  So the kernel takes the shapes whose row blocks times slices fit one wave with slices of
// at least 8 tiles (the narrow, deep products: output and down projections) and leaves wide
// products, which the library streams well without cutting k, and more than 16 tokens to it.
LILY_API int lily_skinny_gemm_splits(int M, int N, int K) {
    if (K % skinny::KB != 0 || M < 1 || M > 16 || K < skinny::KB) return 0;
    const skinny::Shape sh = skinny::shape_for(M);
    const int rows_per_block = sh.warps * 16 * sh.mt;
    const int row_blocks = (N + rows_per_block - 1) / rows_per_block;
    const int tiles = K / sh.kt;
    const int held = sm_count() * 2;
    if (row_blocks > held / 2) return 0;
    int s = held / row_blocks;
    const int longest = tiles * sh.kt / 512 > 0 ? tiles * sh.kt / 512 : 1;      // slices of at least 512 k
    s = s < 1 ? 1 : (s > longest ? longest : s);
    // a slice of x that does not fit beside the rings: a few tokens read x from global memory instead; more
    // tokens take more, shorter slices while those still fit one wave
    if (!skinny::x_from_global(sh, (tiles + s - 1) / s, M, K))
        while (s < tiles && skinny::smem_bytes(sh, (tiles + s - 1) / s) > skinny::kHalfSm) ++s;
    return row_blocks * s <= held ? s : 0;
}

LILY_API int lily_skinny_gemm(const void* x, const void* w, float* parts, int M, int N, int K, int ksplit,
                              cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    LILY_REQUIRE(M >= 1 && M <= 64, "skinny_gemm: %d tokens (takes 1..64)", M);
    LILY_REQUIRE(K > 0 && K % skinny::KB == 0, "skinny_gemm: K=%d is not a multiple of %d", K, skinny::KB);
    const skinny::Shape sh = skinny::shape_for(M);
    LILY_REQUIRE(ksplit >= 1 && ksplit <= K / sh.kt, "skinny_gemm: %d slices of K=%d", ksplit, K);
    LILY_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "skinny_gemm: operands must be 16-byte aligned");
    const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
    int rc;
    if (M <= 8) rc = skinny::launch<1, 1, 8, 5, 64>(xp, wp, parts, M, N, K, ksplit, stream);
    else if (M <= 16) rc = skinny::launch<2, 1, 8, 4, 64>(xp, wp, parts, M, N, K, ksplit, stream);
    else if (M <= 32) rc = skinny::launch<4, 2, 4, 5, 64>(xp, wp, parts, M, N, K, ksplit, stream);
    else rc = skinny::launch<8, 2, 4, 5, 64>(xp, wp, parts, M, N, K, ksplit, stream);
    if (rc) return rc;
    LILY_CHECK_LAUNCH("skinny_gemm");
    return 0;
}

// Whether the fused gate/up product takes this shape, and what it needs: `scratch_floats` float32 of scratch and
// `counters` int32 that are zero before the first launch (the kernel leaves them zero).  Returns 0 for a shape the
// kernel does not take, 2 for one it takes but where the library product followed by SiLU*mul is the faster pair: wide
// inputs whose x does not fit beside the rings, so that the lanes read it from global memory, a cost that grows with
// the tokens (measured, x from global memory against the library: K = 5120, I = 25600: 84 / 94 us at 1 token, 86 / 95 at
// 4, 95 / 96 at 8; K = 8192, I = 28672: 145 / 151 at 1, 152 / 149 at 4, 162 / 145 at 8), and 1 otherwise.
LILY_API int lily_skinny_swiglu_need(int M, int I, int K, int run, size_t* scratch_floats, int* counters) {
    const skinny::SwigluPlan p = skinny::swiglu_plan(M, I, K, run);
    if (p.grid == 0) return 0;
    if (scratch_floats) *scratch_floats = p.scratch_floats;
    if (counters) *counters = p.row_blocks;
    return !p.xsmem && (long long)M * K > 3 * 8192 ? 2 : 1;
}

// out [M, I] bfloat16 = silu(x . gate^T) * (x . up^T); w [2 I, K] holds runs of `run` gate rows and the `run` up
// rows of the same outputs (run == I: all gate rows, then all up rows).
LILY_API int lily_skinny_swiglu(const void* x, const void* w, void* out, float* scratch, int* counters, int M, int I,
                                int K, int run, cudaStream_t stream) {
    if (M == 0 || I == 0) return 0;
    const skinny::SwigluPlan p = skinny::swiglu_plan(M, I, K, run);
    LILY_REQUIRE(p.grid > 0, "skinny_swiglu: does not take M=%d I=%d K=%d run=%d (1 to 8 tokens, K a multiple of 64, "
                 "I a multiple of run, run a multiple of 8)", M, I, K, run);
    LILY_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && scratch != nullptr && counters != nullptr,
                 "skinny_swiglu: operands must be 16-byte aligned and scratch and counters given");
    const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
    __nv_bfloat16* op = (__nv_bfloat16*)out;
    const int rc = p.xsmem ? skinny::launch_swiglu<true>(p, xp, wp, op, scratch, counters, M, I, K, run, stream)
                           : skinny::launch_swiglu<false>(p, xp, wp, op, scratch, counters, M, I, K, run, stream);
    if (rc) return rc;
    LILY_CHECK_LAUNCH("skinny_swiglu");
    return 0;
}
