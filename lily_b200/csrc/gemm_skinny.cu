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

namespace lily {
namespace skinny {

constexpr int KB = 64;            // granule of k: K must be a multiple of it, slices are counted in it

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
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
// tile (64: 128 contiguous bytes of each row per copy round).
template <int NT, int MT, int WARPS, int STAGES, int KT>
__global__ void __launch_bounds__(WARPS * 32)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   float* __restrict__ parts, int M, int N, int K, int blocks_per_slice) {
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
    for (int i = tid; i < NT * 8 * chunks; i += WARPS * 32) {
        const int r = i / chunks, ch = i % chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < M) v = *reinterpret_cast<const uint4*>(x + (size_t)r * K + (size_t)kb0 * KT + ch * 8);
        *reinterpret_cast<uint4*>(xs + ((size_t)r * chunks + (ch ^ (r & 7))) * 16) = v;
    }
    __syncthreads();

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
                ldmatrix_x4(smem_u32(xs + ((size_t)rr * chunks + (ch ^ (rr & 7))) * 16), b0, b1, b2, b3);
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
    if (M <= 16) return {2, 1, 8, 5, 64};
    if (M <= 32) return {4, 2, 4, 5, 64};
    return {8, 2, 4, 5, 64};
}
static size_t smem_bytes(const Shape& s, int tiles_per_slice) {
    return (size_t)s.warps * s.stages * 16 * s.mt * s.kt * 2 + (size_t)s.nt * 8 * tiles_per_slice * s.kt * 2;
}

template <int NT, int MT, int WARPS, int STAGES, int KT>
static int launch(const __nv_bfloat16* x, const __nv_bfloat16* w, float* parts, int M, int N, int K, int ksplit,
                  cudaStream_t stream) {
    const int tiles = K / KT;
    const int per = (tiles + ksplit - 1) / ksplit;
    const size_t smem = smem_bytes(Shape{NT, MT, WARPS, STAGES, KT}, per);
    auto kern = skinny_gemm_kernel<NT, MT, WARPS, STAGES, KT>;
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
    while (s < tiles && skinny::smem_bytes(sh, (tiles + s - 1) / s) > 112 * 1024) ++s;
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
    else if (M <= 16) rc = skinny::launch<2, 1, 8, 5, 64>(xp, wp, parts, M, N, K, ksplit, stream);
    else if (M <= 32) rc = skinny::launch<4, 2, 4, 5, 64>(xp, wp, parts, M, N, K, ksplit, stream);
    else rc = skinny::launch<8, 2, 4, 5, 64>(xp, wp, parts, M, N, K, ksplit, stream);
    if (rc) return rc;
    LILY_CHECK_LAUNCH("skinny_gemm");
    return 0;
}
