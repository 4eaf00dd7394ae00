// bfloat16 matrix product on the fifth-generation tensor cores: C[M,N] = A[M,K] . B[N,K]^T with
// both operands k-contiguous, float32 accumulation in tensor memory, for the prefill-sized
// products of the step (M > 64 tokens).
//
// Blocks are persistent (one per SM) and walk the 128 x 256 output tiles in an order that keeps a
// panel of B in L2 while the blocks sweep M.  A block is warp specialised:
//   warp 0  one thread issues the TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the
//           A [128 x 64] and B [256 x 64] tiles of each k block into a ring of STAGES stages and
//           tells the stage's `full` mbarrier how many bytes to expect;
//   warp 1  allocates all 512 columns of tensor memory as two accumulators; one thread waits for
//           `full`, issues four tcgen05.mma (128 x 256 x 16, kind::f16) per k block from
//           shared-memory descriptors, and tcgen05.commit hands the stage back through its `empty`
//           mbarrier; a last commit per tile signals that accumulator's `ready`;
//   warps 2-9  wait for `ready`, read their 32-lane quarter and column half of the accumulator with tcgen05.ld
//           (32 columns at a time), apply the epilogue, store, and release the accumulator
//           (`drained`), so the epilogue of one tile runs under the products of the next.
// Epilogues: plain (bfloat16 out, optional bias) and SiLU*mul for a gate/up product whose weight
// rows are interleaved in blocks of 128 (rows [256 j, 256 j + 128) gate, the next 128 up), so that
// a tile holds gate and up of the same 128 outputs and the product leaves as [M, N / 2] without the
// [M, N] intermediate ever reaching memory (lily/models/llama.py:42-47 computes it in two steps).
//
// No cluster, no multicast: every block fetches its own tiles.  Every wait on an mbarrier is
// bounded; a wait that runs out sets a device-side status word (read by lily_gemm_tc_status),
// makes the block's roles leave their loops, and the block still frees its tensor memory.
// M, N and K need not be multiples of the tile: TMA fills what lies outside with zeros and the
// epilogue masks rows and columns.  K must be a multiple of 8 (16-byte row pitch).
#include "common.cuh"

#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace lily {
namespace tc {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 320;              // loader warp, mma warp, eight epilogue warps
constexpr uint32_t SPIN_LIMIT = 1u << 24;     // ~ a second of polling before a wait gives up

__device__ int g_status = 0;                  // 0 ok; else (code << 16 | block) of the first wait that gave up

enum Epilogue : int { kPlain = 0, kSiluMul = 1 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the phase of `parity`; gives up after SPIN_LIMIT polls or when another role has.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(&g_status, 0, (code << 16) | (int)(blockIdx.x + blockIdx.y * gridDim.x));
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptor of a k-major tile with 128-byte swizzle: rows of 128 bytes,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);            // start address
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride between 8-row groups
    d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void umma(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

template <int EPI>
__device__ __forceinline__ void epilogue_tile(uint32_t tbase, __nv_bfloat16* __restrict__ C,
                                              const __nv_bfloat16* __restrict__ bias, int row, int m_ok, int n0, int N,
                                              int ldc, int half) {
    if (EPI == kPlain) {
#pragma unroll 1
        for (int cc = half * (BN / 64); cc < (half + 1) * (BN / 64); ++cc) {   // this warp's half of the columns
            uint32_t r[32];
            tmem_ld32(tbase + cc * 32, r);
            const int col = n0 + cc * 32;
            if (m_ok && col < N) {
                __nv_bfloat16* dst = C + (size_t)row * ldc + col;
                if (col + 32 <= N && (ldc & 7) == 0) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        float f[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            f[e] = __uint_as_float(r[v * 8 + e]) + (bias ? __bfloat162float(bias[col + v * 8 + e]) : 0.f);
                        *reinterpret_cast<uint4*>(dst + v * 8) =
                            make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
                    }
                } else {
                    for (int e = 0; e < 32 && col + e < N; ++e)
                        dst[e] = __float2bfloat16_rn(__uint_as_float(r[e]) + (bias ? __bfloat162float(bias[col + e]) : 0.f));
                }
            }
        }
    } else {
        // columns [0, 128) of the tile are gate, [128, 256) up, of outputs n0 / 2 + [0, 128)
        const int out0 = n0 / 2;
#pragma unroll 1
        for (int cc = half * (BN / 128); cc < (half + 1) * (BN / 128); ++cc) {
            uint32_t gte[32], up[32];
            tmem_ld32(tbase + cc * 32, gte);
            tmem_ld32(tbase + BN / 2 + cc * 32, up);
            const int col = out0 + cc * 32;
            if (m_ok && col < N / 2) {
                __nv_bfloat16* dst = C + (size_t)row * ldc + col;
                float f[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const float gv = __uint_as_float(gte[e]);
                    f[e] = __fdividef(gv, 1.f + __expf(-gv)) * __uint_as_float(up[e]);
                }
                if (col + 32 <= N / 2 && (ldc & 7) == 0) {
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(pack2(f[v * 8], f[v * 8 + 1]), pack2(f[v * 8 + 2], f[v * 8 + 3]),
                                                                            pack2(f[v * 8 + 4], f[v * 8 + 5]), pack2(f[v * 8 + 6], f[v * 8 + 7]));
                } else {
                    for (int e = 0; e < 32 && col + e < N / 2; ++e) dst[e] = __float2bfloat16_rn(f[e]);
                }
            }
        }
    }
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the dynamic region is only guaranteed 16-byte alignment: round up to the 1024 the swizzle needs
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;
    const int m_blocks = (M + BM - 1) / BM, n_blocks = (N + BN - 1) / BN, tiles = m_blocks * n_blocks;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t ready0 = smem_u32(&bars[2 * STAGES]), drained0 = smem_u32(&bars[2 * STAGES + 2]);

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(ready0 + 8 * a, 1);
            mbar_init(drained0 + 8 * a, 8);                    // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    volatile int* abort_flag = &abort_s;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                        // k blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_blocks) * BM, n0 = (tile / m_blocks) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, abort_flag, 1);
                    if (!ok) break;
                    mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    const uint32_t a_dst = smem_u32(smem + s * STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, full0 + 8 * s, kb * BK, m0);
                    tma_load_2d(a_dst + A_BYTES, &map_b, full0 + 8 * s, kb * BK, n0);
                }
            }
            if (*abort_flag) {
                // copies already issued still land in this block's shared memory: give each a bounded wait
                for (int j = max(0, it - STAGES); j < it; ++j)
                    for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1); ++i) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // kind::f16, bfloat16 a and b (k-major), float32 d, n = 256, m = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
                const int acc = local & 1;
                ok = mbar_wait(drained0 + 8 * acc, ((local >> 1) & 1) ^ 1, abort_flag, 4);   // the epilogue has emptied it
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t tacc = tmem + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1, abort_flag, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint64_t da = smem_desc(smem_u32(smem + s * STAGE_BYTES));
                    const uint64_t db = smem_desc(smem_u32(smem + s * STAGE_BYTES + A_BYTES));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)       // 16 k = 32 bytes further inside the swizzled row
                        umma(tacc, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb | kk) != 0 ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);               // the stage is free once these have read it
                }
                umma_commit(ready0 + 8 * acc);                 // arrives when this tile's products are done
            }
        }
    } else {
        const int quarter = warp & 3;                          // the 32 lanes of tensor memory this warp may read
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const int acc = local & 1;
            const int m0 = (tile % m_blocks) * BM, n0 = (tile / m_blocks) * BN;
            if (!mbar_wait(ready0 + 8 * acc, (local >> 1) & 1, abort_flag, 3)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            epilogue_tile<EPI>(tmem + acc * BN + ((uint32_t)(quarter * 32) << 16), C, bias, row, row < M, n0, N, ldc, (warp - 2) >> 2);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(drained0 + 8 * acc);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * BN) : "memory");
    }
}

// ---- the same product over pairs of blocks ---------------------------------------------------------
//
// Two blocks of a cluster (two SMs) work on one 256 x 256 output tile with `tcgen05.mma.cta_group::2`:
// each block loads its own 128 rows of A and its own 128 of the tile's 256 rows of B, the even
// block's mma thread issues 256 x 256 x 16 products that read A from both blocks (128 rows each) and B
// from both (one half each), and each block ends up with its 128 rows of the tile in its own tensor
// memory.  Per block and k step that is 32 KB of operands for twice the arithmetic of the one-block
// kernel's 48 KB, and the tensor cores run at their full rate, which one-block products do not reach.
//   * the `full` barrier of a stage lives in the even block; both blocks' TMA loads complete their
//     bytes on it (`cp.async.bulk.tensor ... cta_group::2`) and the even block's loader announces the
//     sum of both;
//   * `empty` and `ready` are in each block and the mma thread's commits reach both at once
//     (`tcgen05.commit ... multicast::cluster`);
//   * `drained` lives in the even block; the epilogue warps of both blocks arrive there.
// Every wait is bounded as in the one-block kernel; both blocks meet at a cluster barrier before
// they free tensor memory.

constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_BYTES = 128 * BK * 2;                 // this block's half of the B tile
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of the same variable in block `rank` of the cluster.
__device__ __forceinline__ uint32_t in_block(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_in_even_block, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar_in_even_block), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, when the products issued so far are done, on the barrier at this offset in both blocks.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_in_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar_in_cluster) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * PAIR_STAGES + 4];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                      // 0: the block whose mma thread issues for both
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int num_kb = (K + BK - 1) / BK;
    const int m_blocks = (M + 2 * BM - 1) / (2 * BM), n_blocks = (N + BN - 1) / BN, tiles = m_blocks * n_blocks;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[PAIR_STAGES]);
    const uint32_t ready0 = smem_u32(&bars[2 * PAIR_STAGES]), drained0 = smem_u32(&bars[2 * PAIR_STAGES + 2]);

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);                       // waited on in the even block only
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(ready0 + 8 * a, 1);
            mbar_init(drained0 + 8 * a, 16);                   // the eight epilogue warps of each block (even block's copy)
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                        // both blocks' barriers exist before anyone signals the other's
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    volatile int* abort_flag = &abort_s;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < tiles && ok; tile += pairs) {
                const int m0 = (tile % m_blocks) * 2 * BM + (int)rank * BM, n0 = (tile / m_blocks) * BN + (int)rank * 128;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    ok = mbar_wait(empty0 + 8 * s, ((it / PAIR_STAGES) & 1) ^ 1, abort_flag, 1);
                    if (!ok) break;
                    const uint32_t full_even = in_block(full0 + 8 * s, 0);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * PAIR_STAGE_BYTES);     // this block's bytes and the other's
                    const uint32_t a_dst = smem_u32(smem + s * PAIR_STAGE_BYTES);
                    tma_load_2d_pair(a_dst, &map_a, full_even, kb * BK, m0);
                    tma_load_2d_pair(a_dst + A_BYTES, &map_b, full_even, kb * BK, n0);
                }
            }
            if (*abort_flag && rank == 0) {
                for (int j = max(0, it - PAIR_STAGES); j < it; ++j)
                    for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(full0 + 8 * (j % PAIR_STAGES), (j / PAIR_STAGES) & 1); ++i) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // kind::f16, bfloat16 a and b (k-major), float32 d, n = 256, m = 256 over the two blocks
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < tiles && ok; tile += pairs, ++local) {
                const int acc = local & 1;
                ok = mbar_wait(drained0 + 8 * acc, ((local >> 1) & 1) ^ 1, abort_flag, 4);   // both blocks' epilogues have emptied it
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t tacc = tmem + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    ok = mbar_wait(full0 + 8 * s, (it / PAIR_STAGES) & 1, abort_flag, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint64_t da = smem_desc(smem_u32(smem + s * PAIR_STAGE_BYTES));
                    const uint64_t db = smem_desc(smem_u32(smem + s * PAIR_STAGE_BYTES + A_BYTES));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)
                        umma_pair(tacc, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb | kk) != 0 ? 1u : 0u);
                    umma_commit_pair(empty0 + 8 * s);          // the stage is free in both blocks once these have read it
                }
                umma_commit_pair(ready0 + 8 * acc);            // both blocks' epilogues may read their half
            }
        }
    } else {
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = pair; tile < tiles; tile += pairs, ++local) {
            const int acc = local & 1;
            const int m0 = (tile % m_blocks) * 2 * BM + (int)rank * BM, n0 = (tile / m_blocks) * BN;
            if (!mbar_wait(ready0 + 8 * acc, (local >> 1) & 1, abort_flag, 3)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int row = m0 + quarter * 32 + lane;
            epilogue_tile<EPI>(tmem + acc * BN + ((uint32_t)(quarter * 32) << 16), C, bias, row, row < M, n0, N, ldc, (warp - 2) >> 2);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(in_block(drained0 + 8 * acc, 0));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                        // nobody frees tensor memory or leaves while the other block works
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * BN) : "memory");
    }
}

// ---- host side: tensor maps -----------------------------------------------------------------

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    });
    return fn;
}

// A [rows, k] bfloat16 matrix with k contiguous, read in boxes of [box_rows, 64].
static int make_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
    EncodeTiled enc = encoder();
    LILY_REQUIRE(enc != nullptr, "gemm_tc: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    LILY_REQUIRE(rc == CUDA_SUCCESS, "gemm_tc: cuTensorMapEncodeTiled failed with %d (rows=%d k=%d ld=%d)", (int)rc, rows, k, ld);
    return 0;
}

// LILY_B200_GEMM_PAIR=0 keeps every product on the one-block kernel.
static bool pair_enabled() {
    static const bool on = [] {
        const char* v = getenv("LILY_B200_GEMM_PAIR");
        return !(v && v[0] == '0');
    }();
    return on;
}

template <int EPI>
static int launch(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldc,
                  cudaStream_t stream) {
    const int sms = sm_count();
    // The pair form works on 256 rows at a time: an odd number of 128-row blocks costs it a whole block of padding,
    // which up to some 2,000 rows is more than the pair's better rate gives back (gate/up product of Qwen3-8B, pair /
    // one block, us: 320 rows 76.5 / 64.7, 384 78.5 / 66.5, 896 149.2 / 140.1, 1152 179.6 / 170.2; even counts: 448
    // 80.5 / 84.7, 768 112.9 / 117.7, 1536 211.2 / 220.9).
    const int row_blocks = (M + BM - 1) / BM;
    if (pair_enabled() && M > BM && !(row_blocks % 2 == 1 && row_blocks <= 15)) {
        // pairs of blocks on 256 x 256 tiles
        CUtensorMap ma, mb;
        if (make_map(&ma, A, M, K, lda, BM)) return 1;
        if (make_map(&mb, B, N, K, K, 128)) return 1;
        const size_t smem = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 1024;
        auto kern = gemm_tc_pair_kernel<EPI>;
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) {
                set_error("gemm_tc: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
                return 2;
            }
            configured = true;
        }
        const long tiles = (long)((N + BN - 1) / BN) * ((M + 2 * BM - 1) / (2 * BM));
        const long pairs = tiles < sms / 2 ? tiles : sms / 2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(2 * pairs));
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, kern, ma, mb, (__nv_bfloat16*)C, (const __nv_bfloat16*)bias, M, N, K, ldc);
        return 0;
    }
    CUtensorMap ma, mb;
    if (make_map(&ma, A, M, K, lda, BM)) return 1;
    if (make_map(&mb, B, N, K, K, BN)) return 1;
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
    auto kern = gemm_tc_kernel<EPI>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error("gemm_tc: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return 2;
        }
        configured = true;
    }
    const long tiles = (long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
    dim3 grid((unsigned)(tiles < sms ? tiles : sms));
    kern<<<grid, THREADS, smem, stream>>>(ma, mb, (__nv_bfloat16*)C, (const __nv_bfloat16*)bias, M, N, K, ldc);
    return 0;
}

}  // namespace tc
}  // namespace lily

using namespace lily;

// 0 while no wait has given up since the last call; else (code << 16 | block): code 1 the loader
// waiting for a free stage, 2 the mma thread waiting for a tile, 3 the epilogue waiting for an
// accumulator, 4 the mma thread waiting for the epilogue to drain one.  Synchronises the device.
// Reading clears it.
LILY_API int lily_gemm_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(tc::g_status, &zero, sizeof(int));
    return v;
}

// epilogue 0: C [M, N] = A . B^T (+ bias [N]).  epilogue 1: C [M, N / 2] = silu(gate) * up where the
// rows of B alternate between 128 gate rows and the 128 up rows of the same outputs (N % 256 == 0).
LILY_API int lily_gemm_tc(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldc,
                          int epilogue, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    LILY_REQUIRE(K > 0 && K % 8 == 0 && lda % 8 == 0 && lda >= K, "gemm_tc: K=%d, lda=%d must be multiples of 8", K, lda);
    LILY_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)B % 16 == 0) && ((uintptr_t)C % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
    int rc;
    if (epilogue == tc::kSiluMul) {
        LILY_REQUIRE(N % 256 == 0 && bias == nullptr && ldc >= N / 2, "gemm_tc: the SiLU*mul epilogue takes N %% 256 == 0 and no bias");
        rc = tc::launch<tc::kSiluMul>(A, B, C, nullptr, M, N, K, lda, ldc, stream);
    } else {
        LILY_REQUIRE(epilogue == tc::kPlain && ldc >= N, "gemm_tc: epilogue %d, ldc %d", epilogue, ldc);
        rc = tc::launch<tc::kPlain>(A, B, C, bias, M, N, K, lda, ldc, stream);
    }
    if (rc) return rc;
    LILY_CHECK_LAUNCH("gemm_tc");
    return 0;
}
