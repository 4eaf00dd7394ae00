// Causal paged attention for prefill on the fifth-generation tensor cores (bfloat16, head sizes 128 and 64;
// the numbers below are for 128, where a row of Q, K or V is two 128-byte sub-tiles; 64 has one):
// both products of a tile, S = Q K^T and O += P V, are tcgen05.mma instructions with their
// accumulators in tensor memory, the operands arrive by TMA, and the softmax runs two threads per
// query row straight out of tensor memory.  (The reference runs prefill attention through a
// library: lily/layers/attention/flashinfer_backend.py:188-203.)
//
// Two kernels.  The first: one block works on 128 new tokens of one request and one query head,
// walking the keys in tiles of 128 from the first the window allows to the last the causal rule
// allows.  Its ten warps:
//   warp 0   one thread issues the TMA loads: Q once (two [128 x 64] boxes, 128-byte swizzle), then
//            for each tile K and V as [64 keys x 64 features] boxes taken from the request's pages
//            (a box never crosses a page: the page size is a multiple of 64), into two stages each;
//   warp 1   allocates tensor memory (S twice, 128 columns each, and O, 128 columns); one thread
//            issues S_{j+1} = Q K_{j+1}^T (eight 128 x 128 x 16 products, both operands k-major)
//            before it waits for P_j, then O += P_j V_j (V is read as it lies in the cache,
//            [key][feature], which is the MN-major form of the B operand), so that the tensor cores
//            work on the next scores while the softmax of the current ones runs;
//   warps 2-9  two threads per query row, each with 64 of the tile's 128 keys: read their half of the
//            row of S from tensor memory (tcgen05.ld), mask the tiles on the diagonal and at the
//            window's edge, agree on the row's maximum, keep the running maximum and sum in float32,
//            write P = exp2(s * scale - max) as bfloat16 pairs over the tensor-memory columns of the S
//            tile it came from, where the second product reads it as its A operand, and at the end
//            divide their half of O by the sum and store it.
// The second kernel (further down) gives a block two query heads of one kv head, a softmax group each,
// and is the one that runs when the group size is even and the prompt long enough to fill the device.
// The maximum that P is taken against only moves when the true maximum has grown by more than 2^8
// since (then O and the sum are rescaled by the threads that own the row, in tensor memory), so
// the usual tile costs no pass over O; the result is the same quotient of sums either way.
//
// Keys past the request's length and rows past its new tokens are computed on whatever the pages
// hold (the cache is finite everywhere: it starts as zeros) and masked: P is exactly 0 for the
// former and the latter are not stored.  Every wait on an mbarrier is bounded; a wait that runs out
// sets a status word (lily_attention_tc_status), the roles leave their loops and the block frees
// its tensor memory.
#include "common.cuh"

#include <cuda.h>

#include <cstdlib>
#include <mutex>

namespace lily {
namespace fa {

constexpr int BQ = 128;                   // query rows per block
constexpr int BKV = 128;                  // keys per tile
// head sizes: 128 and 64 (the kernels are templates over D; a row of Q, K or V is D / 64 sub-tiles of 128 bytes)
// P (the second product's A operand) either goes through shared memory, or, packed as bfloat16
// pairs, into the tensor-memory columns of the S tile it was computed from; the latter leaves
// shared memory to K, V and Q alone (a third K/V stage fits) and spares the async-proxy fence.
#ifndef LILY_FA_PARTS
#define LILY_FA_PARTS 2
#endif
constexpr int PARTS = LILY_FA_PARTS;      // softmax threads per query row (2 or 4), each with 128 / PARTS of a tile's keys
#ifdef LILY_FA_P_IN_SMEM
constexpr bool P_TMEM = false;
constexpr int STAGES = 2;                 // K stages, V stages
#else
constexpr bool P_TMEM = true;
constexpr int STAGES = PARTS == 2 ? 3 : 2;
#endif
constexpr int SBUF = 2;                   // S accumulators (and P buffers)
constexpr int SUB = 128 * 64 * 2;         // a [128 rows][64 elements] sub-tile with 128-byte rows: 16 KB
constexpr int tile_bytes(int d) { return d / 64 * SUB; }      // Q, one K stage, one V stage: 128 rows of d features
constexpr int P_TILE = 2 * SUB;           // a P buffer in shared memory: 128 rows x 128 keys
constexpr int BOX = 64 * 64 * 2;          // one TMA box of K or V: 8 KB
constexpr int SOFTMAX_THREADS = PARTS * 128;
constexpr int THREADS = 64 + SOFTMAX_THREADS;
constexpr int NUM_BARS = 1 + 4 * STAGES + 3 * SBUF;
// shared memory, all of it dynamic and 1024-byte aligned: Q | K stages | V stages | P buffers | mbarriers |
// tensor-memory base and abort flag | the row maxima and sums that the two threads of a row exchange
constexpr int off_p(int d) { return (1 + 2 * STAGES) * tile_bytes(d); }
constexpr int off_bars(int d) { return off_p(d) + (P_TMEM ? 0 : SBUF) * P_TILE; }
constexpr int off_misc(int d) { return off_bars(d) + 8 * NUM_BARS + 8; }
constexpr int off_xch(int d) { return off_misc(d) + 16; }
constexpr int smem_one(int d) { return off_xch(d) + 2 * PARTS * BQ * 4; }
constexpr uint32_t SPIN_LIMIT = 1u << 24;
constexpr float GROW_LOG2 = 8.f;          // the reference maximum moves when the true one is 2^8 ahead

__device__ int g_status = 0;              // 0 ok; else (code << 24 | block) of the first wait that gave up

// Built with -DLILY_FA_TIMING, block (0, 0) adds up the cycles its roles spend in each phase
// (lily_attention_tc_timing reads them); without it the macros vanish.
#ifdef LILY_FA_TIMING
__device__ unsigned long long g_timing[32];
#define FA_TIC() const long long tic__ = clock64()
#define FA_TOC(slot, who) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (who)) g_timing[slot] += (unsigned long long)(clock64() - tic__); } while (0)
#else
#define FA_TIC() do {} while (0)
#define FA_TOC(slot, who) do {} while (0)
#endif

struct Params {
    const int* block_table;
    const int* cu_seqlens;
    const int* prefix_lens;
    const int* tile_req;
    const int* tile_start;
    __nv_bfloat16* out;
    int bt_stride, tiles, nq, nkv, page_size, window;
    float scale_log2;                     // softmax scale times log2(e)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(&g_status, 0, (code << 24) | (int)((blockIdx.x + blockIdx.y * gridDim.x) & 0xFFFFFF));
    return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// k-major operand tile with 128-byte swizzle: rows of 128 bytes, groups of eight rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operand ([k][n] with n contiguous) with 128-byte swizzle: a row of 64 n per k, groups of
// eight k 1024 bytes apart (stride field), the next 64 n `SUB` bytes further (leading field).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(SUB >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory (128 lanes x k / 2 columns of bfloat16 pairs).
__device__ __forceinline__ void umma_ts(uint32_t tmem_c, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(tmem_c), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// 32 consecutive columns of this thread's lane of tensor memory; follow with tmem_wait_ld().
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* r) {
    uint32_t* u = reinterpret_cast<uint32_t*>(r);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
                   "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]),
                   "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]),
                   "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* r) {
    const uint32_t* u = reinterpret_cast<const uint32_t*>(r);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};\n"
                 ::"r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
                   "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]),
                   "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]),
                   "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31]),
                   "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* r) {
    const uint32_t* u = reinterpret_cast<const uint32_t*>(r);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};\n"
                 ::"r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
                   "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]),
                   "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const Params p) {
    static_assert(D == 64 || D == 128, "head sizes 64 and 128");
    static_assert(D / PARTS % 32 == 0, "a softmax thread's share of a row of O comes in pieces of 32 columns");
    constexpr int TILE = tile_bytes(D), DH = D / 64;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off_bars(D));
    uint32_t& tmem_base_s = *reinterpret_cast<uint32_t*>(smem + off_misc(D));
    int& abort_s = *reinterpret_cast<int*>(smem + off_misc(D) + 4);
    float* xch = reinterpret_cast<float*>(smem + off_xch(D));   // [tile parity][half][row]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((smem_u32(smem) & 1023u) != 0) {                        // the swizzled tiles need it; never seen, but checked
        if (threadIdx.x == 0) atomicCAS(&g_status, 0, (11 << 24) | (int)((blockIdx.x + blockIdx.y * gridDim.x) & 0xFFFFFF));
        return;
    }

    const uint32_t q_smem = smem_u32(smem);
    const uint32_t k_smem = q_smem + TILE, v_smem = k_smem + STAGES * TILE, p_smem = v_smem + STAGES * TILE;
    const uint32_t q_full = smem_u32(&bars[0]);
    const uint32_t k_full = q_full + 8, k_empty = k_full + 8 * STAGES, v_full = k_empty + 8 * STAGES,
                   v_empty = v_full + 8 * STAGES, s_full = v_empty + 8 * STAGES, p_full = s_full + 8 * SBUF,
                   pv_done = p_full + 8 * SBUF;

    if (threadIdx.x == 0) {
        abort_s = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(k_full + 8 * s, 1);
            mbar_init(k_empty + 8 * s, 1);
            mbar_init(v_full + 8 * s, 1);
            mbar_init(v_empty + 8 * s, 1);
        }
        for (int s = 0; s < SBUF; ++s) {
            mbar_init(s_full + 8 * s, 1);
            mbar_init(p_full + 8 * s, SOFTMAX_THREADS); // one arrival per softmax thread
            mbar_init(pv_done + 8 * s, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    for (int i = threadIdx.x; i < PARTS * BQ; i += THREADS) {    // exchange slots start with the tag before their first
        reinterpret_cast<uint32_t*>(xch)[i] = 3u;                                 // parity 0: tags 1, 3, 1, ...
        reinterpret_cast<uint32_t*>(xch)[PARTS * BQ + i] = 0u;                    // parity 1: tags 2, 0, 2, ...
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    const uint32_t tmem_o = tmem + 2 * BKV;
    volatile int* abort_flag = &abort_s;

    // q and the cache come from the kernels before this one
    pdl_wait();
    pdl_launch_dependents();

    // the tiles were listed in order of position: the last ones, which see the most keys, go first
    const int tile = p.tiles - 1 - (int)blockIdx.y;
    const int head = blockIdx.x;
    const int req = p.tile_req[tile], start = p.tile_start[tile];
    const int q_begin = p.cu_seqlens[req];
    const int new_len = p.cu_seqlens[req + 1] - q_begin;
    const int rows_valid = min(BQ, new_len - start);
    const int pos0 = p.prefix_lens[req] + start;         // position of the tile's first row
    const int kv_end = pos0 + rows_valid;                // keys the last row sees, exclusive
    const int k_lo = (p.window > 0 && pos0 + 1 > p.window) ? pos0 + 1 - p.window : 0;
    const int jt0 = k_lo / BKV;
    const int n = (kv_end - 1) / BKV - jt0 + 1;          // key tiles of this block (>= 1)

    if (warp == 0) {
        if (lane == 0) {
            const int kvh = head / (p.nq / p.nkv);
            const int* table = p.block_table + (size_t)req * p.bt_stride;
            mbar_expect_tx(q_full, TILE);
            for (int dh = 0; dh < DH; ++dh) tma_load_3d(q_smem + dh * SUB, &map_q, q_full, dh * 64, head, q_begin + start);
            bool ok = true;
            int issued_k = 0, issued_v = 0;
            for (int j = 0; j < n && ok; ++j) {
                const int s = j % STAGES;
                const uint32_t par = (uint32_t)((j / STAGES) & 1);
                int page[2], off[2];
                for (int h = 0; h < 2; ++h) {            // the two 64-key boxes of the tile
                    const int key = (jt0 + j) * BKV + 64 * h;
                    const bool held = key < kv_end;
                    page[h] = held ? table[key / p.page_size] : 0;
                    off[h] = held ? key % p.page_size : 0;
                }
                { FA_TIC(); ok = mbar_wait(k_empty + 8 * s, par ^ 1, abort_flag, 1); FA_TOC(0, true); }
                if (!ok) break;
                mbar_expect_tx(k_full + 8 * s, TILE);
                for (int h = 0; h < 2; ++h)
                    for (int dh = 0; dh < DH; ++dh)
                        tma_load_4d(k_smem + s * TILE + dh * SUB + h * BOX, &map_kv, k_full + 8 * s, dh * 64, off[h], kvh, page[h]);
                ++issued_k;
                { FA_TIC(); ok = mbar_wait(v_empty + 8 * s, par ^ 1, abort_flag, 2); FA_TOC(1, true); }
                if (!ok) break;
                mbar_expect_tx(v_full + 8 * s, TILE);
                for (int h = 0; h < 2; ++h)
                    for (int dh = 0; dh < DH; ++dh)
                        tma_load_4d(v_smem + s * TILE + dh * SUB + h * BOX, &map_kv, v_full + 8 * s, dh * 64, off[h], p.nkv + kvh, page[h]);
                ++issued_v;
            }
            if (*abort_flag) {
                // copies already issued still land in this block's shared memory: give each a bounded wait
                for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(q_full, 0); ++i) {}
                for (int j = max(0, issued_k - STAGES); j < issued_k; ++j)
                    for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(k_full + 8 * (j % STAGES), (j / STAGES) & 1); ++i) {}
                for (int j = max(0, issued_v - STAGES); j < issued_v; ++j)
                    for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(v_full + 8 * (j % STAGES), (j / STAGES) & 1); ++i) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // kind::f16: float32 accumulator, bfloat16 a and b, n = 128, m = 128; bit 16 makes b MN-major
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKV >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            bool ok = mbar_wait(q_full, 0, abort_flag, 3);
            auto scores = [&](int i) {                   // S_i = Q K_i^T into accumulator i % 2
                const int s = i % STAGES;
                {
                    FA_TIC();
                    const bool got = mbar_wait(k_full + 8 * s, (uint32_t)((i / STAGES) & 1), abort_flag, 4);
                    FA_TOC(2, true);
                    if (!got) return false;
                }
                tc_fence_after();
                // the descriptors of the eight k steps differ from the tile's by constants (address field in 16-byte units)
                const uint64_t dq = desc_k_major(q_smem), dk = desc_k_major(k_smem + s * TILE);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t inside = (uint64_t)(((kk >> 2) * SUB + (kk & 3) * 32) >> 4);
                    umma(tmem + (uint32_t)(i & 1) * BKV, dq + inside, dk + inside, idesc_s, kk != 0 ? 1u : 0u);
                }
                umma_commit(k_empty + 8 * s);
                umma_commit(s_full + 8 * (i & 1));
                return true;
            };
            if (ok) ok = scores(0);
            for (int j = 0; j < n && ok; ++j) {
                const int s = j % STAGES, b = j & 1;
                if (j + 1 < n) {
                    ok = scores(j + 1);
                    if (!ok) break;
                }
                { FA_TIC(); ok = mbar_wait(p_full + 8 * b, (uint32_t)((j >> 1) & 1), abort_flag, 5); FA_TOC(4, true); }
                if (ok) { FA_TIC(); ok = mbar_wait(v_full + 8 * s, (uint32_t)((j / STAGES) & 1), abort_flag, 6); FA_TOC(3, true); }
                if (!ok) break;
                tc_fence_after();
                const uint64_t dv = desc_mn_major(v_smem + s * TILE), dp = desc_k_major(p_smem + b * P_TILE);
#pragma unroll
                for (int kk = 0; kk < BKV / 16; ++kk) {
                    const uint64_t db = dv + (uint64_t)(kk * 2048 >> 4);
                    if (P_TMEM) {
                        // A from tensor memory: 16 keys of P are 8 columns of bfloat16 pairs in S's buffer
                        umma_ts(tmem_o, tmem + (uint32_t)(b * BKV + kk * 8), db, idesc_o, (j | kk) != 0 ? 1u : 0u);
                    } else {
                        umma(tmem_o, dp + (uint64_t)(((kk >> 2) * SUB + (kk & 3) * 32) >> 4), db, idesc_o, (j | kk) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(v_empty + 8 * s);
                umma_commit(pv_done + 8 * b);
            }
        }
    } else {
        // PARTS threads share a query row, each with COLS of a tile's keys (warps 2-5 the first COLS keys,
        // the next four warps the next, ...); a warp reads the quarter of tensor memory (32 lanes = 32
        // query rows) that its index modulo 4 names
        constexpr int COLS = BKV / PARTS, OCOLS = D / PARTS;
        const int quarter = warp & 3, part = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int pos = pos0 + row;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        // The threads of a row hand each other one float per tile (the maximum of their keys; at the end
        // their sum) through words of shared memory whose two lowest mantissa bits carry a sequence
        // tag, so a reader knows the word is this tile's without a barrier that an aborted partner
        // would never reach.  Slots alternate with the tile's parity; every thread drops the same two
        // bits of its own value, so all agree on the result.  `combine` folds the values in part order.
        volatile uint32_t* xw = reinterpret_cast<volatile uint32_t*>(xch);
        auto exchange = [&](int seq, float mine, bool sum, float& result) {
            const uint32_t tag = (uint32_t)(seq + 1) & 3u;
            const uint32_t bits = __float_as_uint(mine) & ~3u;
            xw[((seq & 1) * PARTS + part) * BQ + row] = bits | tag;
            float acc = sum ? 0.f : -INFINITY;
#pragma unroll
            for (int q = 0; q < PARTS; ++q) {
                float v = __uint_as_float(bits);
                if (q != part) {
                    volatile uint32_t* from = xw + ((seq & 1) * PARTS + q) * BQ + row;
                    bool got = false;
                    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
                        const uint32_t w = *from;
                        if ((w & 3u) == tag) {
                            v = __uint_as_float(w & ~3u);
                            got = true;
                            break;
                        }
                        if ((i & 1023u) == 1023u && *abort_flag) return false;
                    }
                    if (!got) {
                        *abort_flag = 1;
                        atomicCAS(&g_status, 0, (12 << 24) | (int)((blockIdx.x + blockIdx.y * gridDim.x) & 0xFFFFFF));
                        return false;
                    }
                }
                acc = sum ? acc + v : fmaxf(acc, v);
            }
            result = acc;
            return true;
        };
        for (int j = 0; j < n && ok; ++j) {
            const int b = j & 1;
            { FA_TIC(); ok = mbar_wait(s_full + 8 * b, (uint32_t)((j >> 1) & 1), abort_flag, 7); FA_TOC(8 + (part & 1), row == 0); }
            if (!ok) break;
            FA_TIC();
            tc_fence_after();
            float s[COLS];
#pragma unroll
            for (int c = 0; c < COLS / 32; ++c) tmem_ld32(tmem + lane_addr + (uint32_t)(b * BKV + part * COLS + c * 32), s + c * 32);
            tmem_wait_ld();
            FA_TOC(10 + (part & 1), row == 0);
            const int kb = (jt0 + j) * BKV + part * COLS;
            const bool need_mask = kb + COLS - 1 > pos0 || (p.window > 0 && kb <= pos0 + BQ - 1 - p.window);
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < COLS; ++c) {
                    const int key = kb + c;
                    const bool seen = key <= pos && (p.window <= 0 || key > pos - p.window);
                    s[c] = seen ? s[c] : -INFINITY;
                }
            }
            float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
            for (int c = 4; c < COLS; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
            const float mine = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            FA_TOC(18 + (part & 1), row == 0);
            float row_max;
            ok = exchange(j, mine, false, row_max);
            if (!ok) break;
            FA_TOC(20 + (part & 1), row == 0);
            const float m_new = fmaxf(m_used, row_max);
            if (j == 0) {
                m_used = m_new;
            } else {
                const bool grow = (m_new - m_used) * p.scale_log2 > GROW_LOG2;      // also when m_used is -inf
                if (__any_sync(0xffffffffu, grow)) {
                    // O must hold every product up to tile j - 1 before its rows are rescaled
                    ok = mbar_wait(pv_done + 8 * ((j - 1) & 1), (uint32_t)(((j - 1) >> 1) & 1), abort_flag, 8);
                    if (!ok) break;
                    tc_fence_after();
                    const float alpha = grow ? ex2((m_used - m_new) * p.scale_log2) : 1.f;
                    if (grow) m_used = m_new;
                    l *= alpha;
#pragma unroll 1
                    for (int c = 0; c < OCOLS / 32; ++c) {     // this thread's share of the row of O
                        float o[32];
                        tmem_ld32(tmem_o + lane_addr + (uint32_t)(part * OCOLS + c * 32), o);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] *= alpha;
                        tmem_st32(tmem_o + lane_addr + (uint32_t)(part * OCOLS + c * 32), o);
                    }
                    tmem_wait_st();
                }
            }
            FA_TOC(22 + (part & 1), row == 0);
            const float mb = (m_used == -INFINITY ? 0.f : m_used) * p.scale_log2;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < COLS; ++c) {
                s[c] = ex2(fmaf(s[c], p.scale_log2, -mb));
                sum4[c & 3] += s[c];
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            FA_TOC(12 + (part & 1), row == 0);
            if (P_TMEM) {
                // P over the first 64 columns of the S buffer it came from: this thread's 64 keys are 32
                // columns of bfloat16 pairs.  The other thread of the row has read its scores (it posted
                // its maximum after that), and the product that read this buffer's last P ran before the
                // S product whose result was just read.
                uint32_t packed[COLS / 2];
#pragma unroll
                for (int c = 0; c < COLS / 2; ++c) packed[c] = pack2(s[2 * c], s[2 * c + 1]);
                if (COLS == 64) tmem_st32(tmem + lane_addr + (uint32_t)(b * BKV + part * (COLS / 2)), reinterpret_cast<const float*>(packed));
                else tmem_st16(tmem + lane_addr + (uint32_t)(b * BKV + part * (COLS / 2)), reinterpret_cast<const float*>(packed));
                FA_TOC(24 + (part & 1), row == 0);
                tmem_wait_st();
                FA_TOC(26 + (part & 1), row == 0);
            } else {
                if (j >= 2) {                              // the product that read this P buffer last is done
                    FA_TIC();
                    ok = mbar_wait(pv_done + 8 * b, (uint32_t)(((j - 2) >> 1) & 1), abort_flag, 9);
                    FA_TOC(14 + (part & 1), row == 0);
                    if (!ok) break;
                }
                // this thread's keys lie in sub-tile (part * COLS) / 64 of P: 128-byte rows, 16-byte pieces swizzled
                unsigned char* prow = smem + (size_t)off_p(D) + (size_t)b * P_TILE + (size_t)((part * COLS) / 64) * SUB + (size_t)row * 128;
                const int c0 = ((part * COLS) % 64) / 8;
#pragma unroll
                for (int c = 0; c < COLS / 8; ++c) {
                    const float* v = s + c * 8;
                    *reinterpret_cast<uint4*>(prow + (((c0 + c) ^ (row & 7)) << 4)) =
                        make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the tensor cores read P through the async proxy
            }
            tc_fence_before();
            mbar_arrive(p_full + 8 * b);
            FA_TOC(16 + (part & 1), row == 0);
        }
        // the threads of a row add their sums (slots of the parity that the last tile did not use)
        if (ok) {
            float total;
            ok = exchange(n, l, true, total);
            l = total;
        }
        if (ok) {
            ok = mbar_wait(pv_done + 8 * ((n - 1) & 1), (uint32_t)(((n - 1) >> 1) & 1), abort_flag, 10);
        }
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = p.out + ((size_t)(q_begin + start + row) * p.nq + head) * D + part * OCOLS;
#pragma unroll 1
            for (int c = 0; c < OCOLS / 32; ++c) {
                float o[32];
                tmem_ld32(tmem_o + lane_addr + (uint32_t)(part * OCOLS + c * 32), o);
                tmem_wait_ld();
                if (row < rows_valid) {
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) =
                            make_uint4(pack2(o[v * 8] * inv, o[v * 8 + 1] * inv), pack2(o[v * 8 + 2] * inv, o[v * 8 + 3] * inv),
                                       pack2(o[v * 8 + 4] * inv, o[v * 8 + 5] * inv), pack2(o[v * 8 + 6] * inv, o[v * 8 + 7] * inv));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
    }
}

// ---- two query heads a block ---------------------------------------------------------------------
//
// The same work for two query heads that share a kv head (an even group size): every K and V tile
// that comes up from L2 feeds both heads, and the two heads' softmax groups (warps 2-5 and 6-9, one
// thread per query row and no exchange between threads) work half a period apart, one in its
// exponentials while the other finds its maximum or packs P, with the tensor cores busy on the other
// head's products meanwhile.  S of each head has one accumulator (128 columns) whose first 64 columns
// then hold P; O of each head another 128 columns: all 512.  The mma thread's order is
//   S_0(0) S_1(0), then for every tile j:  PV_0(j) S_0(j+1) PV_1(j) S_1(j+1)
// where PV_h(j) waits for P_h(j); S_h(j+1) follows PV_h(j) in issue order, which is what keeps it from
// overwriting P_h(j) too early.  A softmax thread goes over its row twice in pieces of 32 columns (first
// the maximum, then the exponentials), so that it never holds more than a piece in registers.

constexpr int NH2 = 2;
constexpr int KV2 = 2;                                   // K stages, V stages
constexpr int THREADS2 = 64 + NH2 * BQ;
constexpr int NUM_BARS2 = 1 + 4 * KV2 + 3 * NH2 + 1;   // the last one is the timing build's probe
constexpr int off2_k(int d) { return NH2 * tile_bytes(d); }
constexpr int off2_v(int d) { return off2_k(d) + KV2 * tile_bytes(d); }
constexpr int off2_bars(int d) { return off2_v(d) + KV2 * tile_bytes(d); }
constexpr int off2_misc(int d) { return off2_bars(d) + 8 * NUM_BARS2 + 8; }
constexpr int smem_two(int d) { return off2_misc(d) + 16; }

template <int D>
__global__ void __launch_bounds__(THREADS2, 1)
attention_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const Params p) {
    static_assert(D == 64 || D == 128, "head sizes 64 and 128");
    constexpr int TILE = tile_bytes(D), DH = D / 64;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off2_bars(D));
    uint32_t& tmem_base_s = *reinterpret_cast<uint32_t*>(smem + off2_misc(D));
    int& abort_s = *reinterpret_cast<int*>(smem + off2_misc(D) + 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicCAS(&g_status, 0, (11 << 24) | (int)((blockIdx.x + blockIdx.y * gridDim.x) & 0xFFFFFF));
        return;
    }
    const uint32_t q_smem = smem_u32(smem), k_smem = q_smem + off2_k(D), v_smem = q_smem + off2_v(D);
    const uint32_t q_full = smem_u32(&bars[0]);
    const uint32_t k_full = q_full + 8, k_empty = k_full + 8 * KV2, v_full = k_empty + 8 * KV2, v_empty = v_full + 8 * KV2;
    const uint32_t s_full = v_empty + 8 * KV2, p_full = s_full + 8 * NH2, pv_done = p_full + 8 * NH2;   // one per head

    if (threadIdx.x == 0) {
        abort_s = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < KV2; ++s) {
            mbar_init(k_full + 8 * s, 1);
            mbar_init(k_empty + 8 * s, 1);
            mbar_init(v_full + 8 * s, 1);
            mbar_init(v_empty + 8 * s, 1);
        }
        for (int h = 0; h < NH2; ++h) {
            mbar_init(s_full + 8 * h, 1);
            mbar_init(p_full + 8 * h, BQ);                      // one arrival per softmax thread of the head
            mbar_init(pv_done + 8 * h, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;                          // S (then P) of head h: columns 128 h
    const uint32_t tmem_o = tmem + NH2 * BKV;                   // O of head h: columns 256 + 128 h
    volatile int* abort_flag = &abort_s;

    pdl_wait();
    pdl_launch_dependents();

    const int tile = p.tiles - 1 - (int)blockIdx.y;             // the last tiles, which see the most keys, go first
    const int head0 = blockIdx.x * NH2;
    const int req = p.tile_req[tile], start = p.tile_start[tile];
    const int q_begin = p.cu_seqlens[req];
    const int new_len = p.cu_seqlens[req + 1] - q_begin;
    const int rows_valid = min(BQ, new_len - start);
    const int pos0 = p.prefix_lens[req] + start;
    const int kv_end = pos0 + rows_valid;
    const int k_lo = (p.window > 0 && pos0 + 1 > p.window) ? pos0 + 1 - p.window : 0;
    const int jt0 = k_lo / BKV;
    const int n = (kv_end - 1) / BKV - jt0 + 1;

    if (warp == 0) {
        if (lane == 0) {
            const int kvh = head0 / (p.nq / p.nkv);
            const int* table = p.block_table + (size_t)req * p.bt_stride;
            mbar_expect_tx(q_full, NH2 * TILE);
            for (int h = 0; h < NH2; ++h)
                for (int dh = 0; dh < DH; ++dh)
                    tma_load_3d(q_smem + h * TILE + dh * SUB, &map_q, q_full, dh * 64, head0 + h, q_begin + start);
            bool ok = true;
            int issued_k = 0, issued_v = 0;
            for (int j = 0; j < n && ok; ++j) {
                const int s = j % KV2;
                const uint32_t par = (uint32_t)((j / KV2) & 1);
                int page[2], off[2];
                for (int h = 0; h < 2; ++h) {            // the two 64-key boxes of the tile
                    const int key = (jt0 + j) * BKV + 64 * h;
                    const bool held = key < kv_end;
                    page[h] = held ? table[key / p.page_size] : 0;
                    off[h] = held ? key % p.page_size : 0;
                }
                ok = mbar_wait(k_empty + 8 * s, par ^ 1, abort_flag, 1);
                if (!ok) break;
                mbar_expect_tx(k_full + 8 * s, TILE);
                for (int h = 0; h < 2; ++h)
                    for (int dh = 0; dh < DH; ++dh)
                        tma_load_4d(k_smem + s * TILE + dh * SUB + h * BOX, &map_kv, k_full + 8 * s, dh * 64, off[h], kvh, page[h]);
                ++issued_k;
                ok = mbar_wait(v_empty + 8 * s, par ^ 1, abort_flag, 2);
                if (!ok) break;
                mbar_expect_tx(v_full + 8 * s, TILE);
                for (int h = 0; h < 2; ++h)
                    for (int dh = 0; dh < DH; ++dh)
                        tma_load_4d(v_smem + s * TILE + dh * SUB + h * BOX, &map_kv, v_full + 8 * s, dh * 64, off[h], p.nkv + kvh, page[h]);
                ++issued_v;
            }
            if (*abort_flag) {
                for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(q_full, 0); ++i) {}
                for (int j = max(0, issued_k - KV2); j < issued_k; ++j)
                    for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(k_full + 8 * (j % KV2), (j / KV2) & 1); ++i) {}
                for (int j = max(0, issued_v - KV2); j < issued_v; ++j)
                    for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(v_full + 8 * (j % KV2), (j / KV2) & 1); ++i) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKV >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            bool ok = mbar_wait(q_full, 0, abort_flag, 3);
            auto scores = [&](int h, int i) {            // S_h(i) = Q_h K_i^T; the second head hands the K stage back
                const int s = i % KV2;
                const uint64_t dq = desc_k_major(q_smem + h * TILE), dk = desc_k_major(k_smem + s * TILE);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t inside = (uint64_t)(((kk >> 2) * SUB + (kk & 3) * 32) >> 4);
                    umma(tmem + (uint32_t)(h * BKV), dq + inside, dk + inside, idesc_s, kk != 0 ? 1u : 0u);
                }
                umma_commit(s_full + 8 * h);
                if (h == NH2 - 1) umma_commit(k_empty + 8 * s);
            };
            if (ok) ok = mbar_wait(k_full, 0, abort_flag, 4);
#ifdef LILY_FA_TIMING
            if (ok && n >= 2) {
                // how long 32 products of each kind take back to back, on tiles that are about to be overwritten:
                // slot 28 S products (Q and K from shared memory), slot 29 the same issued as 8, slot 30 PV products
                // (P from tensor memory, V from shared memory), slot 31 the empty commit-and-wait round trip
                const uint32_t probe = pv_done + 8 * NH2;
                mbar_init(probe, 1);
                asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
                ok = mbar_wait(v_full, 0, abort_flag, 6);
                tc_fence_after();
                uint32_t phase = 0;
                const uint64_t dq = desc_k_major(q_smem), dk = desc_k_major(k_smem), dv = desc_mn_major(v_smem);
                for (int kind = 0; kind < 4 && ok; ++kind) {
                    FA_TIC();
                    const int reps = kind == 0 ? 4 : (kind == 3 ? 0 : (kind == 1 ? 1 : 4));
                    for (int r = 0; r < reps; ++r)
#pragma unroll
                        for (int kk = 0; kk < D / 16; ++kk) {
                            const uint64_t inside = (uint64_t)(((kk >> 2) * SUB + (kk & 3) * 32) >> 4);
                            if (kind <= 1) umma(tmem, dq + inside, dk + inside, idesc_s, 1u);
                            else umma_ts(tmem_o, tmem + (uint32_t)(kk * 8), dv + (uint64_t)(kk * 2048 >> 4), idesc_o, 1u);
                        }
                    umma_commit(probe);
                    ok = mbar_wait(probe, phase, abort_flag, 13);
                    phase ^= 1;
                    FA_TOC(28 + (kind == 0 ? 0 : kind == 1 ? 1 : kind == 2 ? 2 : 3), true);
                }
                tc_fence_after();
            }
#endif
            if (ok) {
                tc_fence_after();
                scores(0, 0);
                scores(1, 0);
            }
            for (int j = 0; j < n && ok; ++j) {
                const int s = j % KV2;
                ok = mbar_wait(v_full + 8 * s, (uint32_t)((j / KV2) & 1), abort_flag, 6);
                for (int h = 0; h < NH2 && ok; ++h) {
                    { FA_TIC(); ok = mbar_wait(p_full + 8 * h, (uint32_t)(j & 1), abort_flag, 5); FA_TOC(4 + h, true); }
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t dv = desc_mn_major(v_smem + s * TILE);
#pragma unroll
                    for (int kk = 0; kk < BKV / 16; ++kk)
                        umma_ts(tmem_o + (uint32_t)(h * D), tmem + (uint32_t)(h * BKV + kk * 8), dv + (uint64_t)(kk * 2048 >> 4), idesc_o,
                                (j | kk) != 0 ? 1u : 0u);
                    umma_commit(pv_done + 8 * h);
                    if (h == NH2 - 1) umma_commit(v_empty + 8 * s);
                    if (j + 1 < n) {
                        if (h == 0) {
                            ok = mbar_wait(k_full + 8 * ((j + 1) % KV2), (uint32_t)(((j + 1) / KV2) & 1), abort_flag, 4);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        scores(h, j + 1);
                    }
                }
            }
        }
    } else {
        const int h = (warp - 2) >> 2, quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t my_s = tmem + lane_addr + (uint32_t)(h * BKV), my_o = tmem_o + lane_addr + (uint32_t)(h * D);
        const int pos = pos0 + row;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n && ok; ++j) {
            { FA_TIC(); ok = mbar_wait(s_full + 8 * h, (uint32_t)(j & 1), abort_flag, 7); FA_TOC(8 + h, row == 0); }
            if (!ok) break;
            FA_TIC();
            tc_fence_after();
            const int kb = (jt0 + j) * BKV;
            const bool need_mask = kb + BKV - 1 > pos0 || (p.window > 0 && kb <= pos0 + BQ - 1 - p.window);
            // first pass: the row's maximum
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                float s[32];
                tmem_ld32(my_s + (uint32_t)(c * 32), s);
                tmem_wait_ld();
                if (need_mask) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const int key = kb + c * 32 + e;
                        const bool seen = key <= pos && (p.window <= 0 || key > pos - p.window);
                        s[e] = seen ? s[e] : -INFINITY;
                    }
                }
#pragma unroll
                for (int e = 0; e < 32; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], s[e]);
            }
            const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
            FA_TOC(10 + h, row == 0);
            if (j == 0) {
                m_used = m_new;
            } else {
                const bool grow = (m_new - m_used) * p.scale_log2 > GROW_LOG2;      // also when m_used is -inf
                if (__any_sync(0xffffffffu, grow)) {
                    // O must hold every product up to tile j - 1 before its rows are rescaled
                    ok = mbar_wait(pv_done + 8 * h, (uint32_t)((j - 1) & 1), abort_flag, 8);
                    if (!ok) break;
                    tc_fence_after();
                    const float alpha = grow ? ex2((m_used - m_new) * p.scale_log2) : 1.f;
                    if (grow) m_used = m_new;
                    l *= alpha;
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        float o[32];
                        tmem_ld32(my_o + (uint32_t)(c * 32), o);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] *= alpha;
                        tmem_st32(my_o + (uint32_t)(c * 32), o);
                    }
                    tmem_wait_st();
                }
            }
            // second pass: P = exp2(s * scale - max) as bfloat16 pairs over the first 64 columns of S.  Piece c
            // lands on columns [16 c, 16 c + 16), all of them in pieces that this pass has read already.
            const float mb = (m_used == -INFINITY ? 0.f : m_used) * p.scale_log2;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                float s[32];
                tmem_ld32(my_s + (uint32_t)(c * 32), s);
                tmem_wait_ld();
                if (need_mask) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const int key = kb + c * 32 + e;
                        const bool seen = key <= pos && (p.window <= 0 || key > pos - p.window);
                        s[e] = seen ? s[e] : -INFINITY;
                    }
                }
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    s[e] = ex2(fmaf(s[e], p.scale_log2, -mb));
                    sum4[e & 3] += s[e];
                }
                uint32_t packed[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) packed[e] = pack2(s[2 * e], s[2 * e + 1]);
                tmem_st16(my_s + (uint32_t)(c * 16), reinterpret_cast<const float*>(packed));
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            FA_TOC(12 + h, row == 0);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(p_full + 8 * h);
            FA_TOC(16 + h, row == 0);
        }
        if (ok) ok = mbar_wait(pv_done + 8 * h, (uint32_t)((n - 1) & 1), abort_flag, 10);
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = p.out + ((size_t)(q_begin + start + row) * p.nq + head0 + h) * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                float o[32];
                tmem_ld32(my_o + (uint32_t)(c * 32), o);
                tmem_wait_ld();
                if (row < rows_valid) {
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) =
                            make_uint4(pack2(o[v * 8] * inv, o[v * 8 + 1] * inv), pack2(o[v * 8 + 2] * inv, o[v * 8 + 3] * inv),
                                       pack2(o[v * 8 + 4] * inv, o[v * 8 + 5] * inv), pack2(o[v * 8 + 6] * inv, o[v * 8 + 7] * inv));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
    }
}

// ---- host side --------------------------------------------------------------------------------

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)ptr;
    });
    return fn;
}

// Launches the kernel of head size D with one head or two heads a block (the shared memory limits are raised once).
template <int D>
static int launch(bool two, int nq, int tiles, cudaStream_t stream, const CUtensorMap& map_q, const CUtensorMap& map_kv, const Params& p) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_one(D));
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attention_prefill_tc2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_two(D));
        if (e != cudaSuccess) {
            set_error("attention_prefill_tc: cannot get %d bytes of shared memory: %s", smem_one(D), cudaGetErrorString(e));
            return 2;
        }
        configured = true;
    }
    if (two)
        launch_pdl(attention_prefill_tc2_kernel<D>, dim3(nq / 2, tiles), dim3(THREADS2), (size_t)smem_two(D), stream, map_q, map_kv, p);
    else
        launch_pdl(attention_prefill_tc_kernel<D>, dim3(nq, tiles), dim3(THREADS), (size_t)smem_one(D), stream, map_q, map_kv, p);
    return 0;
}

}  // namespace fa
}  // namespace lily

using namespace lily;

#ifdef LILY_FA_TIMING
// Copies the 32 phase counters of block (0, 0) to `out` and clears them.  Slots: 0, 1 the loader waiting
// for a K, V stage; 2, 3, 4 the mma thread waiting for K, V, P; for the softmax thread of row 0 with key half
// h: 8 + h waiting for S, then measured from the start of the tile's work: 10 + h S read, 12 + h sums done,
// 16 + h arrived on the P barrier; 14 + h the wait for the P buffer inside that.
LILY_API int lily_attention_tc_timing(unsigned long long* out) {
    unsigned long long zero[32] = {};
    if (cudaMemcpyFromSymbol(out, fa::g_timing, sizeof(zero)) != cudaSuccess) return 1;
    return cudaMemcpyToSymbol(fa::g_timing, zero, sizeof(zero)) == cudaSuccess ? 0 : 1;
}
#endif

LILY_API int lily_attention_prefill_tc_rows() { return fa::BQ; }

// Whether the tcgen05 kernel takes this head size and page size (bfloat16 only).
LILY_API int lily_attention_prefill_tc_takes(int d, int page_size) { return (d == 64 || d == 128) && page_size > 0 && page_size % 64 == 0; }

// 0 while no wait has given up since the last call; else (code << 24 | block).  Codes: 1, 2 the
// loader waiting for a free K or V stage; 3, 4, 6 the mma thread waiting for Q, K or V; 5 the mma
// thread waiting for P; 7 the softmax waiting for scores; 8, 9, 10 the softmax waiting for a product
// into O.  Synchronises the device.  Reading clears it.
LILY_API int lily_attention_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, fa::g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(fa::g_status, &zero, sizeof(int));
    return v;
}

// The arguments of lily_attention_prefill_mma with tiles of 128 rows, plus the number of pages of
// the layer (`kv` is [num_pages, 2, nkv, page_size, d]) and of new tokens (`q` is [tokens, nq, d]);
// heads_per_block 1 or 2 names the kernel, 0 leaves the choice to the launcher.
LILY_API int lily_attention_prefill_tc(const void* q, const void* kv, void* out, const int* block_table, int bt_stride,
                                       const int* cu_seqlens, const int* prefix_lens, const int* tile_req,
                                       const int* tile_start, int tiles, int nq, int nkv, int d, int page_size, int window,
                                       float scale, int tokens, int num_pages, int heads_per_block, cudaStream_t stream) {
    if (tiles == 0) return 0;
    LILY_REQUIRE(lily_attention_prefill_tc_takes(d, page_size), "attention_prefill_tc: head size %d, page size %d (takes 64 or 128, and multiples of 64)",
                 d, page_size);
    LILY_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_prefill_tc: %d query heads over %d kv heads", nq, nkv);
    LILY_REQUIRE(tiles <= 65535 && tokens > 0 && num_pages > 0, "attention_prefill_tc: tiles=%d tokens=%d pages=%d", tiles, tokens, num_pages);
    LILY_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)kv % 16 == 0) && ((uintptr_t)out % 16 == 0), "attention_prefill_tc: operands must be 16-byte aligned");
    fa::EncodeTiled enc = fa::encoder();
    LILY_REQUIRE(enc != nullptr, "attention_prefill_tc: the driver does not offer cuTensorMapEncodeTiled");
    CUtensorMap map_q, map_kv;
    {
        const cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)nq, (cuuint64_t)tokens};
        const cuuint64_t strides[2] = {(cuuint64_t)d * 2, (cuuint64_t)nq * d * 2};
        const cuuint32_t box[3] = {64, 1, (cuuint32_t)fa::BQ};
        const cuuint32_t elem[3] = {1, 1, 1};
        const CUresult rc = enc(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        LILY_REQUIRE(rc == CUDA_SUCCESS, "attention_prefill_tc: cuTensorMapEncodeTiled (q) failed with %d", (int)rc);
    }
    {
        const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)page_size, (cuuint64_t)2 * nkv, (cuuint64_t)num_pages};
        const cuuint64_t strides[3] = {(cuuint64_t)d * 2, (cuuint64_t)page_size * d * 2, (cuuint64_t)2 * nkv * page_size * d * 2};
        const cuuint32_t box[4] = {64, 64, 1, 1};
        const cuuint32_t elem[4] = {1, 1, 1, 1};
        const CUresult rc = enc(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(kv), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        LILY_REQUIRE(rc == CUDA_SUCCESS, "attention_prefill_tc: cuTensorMapEncodeTiled (cache) failed with %d", (int)rc);
    }
    fa::Params p{};
    p.block_table = block_table; p.cu_seqlens = cu_seqlens; p.prefix_lens = prefix_lens; p.tile_req = tile_req;
    p.tile_start = tile_start; p.out = (__nv_bfloat16*)out; p.bt_stride = bt_stride; p.tiles = tiles; p.nq = nq; p.nkv = nkv;
    p.page_size = page_size; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
    // two heads of a kv head a block when the group size is even and, unless the caller says which, when
    // that still leaves a block for every SM (short prompts fill the device better with a head a block)
    const int sms = sm_count();
    const bool even = (nq / nkv) % 2 == 0;
    LILY_REQUIRE(heads_per_block >= 0 && heads_per_block <= 2 && (heads_per_block != 2 || even),
                 "attention_prefill_tc: %d heads a block with %d query heads per kv head", heads_per_block, nq / nkv);
    const bool two = heads_per_block == 2 || (heads_per_block == 0 && even && (long)tiles * (nq / 2) >= sms);
    const int rc = d == 64 ? fa::launch<64>(two, nq, tiles, stream, map_q, map_kv, p) : fa::launch<128>(two, nq, tiles, stream, map_q, map_kv, p);
    if (rc) return rc;
    LILY_CHECK_LAUNCH("attention_prefill_tc");
    return 0;
}
