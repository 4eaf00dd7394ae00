// True float32 matrix product for the 32-bit path: C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]).
//
// FFMA only (no tensor cores, no TF32).  Each output element is summed over k in a fixed order
// whatever M and N are (runs of 256 products, each run summed left to right, the runs' sums added
// left to right), so a row's result does not depend on what else is in the batch; summing in runs
// keeps the rounding error of a sum over 12,288 products near that of one over a few hundred.
// Takes the place of F.linear in float32 (lily/layers/quantization/base.py:69-72).
#include "common.cuh"

namespace lily {

constexpr int BM = 64, BN = 64, BK = 16;
constexpr int RUN = 256;               // products per run (a multiple of BK)

__global__ void __launch_bounds__(256)
gemm_fp32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                 float* __restrict__ C, int M, int N, int K, int lda, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = threadIdx.x >> 2, lc = (threadIdx.x & 3) * 4;   // loader: row 0..63, k offset 0,4,8,12
    float acc[4][4] = {}, total[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        if (k0 != 0 && k0 % RUN == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    total[i][j] += acc[i][j];
                    acc[i][j] = 0.f;
                }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lc + j;
            const int am = m0 + lr, wn = n0 + lr;
            As[lc + j][lr] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
            Ws[lc + j][lr] = (wn < N && k < K) ? W[(size_t)wn * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = (total[i][j] + acc[i][j]) + (bias ? bias[n] : 0.f);
        }
    }
}

}  // namespace lily

using namespace lily;

LILY_API int lily_gemm_fp32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                            int lda, int ldc, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    LILY_REQUIRE(K > 0 && lda >= K && ldc >= N, "gemm_fp32: bad sizes M=%d N=%d K=%d lda=%d ldc=%d", M, N, K, lda, ldc);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    LILY_REQUIRE(grid.y <= 65535, "gemm_fp32: M=%d is too large for one launch", M);
    gemm_fp32_kernel<<<grid, 256, 0, stream>>>(A, W, bias, C, M, N, K, lda, ldc);
    LILY_CHECK_LAUNCH("gemm_fp32");
    return 0;
}
