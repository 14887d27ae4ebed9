// C[M, N] = A[M, K] @ W[N, K]^T in true float32 on the CUDA cores (FFMA only: no
// tensor cores, no TF32).  It is the matrix product of the 32-bit path, where the
// reference calls a library product with TF32 disabled (engine/engine.py:113-114,
// :341-350).  Every output element accumulates k = 0, 1, 2, ... in one accumulator, so a
// row's result does not depend on how many other rows the call has.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256) gemm_f32_kernel(float* __restrict__ C, const float* __restrict__ A,
                                                       const float* __restrict__ W, int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements per operand, 256 threads: 4 each; consecutive threads walk k.
        for (int e = tid; e < BM * BK; e += 256) {
            const int r = e / BK, c = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * K + gk] : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * N + gn] = acc[i][j];
        }
    }
}
}  // namespace

THN_API int thn_gemm_f32(float* C, const float* A, const float* W, int M, int N, int K, cudaStream_t stream) {
    THN_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return THN_OK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    THN_UNSUPPORTED_IF(grid.y > 65535, "gemm_f32: %d rows exceed the grid limit", M);
    thn_launch(gemm_f32_kernel, grid, 256, 0, stream, C, A, W, M, N, K);
    return thn_launch_status("gemm_f32");
}
