// True 32-bit matrix product  C[M,N] = A[M,K] * W[N,K]^T  (+ nothing else).
//
// The float32 path's only matrix kernel: plain FFMA, no tensor cores, no
// reduced-precision mode.  Every output element is the fused-multiply-add
// chain over k = 0..K-1 in ascending order, whatever M is and wherever the row
// sits in the batch, so a token's result is bit-identical under every split of
// the work.  The reference's fp32 route is cublasSgemm (src/compute/gemm.cu:
// 341-358) and a warp-per-row GEMV (src/compute/gemm.cu:452-493); W is stored
// [N,K] as there (src/compute/gemm.h:18-19).
#include "common.cuh"

constexpr int GF_BM = 64, GF_BN = 64, GF_BK = 16;

__global__ void __launch_bounds__(256) gemm_f32_kernel(float* __restrict__ C, int64_t ldc,
                                                       const float* __restrict__ A, int64_t lda,
                                                       const float* __restrict__ W, int64_t ldw,
                                                       int M, int N, int K) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float As[GF_BK][GF_BM + 4];
    __shared__ float Ws[GF_BK][GF_BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GF_BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread.
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / GF_BK, kk = idx % GF_BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? A[(int64_t)gm * lda + gk] : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? W[(int64_t)gn * ldw + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GF_BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + tm + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tn + j;
            if (gn < N) C[(int64_t)gm * ldc + gn] = acc[i][j];
        }
    }
}

IMP_API int imp_gemm_f32(float* C, int64_t ldc, const float* A, int64_t lda, const float* W, int64_t ldw, int M,
                         int N, int K, void* stream) {
    if (M == 0 || N == 0) return 0;
    IMP_CHECK_ARG(C && A && W && M > 0 && N > 0 && K > 0, "imp_gemm_f32: bad argument");
    IMP_CHECK_ARG(ldc >= N && lda >= K && ldw >= K, "imp_gemm_f32: leading dimension too small");
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    IMP_CHECK_ARG(grid.y <= 65535, "imp_gemm_f32: M %d too large for one launch", M);
    gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(C, ldc, A, lda, W, ldw, M, N, K);
    IMP_RETURN_LAUNCH();
}
