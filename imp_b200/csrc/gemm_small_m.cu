// Weight-streaming matrix product for few rows (decode):  C[M,N] = A[M,K] * W[N,K]^T,
// bfloat16 operands, 32-bit accumulation, bfloat16 or 32-bit output.
//
// One warp per weight row: the row is read once with 16-byte loads and used
// for up to 8 activation rows held in registers' worth of L1-resident data, so
// the kernel is bound by the weight stream.  The reference's counterpart is
// gemv_fp16_kernel / gemv_bf16_kernel (src/compute/gemm.cu:496-649: one warp
// per output row, 128-bit loads, products in half2, sum in fp32), used only for
// M == 1; it hands 2 <= M <= 64 to cuBLASLt (src/compute/gemm.cu:148-156).
// Here products are 32-bit as well, and the sum order of an output element
// (lane-strided partial sums, then a shuffle tree) does not depend on M.
#include "common.cuh"

template <int MT, typename TO>
__global__ void __launch_bounds__(256) gemm_small_m_vec_kernel(TO* __restrict__ C, int64_t ldc,
                                                               const __nv_bfloat16* __restrict__ A, int64_t lda,
                                                               const __nv_bfloat16* __restrict__ W, int64_t ldw,
                                                               int M, int N, int K) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int m0 = blockIdx.y * MT;
    if (n >= N) return;
    const uint4* wrow = reinterpret_cast<const uint4*>(W + (int64_t)n * ldw);
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    const int chunks = K >> 3;
    for (int c = lane; c < chunks; c += 32) {
        const uint4 wv = __ldg(wrow + c);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
        float wf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(w2[i]);
            wf[2 * i] = f.x;
            wf[2 * i + 1] = f.y;
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m0 + m < M) {
                const uint4 av = *(reinterpret_cast<const uint4*>(A + (int64_t)(m0 + m) * lda) + c);
                const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(a2[i]);
                    acc[m] = fmaf(wf[2 * i], f.x, acc[m]);
                    acc[m] = fmaf(wf[2 * i + 1], f.y, acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == 0 && m0 + m < M) C[(int64_t)(m0 + m) * ldc + n] = from_float<TO>(v);
    }
}

// Any K, any alignment: 2-byte loads.
template <typename TO>
__global__ void gemm_small_m_scalar_kernel(TO* __restrict__ C, int64_t ldc, const __nv_bfloat16* __restrict__ A,
                                           int64_t lda, const __nv_bfloat16* __restrict__ W, int64_t ldw, int M,
                                           int N, int K) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int m = blockIdx.y;
    if (n >= N) return;
    const __nv_bfloat16* wrow = W + (int64_t)n * ldw;
    const __nv_bfloat16* arow = A + (int64_t)m * lda;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(to_float(wrow[k]), to_float(arow[k]), acc);
    acc = warp_sum(acc);
    if (lane == 0) C[(int64_t)m * ldc + n] = from_float<TO>(acc);
}

template <typename TO>
static int launch_small_m(TO* C, int64_t ldc, const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* W,
                          int64_t ldw, int M, int N, int K, cudaStream_t s) {
    const int warps = 8;
    const int gx = (N + warps - 1) / warps;
    const bool vec = (K % 8 == 0) && (lda % 8 == 0) && (ldw % 8 == 0) &&
                     (reinterpret_cast<uintptr_t>(A) % 16 == 0) && (reinterpret_cast<uintptr_t>(W) % 16 == 0);
    if (!vec) {
        IMP_CHECK_ARG(M <= 65535, "imp_gemm_bf16_small_m: M %d too large", M);
        gemm_small_m_scalar_kernel<TO><<<dim3(gx, M), warps * 32, 0, s>>>(C, ldc, A, lda, W, ldw, M, N, K);
        IMP_RETURN_LAUNCH();
    }
    if (M == 1)
        gemm_small_m_vec_kernel<1, TO><<<dim3(gx, 1), warps * 32, 0, s>>>(C, ldc, A, lda, W, ldw, M, N, K);
    else if (M == 2)
        gemm_small_m_vec_kernel<2, TO><<<dim3(gx, 1), warps * 32, 0, s>>>(C, ldc, A, lda, W, ldw, M, N, K);
    else if (M <= 4)
        gemm_small_m_vec_kernel<4, TO><<<dim3(gx, 1), warps * 32, 0, s>>>(C, ldc, A, lda, W, ldw, M, N, K);
    else
        gemm_small_m_vec_kernel<8, TO><<<dim3(gx, (M + 7) / 8), warps * 32, 0, s>>>(C, ldc, A, lda, W, ldw, M, N, K);
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_gemm_bf16_small_m(void* C, int64_t ldc, int out_dtype, const void* A, int64_t lda, const void* W,
                                  int64_t ldw, int M, int N, int K, void* stream) {
    if (M == 0 || N == 0) return 0;
    IMP_CHECK_ARG(C && A && W && M > 0 && N > 0 && K > 0, "imp_gemm_bf16_small_m: bad argument");
    IMP_CHECK_ARG(ldc >= N && lda >= K && ldw >= K, "imp_gemm_bf16_small_m: leading dimension too small");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IMP_F32)
        return launch_small_m<float>((float*)C, ldc, (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, ldw, M,
                                     N, K, s);
    return launch_small_m<__nv_bfloat16>((__nv_bfloat16*)C, ldc, (const __nv_bfloat16*)A, lda,
                                         (const __nv_bfloat16*)W, ldw, M, N, K, s);
}
