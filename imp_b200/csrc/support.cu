// Kernels beside the forward pass: random weights on the device, stage statistics for the
// debugging switch, and a plain bfloat16 matrix product for shapes no fast kernel takes.
#include "common.cuh"

#include <math.h>

// ---------------------------------------------------------------------------- random weights
// Element i of a tensor is a function of (tensor seed, i): splitmix64 of the pair gives two 24-bit
// uniforms, Box-Muller gives one normal value.  The host writer (host/weights.cpp) uses the same
// arithmetic.  mode: 0 = std * n, 1 = 1 + norm_std * n, 2 = zero, 3 = i mod 2^15 (integer tables).
__device__ __forceinline__ float random_normal_at(uint64_t tseed, uint64_t i) {
    uint64_t z = tseed + (i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    const float u1 = (float)((z >> 40) + 1) * (1.0f / 16777216.0f);
    const float u2 = (float)(z & 0xFFFFFFull) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

__global__ void random_fill_kernel(void* out, int dtype, int64_t n, uint64_t tseed, int mode, float std, float norm_std,
                                   int round_bf16) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        if (dtype == 2) {
            reinterpret_cast<int*>(out)[i] = mode == 3 ? (int)(i % 32768) : 0;
            continue;
        }
        float v = mode == 2 ? 0.f : mode == 3 ? (float)(i % 32768) : random_normal_at(tseed, (uint64_t)i);
        if (mode == 0) v *= std;
        if (mode == 1) v = 1.0f + norm_std * v;
        if (round_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
        if (dtype == IMP_F32) reinterpret_cast<float*>(out)[i] = v;
        else reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    }
}

IMP_API int imp_random_fill(void* out, int dtype, int64_t n, uint64_t tensor_seed, int mode, float std, float norm_std,
                            int round_bf16, void* stream) {
    IMP_CHECK_ARG(out && n >= 0 && dtype >= 0 && dtype <= 2, "imp_random_fill: bad arguments");
    if (n == 0) return 0;
    const int threads = 256;
    const int64_t want = (n + threads - 1) / threads;
    const int grid = (int)(want < 65535 ? want : 65535);
    random_fill_kernel<<<grid, threads, 0, (cudaStream_t)stream>>>(out, dtype, n, tensor_seed, mode, std, norm_std, round_bf16);
    IMP_RETURN_LAUNCH();
}

// -------------------------------------------------------------------------- stage statistics
// out5 = {min, max, sum, sum of squares, count of NaN/Inf}; finite values only in the first four.
// One block: this runs only under the debugging switch.
__global__ void __launch_bounds__(1024) tensor_stats_kernel(const void* x, int dtype, int64_t n, float* out5) {
    __shared__ float scratch[33];
    float mn = INFINITY, mx = -INFINITY, sum = 0.f, sq = 0.f, bad = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = load_as_float(x, dtype, i);
        if (isfinite(v)) {
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
            sum += v;
            sq += v * v;
        } else {
            bad += 1.f;
        }
    }
    mn = -block_max(-mn, scratch);
    mx = block_max(mx, scratch);
    sum = block_sum(sum, scratch);
    sq = block_sum(sq, scratch);
    bad = block_sum(bad, scratch);
    if (threadIdx.x == 0) {
        out5[0] = mn;
        out5[1] = mx;
        out5[2] = sum;
        out5[3] = sq;
        out5[4] = bad;
    }
}

IMP_API int imp_tensor_stats(const void* x, int dtype, int64_t n, float* out5, void* stream) {
    IMP_CHECK_ARG(x && out5 && n > 0 && (dtype == IMP_F32 || dtype == IMP_BF16), "imp_tensor_stats: bad arguments");
    tensor_stats_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(x, dtype, n, out5);
    IMP_RETURN_LAUNCH();
}

// --------------------------------------------------------------------- plain bfloat16 product
// C[M,N] = A[M,K] W[N,K]^T with 32-bit accumulation, k ascending, for any sizes, strides and
// alignments: what runs when the tensor-core kernels decline a shape (a contraction that is no
// multiple of 8, an unaligned base).  One thread per output element, 32 x 32 tiles in shared memory.
template <typename TO>
__global__ void __launch_bounds__(1024) gemm_bf16_plain_kernel(TO* __restrict__ C, int64_t ldc,
                                                               const __nv_bfloat16* __restrict__ A, int64_t lda,
                                                               const __nv_bfloat16* __restrict__ W, int64_t ldw, int M,
                                                               int N, int K) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float a_s[32][33], w_s[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int m = blockIdx.y * 32 + ty, n = blockIdx.x * 32 + tx;
    float acc = 0.f;
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int ka = k0 + tx;
        a_s[ty][tx] = (m < M && ka < K) ? __bfloat162float(A[(int64_t)m * lda + ka]) : 0.f;
        const int wn = blockIdx.x * 32 + ty;
        w_s[ty][tx] = (wn < N && ka < K) ? __bfloat162float(W[(int64_t)wn * ldw + ka]) : 0.f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 32; ++k) acc = fmaf(a_s[ty][k], w_s[tx][k], acc);
        __syncthreads();
    }
    if (m < M && n < N) C[(int64_t)m * ldc + n] = from_float<TO>(acc);
}

IMP_API int imp_gemm_bf16_plain(void* C, int64_t ldc, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw,
                                int M, int N, int K, void* stream) {
    IMP_CHECK_ARG(C && A && W && M > 0 && N > 0 && K > 0, "imp_gemm_bf16_plain: bad arguments");
    IMP_CHECK_ARG(out_dtype == IMP_F32 || out_dtype == IMP_BF16, "imp_gemm_bf16_plain: output must be float32 or bfloat16");
    const dim3 grid((N + 31) / 32, (M + 31) / 32), block(32, 32);
    cudaError_t e;
    if (out_dtype == IMP_F32)
        e = imp_launch(gemm_bf16_plain_kernel<float>, grid, block, 0, (cudaStream_t)stream, (float*)C, ldc,
                       (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, ldw, M, N, K);
    else
        e = imp_launch(gemm_bf16_plain_kernel<__nv_bfloat16>, grid, block, 0, (cudaStream_t)stream, (__nv_bfloat16*)C, ldc,
                       (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, ldw, M, N, K);
    if (e != cudaSuccess) {
        imp_set_error("imp_gemm_bf16_plain: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}
