// Weight-streaming matrix product for decode batches:  C[M,N] = A[M,K] * W[N,K]^T  with M <= 16,
// bfloat16 operands, 32-bit accumulation on the tensor cores, bfloat16 or 32-bit output.
//
// The product is turned round: 16 weight rows are the M side of an m16n8k16 MMA and 8 tokens its N
// side, so the weight matrix streams through the tensor cores once while the few activation rows
// stay in L1/L2.  A CTA owns 16 weight rows; its 8 warps take the 64-wide blocks of K in turn
// (warp w: blocks w, w+8, ...), so the CTA reads each row as contiguous 1 KiB stretches, and the
// warps' partial sums are added through shared memory in a fixed order.  Fragments are loaded
// straight from global memory with 16-byte loads: within a 64-block, lane t (= lane & 3) of a row
// loads elements [16t, 16t+16), and each k-step of the MMA takes four of them on both operands,
// which is a permutation of the contraction index and leaves the product unchanged.
// The summation order of an output element does not depend on M.
//
// Reference counterpart: gemv_fp16_kernel / gemv_bf16_kernel for M == 1 (src/compute/gemm.cu:
// 496-649, CUDA cores, one warp per output row) and cuBLASLt for 2 <= M <= 64 (:148-156).
#include "common.cuh"

constexpr int GS_WARPS = 8;
constexpr int GS_KB = 64;   // elements of K per block

__device__ __forceinline__ void gs_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 gs_ld_stream(const __nv_bfloat16* p) {
    // weights are read once: keep them from displacing the activations in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int NT, typename TO>
__global__ void __launch_bounds__(GS_WARPS * 32) gemm_stream_kernel(TO* __restrict__ C, int64_t ldc,
                                                                    const __nv_bfloat16* __restrict__ A, int64_t lda,
                                                                    const __nv_bfloat16* __restrict__ W, int64_t ldw,
                                                                    int M, int N, int K) {
    __shared__ float red[GS_WARPS][NT * 4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const __nv_bfloat16* w0 = W + (int64_t)min(n0 + g, N - 1) * ldw + 16 * t;
    const __nv_bfloat16* w1 = W + (int64_t)min(n0 + g + 8, N - 1) * ldw + 16 * t;
    const __nv_bfloat16* ap[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) ap[nt] = A + (int64_t)min(8 * nt + g, M - 1) * lda + 16 * t;

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    const int nkb = (K + GS_KB - 1) / GS_KB;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 2
    for (int kb = warp; kb < nkb; kb += GS_WARPS) {
        const int k = kb * GS_KB + 16 * t;             // this lane's first element of the block
        const bool in0 = k + 8 <= K, in1 = k + 16 <= K;   // K is a multiple of 8: a chunk is all in or all out
        const int64_t o = (int64_t)kb * GS_KB;
        const uint4 wa0 = in0 ? gs_ld_stream(w0 + o) : zero;
        const uint4 wa1 = in1 ? gs_ld_stream(w0 + o + 8) : zero;
        const uint4 wb0 = in0 ? gs_ld_stream(w1 + o) : zero;
        const uint4 wb1 = in1 ? gs_ld_stream(w1 + o + 8) : zero;
        uint4 x0[NT], x1[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            x0[nt] = in0 ? *reinterpret_cast<const uint4*>(ap[nt] + o) : zero;
            x1[nt] = in1 ? *reinterpret_cast<const uint4*>(ap[nt] + o + 8) : zero;
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            gs_mma(acc[nt], wa0.x, wb0.x, wa0.y, wb0.y, x0[nt].x, x0[nt].y);
            gs_mma(acc[nt], wa0.z, wb0.z, wa0.w, wb0.w, x0[nt].z, x0[nt].w);
            gs_mma(acc[nt], wa1.x, wb1.x, wa1.y, wb1.y, x1[nt].x, x1[nt].y);
            gs_mma(acc[nt], wa1.z, wb1.z, wa1.w, wb1.w, x1[nt].z, x1[nt].w);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[warp][nt * 4 + c][lane] = acc[nt][c];
    __syncthreads();
    // 16 rows x 8*NT tokens = NT*128 sums; thread i takes register slot i / 32 of lane i % 32.
    for (int i = threadIdx.x; i < NT * 128; i += GS_WARPS * 32) {
        const int r = i >> 5, l = i & 31;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < GS_WARPS; ++w) s += red[w][r][l];
        const int nt = r >> 2, c = r & 3;
        const int row = n0 + (l >> 2) + ((c & 2) ? 8 : 0);
        const int tok = 8 * nt + 2 * (l & 3) + (c & 1);
        if (row < N && tok < M) C[(int64_t)tok * ldc + row] = from_float<TO>(s);
    }
}

template <typename TO>
static int launch_stream(TO* C, int64_t ldc, const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* W, int64_t ldw,
                         int M, int N, int K, cudaStream_t s) {
    const int grid = (N + 15) / 16;
    if (M <= 8)
        gemm_stream_kernel<1, TO><<<grid, GS_WARPS * 32, 0, s>>>(C, ldc, A, lda, W, ldw, M, N, K);
    else
        gemm_stream_kernel<2, TO><<<grid, GS_WARPS * 32, 0, s>>>(C, ldc, A, lda, W, ldw, M, N, K);
    IMP_RETURN_LAUNCH();
}

// Returns IMP_ERR_UNSUPPORTED (without an error text) when the operands do not allow 16-byte loads;
// the caller then uses the scalar kernel.
IMP_API int imp_gemm_bf16_stream(void* C, int64_t ldc, int out_dtype, const void* A, int64_t lda, const void* W,
                                 int64_t ldw, int M, int N, int K, void* stream) {
    if (M == 0 || N == 0) return 0;
    IMP_CHECK_ARG(C && A && W && M > 0 && N > 0 && K > 0, "imp_gemm_bf16_stream: bad argument");
    IMP_CHECK_ARG(M <= 16, "imp_gemm_bf16_stream: M %d exceeds 16", M);
    IMP_CHECK_ARG(ldc >= N && lda >= K && ldw >= K, "imp_gemm_bf16_stream: leading dimension too small");
    if (K % 8 || lda % 8 || ldw % 8 || (uintptr_t)A % 16 || (uintptr_t)W % 16) return IMP_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IMP_F32)
        return launch_stream<float>((float*)C, ldc, (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, ldw, M, N, K, s);
    return launch_stream<__nv_bfloat16>((__nv_bfloat16*)C, ldc, (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W,
                                        ldw, M, N, K, s);
}
