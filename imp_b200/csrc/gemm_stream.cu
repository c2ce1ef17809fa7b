// Weight-streaming matrix product for decode batches:  C[M,N] = A[M,K] * W[N,K]^T  with M <= 16,
// bfloat16 operands, 32-bit accumulation on the tensor cores, bfloat16 or 32-bit output.
//
// The product is turned round: 16 weight rows are the M side of an m16n8k16 MMA and 8 tokens its N
// side, so the weight matrix streams through the tensor cores once while the few activation rows
// stay in L2.  A tile is 16 weight rows; it is walked along K in stages of 256 elements, and a
// stage (8 KiB of weights and the same slice of the activation rows) arrives in shared memory
// through a 6-deep cp.async ring.  A CTA takes tiles blockIdx.x, blockIdx.x + gridDim.x, ... and
// the ring runs on across tile borders, so it keeps about 40 KiB of weight reads in flight from
// its first instruction to its last and the kernel runs at the rate of the memory, not of its
// round trips.  Each of the 4 warps takes one 64-wide block of every stage; within a block, lane t (= lane & 3) of a row takes elements [16t, 16t+16) for both
// operands, which is a permutation of the contraction index and leaves the product unchanged.
// The warps' partial sums are added through shared memory in a fixed order; the summation order
// of an output element does not depend on M.  The first stages are requested before the kernel
// waits for its predecessor in the stream (the weights do not depend on it).
//
// Reference counterpart: gemv_fp16_kernel / gemv_bf16_kernel for M == 1 (src/compute/gemm.cu:
// 496-649, CUDA cores, one warp per output row) and cuBLASLt for 2 <= M <= 64 (:148-156).
#include "common.cuh"

#include <cstdlib>

IMP_TL_DEFINE(gemm_stream)

constexpr int GS_WARPS = 4;
constexpr int GS_KB = 64;                          // elements of K per warp and stage
constexpr int GS_STAGE_K = GS_KB * GS_WARPS;       // 256 elements of K per stage
constexpr int GS_RED_BYTES = 4 * 8 * 32 * 4;      // reduction buffer per row group: 4 warps x (up to 8 slots) x 32 lanes
constexpr int GS_ROW_BYTES = GS_STAGE_K * 2 + 16;  // 528: rows 16 bytes apart modulo 128 -> conflict-free 16-byte reads
// A CTA owns RG groups of 16 weight rows (RG = 1 or 2; 4 warps per group); the groups share the staged
// activation rows, so with RG = 2 the activations cross from the L2 half as often per weight byte.
constexpr int gs_w_bytes(int rg) { return 16 * rg * GS_ROW_BYTES; }   // weight part of a stage; 8*NT activation rows follow
constexpr int gs_stage_bytes(int nt, int rg) { return (16 * rg + 8 * nt) * GS_ROW_BYTES; }
constexpr int gs_smem_bytes(int nt, int stages, int rg) { return stages * gs_stage_bytes(nt, rg) + rg * GS_RED_BYTES; }

__device__ __forceinline__ void gs_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16-byte asynchronous copy global -> shared; src_bytes == 0 fills the destination with zeros.
__device__ __forceinline__ void gs_cp_async(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void gs_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void gs_wait_group() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// SWIGLU: the 16 rows of a CTA are 8 gate rows followed by their 8 up rows (the caller interleaves
// the two matrices in blocks of 8 rows), so accumulator slots c and c+2 of a lane hold gate and up
// of the same output column and token; the epilogue writes silu(gate) * up into C[M, N/2].
template <int NT, typename TO, bool SWIGLU, int STAGES, int RG>
__global__ void __launch_bounds__(GS_WARPS * 32 * RG) gemm_stream_kernel(TO* __restrict__ C, int64_t ldc,
                                                                    const __nv_bfloat16* __restrict__ A, int64_t lda,
                                                                    const __nv_bfloat16* __restrict__ W, int64_t ldw,
                                                                    int M, int N, int K) {
    IMP_TL_BEGIN(5)
    extern __shared__ __align__(128) unsigned char gs_smem[];
    constexpr int STAGE_BYTES = gs_stage_bytes(NT, RG);
    constexpr int THREADS = GS_WARPS * 32 * RG, ROWS = 16 * RG, W_BYTES = gs_w_bytes(RG);
    const int tid = threadIdx.x, lane = tid & 31;
    const int rg = (tid >> 5) / GS_WARPS, warp = (tid >> 5) % GS_WARPS;   // row group, and K block within a stage
    const int g = lane >> 2, t = lane & 3;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(gs_smem);
    float(*red)[NT * 4][32] = reinterpret_cast<float(*)[NT * 4][32]>(gs_smem + STAGES * STAGE_BYTES) + rg * GS_WARPS;
    const int n_stages = (K + GS_STAGE_K - 1) / GS_STAGE_K;
    const int n_tiles = (N + ROWS - 1) / ROWS;
    const int my_tiles = (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total = my_tiles * n_stages;       // steps of this CTA: (tile, stage) pairs in order

    // Producer side: step q_issue is (tile i_tile, stage i_stage).
    int q_issue = 0, i_tile = blockIdx.x, i_stage = 0;
    // Weight copies of a step: ROWS rows x 32 chunks of 16 bytes, 4 per thread; chunk c ->
    // row c / 32, column chunk c % 32, so a warp copies one row's 512 contiguous bytes.
    auto issue_w = [&]() {
        if (q_issue < total) {
            const uint32_t sbase = smem_base + (q_issue % STAGES) * STAGE_BYTES;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = tid + i * THREADS;
                const int row = c >> 5, col = c & 31;
                const int k = i_stage * GS_STAGE_K + col * 8;
                const __nv_bfloat16* src = W + (int64_t)min(i_tile * ROWS + row, N - 1) * ldw + min(k, K - 8);
                gs_cp_async(sbase + row * GS_ROW_BYTES + col * 16, src, k + 8 <= K ? 16 : 0);
            }
        }
    };
    // Activation copies: 8*NT rows x 32 chunks, 2*NT per thread; rows past M and columns past K are zeros.
    auto issue_a = [&]() {
        if (q_issue < total) {
            const uint32_t sbase = smem_base + (q_issue % STAGES) * STAGE_BYTES + W_BYTES;
#pragma unroll
            for (int i = 0; i < 2 * NT / RG; ++i) {
                const int c = tid + i * THREADS;
                const int row = c >> 5, col = c & 31;
                const int k = i_stage * GS_STAGE_K + col * 8;
                const __nv_bfloat16* src = A + (int64_t)min(row, M - 1) * lda + min(k, K - 8);
                gs_cp_async(sbase + row * GS_ROW_BYTES + col * 16, src, (k + 8 <= K && row < M) ? 16 : 0);
            }
        }
    };
    auto advance = [&]() {
        ++q_issue;
        if (++i_stage == n_stages) { i_stage = 0; i_tile += gridDim.x; }
    };
    // The weights of the first steps do not depend on the kernel before this one: request them, then
    // wait for it, then request the activations of the same steps.
    {
        const int q0 = q_issue, t0 = i_tile, s0 = i_stage;
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) { issue_w(); advance(); }
        q_issue = q0; i_tile = t0; i_stage = s0;
    }
    pdl_wait();
    IMP_TL_WAITED()
    pdl_launch_dependents();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        issue_a();
        gs_commit();           // group s: activations of step s (group 0 also holds all the early weight copies)
        advance();
    }

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    int c_tile = blockIdx.x, c_stage = 0;      // consumer side
    for (int q = 0; q < total; ++q) {
        gs_wait_group<STAGES - 2>();   // step q has landed (for this thread's copies)
        __syncthreads();               // ... and for everyone's; the slot of step q-1 is free again
        issue_w();
        issue_a();
        gs_commit();                   // an empty group keeps the group count in step with the step count
        advance();
        const unsigned char* sp = gs_smem + (q % STAGES) * STAGE_BYTES + warp * (GS_KB * 2) + 32 * t;
        const unsigned char* wp = sp + rg * 16 * GS_ROW_BYTES;     // this row group's 16 weight rows
        const uint4 wa0 = *reinterpret_cast<const uint4*>(wp + g * GS_ROW_BYTES);
        const uint4 wa1 = *reinterpret_cast<const uint4*>(wp + g * GS_ROW_BYTES + 16);
        const uint4 wb0 = *reinterpret_cast<const uint4*>(wp + (g + 8) * GS_ROW_BYTES);
        const uint4 wb1 = *reinterpret_cast<const uint4*>(wp + (g + 8) * GS_ROW_BYTES + 16);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint4 c0 = *reinterpret_cast<const uint4*>(sp + W_BYTES + (8 * nt + g) * GS_ROW_BYTES);
            const uint4 c1 = *reinterpret_cast<const uint4*>(sp + W_BYTES + (8 * nt + g) * GS_ROW_BYTES + 16);
            gs_mma(acc[nt], wa0.x, wb0.x, wa0.y, wb0.y, c0.x, c0.y);
            gs_mma(acc[nt], wa0.z, wb0.z, wa0.w, wb0.w, c0.z, c0.w);
            gs_mma(acc[nt], wa1.x, wb1.x, wa1.y, wb1.y, c1.x, c1.y);
            gs_mma(acc[nt], wa1.z, wb1.z, wa1.w, wb1.w, c1.z, c1.w);
        }
        if (++c_stage < n_stages) continue;
        // ---- the tile is complete: add the four warps' sums in a fixed order and write ------------------
        const int n0 = c_tile * ROWS + rg * 16;
        const int tid_g = tid & (GS_WARPS * 32 - 1);     // thread within the row group
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                red[warp][nt * 4 + c][lane] = acc[nt][c];
                acc[nt][c] = 0.f;
            }
        __syncthreads();
        if (SWIGLU) {
            // 8 columns x 8*NT tokens; thread i takes (tile nt, slot c in {0,1}) = i / 32 and lane i % 32.
            for (int i = tid_g; i < NT * 64; i += GS_WARPS * 32) {
                const int r = i >> 5, l = i & 31;
                const int nt = r >> 1, c = r & 1;
                float gate = 0.f, up = 0.f;
#pragma unroll
                for (int w = 0; w < GS_WARPS; ++w) {
                    gate += red[w][nt * 4 + c][l];
                    up += red[w][nt * 4 + c + 2][l];
                }
                const int col = (c_tile * RG + rg) * 8 + (l >> 2);
                const int tok = 8 * nt + 2 * (l & 3) + c;
                if (n0 + (l >> 2) + 8 < N && tok < M)
                    C[(int64_t)tok * ldc + col] = from_float<TO>(gate / (1.f + expf(-gate)) * up);
            }
        } else {
            // 16 rows x 8*NT tokens = NT*128 sums; thread i takes register slot i / 32 of lane i % 32.
            for (int i = tid_g; i < NT * 128; i += GS_WARPS * 32) {
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
        c_stage = 0;
        c_tile += gridDim.x;
        // `red` is written again only after the next tile's steps, each of which passes a barrier
    }
    gs_wait_group<0>();
    IMP_TL_END()
}

template <int NT, typename TO, bool SWIGLU, int STAGES, int RG>
static cudaError_t launch_stream_st(TO* C, int64_t ldc, const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* W,
                                    int64_t ldw, int M, int N, int K, cudaStream_t s) {
    static bool attr_set = false;   // once per instantiation (one device per process)
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<NT, TO, SWIGLU, STAGES, RG>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, gs_smem_bytes(NT, STAGES, RG));
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const int n_tiles = (N + 16 * RG - 1) / (16 * RG);
    // One tile per CTA measured faster than two persistent CTAs per SM on every shape of the 8B model
    // (the kernel itself takes any grid size: a CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...).
    const int grid = n_tiles;
    return imp_launch(gemm_stream_kernel<NT, TO, SWIGLU, STAGES, RG>, dim3(grid), dim3(GS_WARPS * 32 * RG), gs_smem_bytes(NT, STAGES, RG), s, C, ldc,
                      A, lda, W, ldw, M, N, K);
}

// Ring depth.  Five stages let three CTAs share an SM (444 resident CTAs on a B200's 148 SMs).  A product with
// so few tiles that two CTAs per SM hold them all runs eight stages instead: every CTA then keeps
// 56 KiB of weight reads in flight, which the memory needs when only a few hundred CTAs pull on it.
// IMP_B200_GS_STAGES=4|5|6|8 forces one depth (for measurements).
static int gs_env_stages() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("IMP_B200_GS_STAGES");
        v = e ? atoi(e) : 0;
    }
    return v;
}

template <int NT, typename TO, bool SWIGLU>
static cudaError_t launch_stream_nt(TO* C, int64_t ldc, const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* W,
                                    int64_t ldw, int M, int N, int K, cudaStream_t s) {
    int stages = gs_env_stages();
    // Up to 8 tokens: two row groups per CTA where 32-row tiles still give about one CTA per SM or more.
    // With at least one such tile per SM, four stages of 21 KiB (two CTAs per SM); with 96/148 of that
    // and more (96..147 tiles on 148 SMs), six stages (one CTA per SM, 80 KiB of weight reads in flight each).  IMP_B200_GS_RG=1 keeps 16-row tiles
    // everywhere, =2 uses 32-row tiles only in the first case.
    static int rg_env = -1;
    if (rg_env < 0) { const char* e = getenv("IMP_B200_GS_RG"); rg_env = e ? atoi(e) : 3; }
    // (With one or two tokens the activations are a small share of the traffic and more, smaller CTAs win.)
    const int sms = imp_sm_count();
    if (NT == 1 && M >= 3 && rg_env >= 2 && stages == 0 && (N + 31) / 32 >= sms)
        return launch_stream_st<1, TO, SWIGLU, 4, 2>(C, ldc, A, lda, W, ldw, M, N, K, s);
    if (NT == 1 && M >= 3 && rg_env == 3 && stages == 0 && (N + 31) / 32 >= (sms * 96 + 147) / 148 && (N + 31) / 32 < sms)
        return launch_stream_st<1, TO, SWIGLU, 6, 2>(C, ldc, A, lda, W, ldw, M, N, K, s);
    if (stages == 0) stages = (NT == 1 && (N + 15) / 16 <= 2 * sms) ? 8 : 5;
    switch (stages) {
        case 4: return launch_stream_st<NT, TO, SWIGLU, 4, 1>(C, ldc, A, lda, W, ldw, M, N, K, s);
        case 6: return launch_stream_st<NT, TO, SWIGLU, 6, 1>(C, ldc, A, lda, W, ldw, M, N, K, s);
        case 8: return launch_stream_st<NT, TO, SWIGLU, 8, 1>(C, ldc, A, lda, W, ldw, M, N, K, s);
        default: return launch_stream_st<NT, TO, SWIGLU, 5, 1>(C, ldc, A, lda, W, ldw, M, N, K, s);
    }
}

template <typename TO, bool SWIGLU>
static int launch_stream(TO* C, int64_t ldc, const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* W, int64_t ldw,
                         int M, int N, int K, cudaStream_t s) {
    const cudaError_t e = (M <= 8) ? launch_stream_nt<1, TO, SWIGLU>(C, ldc, A, lda, W, ldw, M, N, K, s)
                                   : launch_stream_nt<2, TO, SWIGLU>(C, ldc, A, lda, W, ldw, M, N, K, s);
    if (e != cudaSuccess) {
        imp_set_error("gemm_stream: %s", cudaGetErrorString(e));
        return (int)e;
    }
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
        return launch_stream<float, false>((float*)C, ldc, (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, ldw, M,
                                           N, K, s);
    return launch_stream<__nv_bfloat16, false>((__nv_bfloat16*)C, ldc, (const __nv_bfloat16*)A, lda,
                                               (const __nv_bfloat16*)W, ldw, M, N, K, s);
}

// C[M, N/2] = silu(gate) * up where W[N, K] holds gate and up rows interleaved in blocks of 8
// (rows 16j..16j+7 = gate rows 8j..8j+7, rows 16j+8..16j+15 = up rows 8j..8j+7); bfloat16 output.
IMP_API int imp_gemm_bf16_stream_swiglu(void* C, int64_t ldc, const void* A, int64_t lda, const void* W, int64_t ldw,
                                        int M, int N, int K, void* stream) {
    if (M == 0 || N == 0) return 0;
    IMP_CHECK_ARG(C && A && W && M > 0 && N > 0 && K > 0, "imp_gemm_bf16_stream_swiglu: bad argument");
    IMP_CHECK_ARG(M <= 16, "imp_gemm_bf16_stream_swiglu: M %d exceeds 16", M);
    IMP_CHECK_ARG(N % 16 == 0, "imp_gemm_bf16_stream_swiglu: %d interleaved rows are not a multiple of 16", N);
    IMP_CHECK_ARG(ldc >= N / 2 && lda >= K && ldw >= K, "imp_gemm_bf16_stream_swiglu: leading dimension too small");
    if (K % 8 || lda % 8 || ldw % 8 || (uintptr_t)A % 16 || (uintptr_t)W % 16) return IMP_ERR_UNSUPPORTED;
    return launch_stream<__nv_bfloat16, true>((__nv_bfloat16*)C, ldc, (const __nv_bfloat16*)A, lda,
                                              (const __nv_bfloat16*)W, ldw, M, N, K, (cudaStream_t)stream);
}
