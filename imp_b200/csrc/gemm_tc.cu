// Prefill matrix product on the fifth-generation tensor cores:  C[M,N] = A[M,K] * W[N,K]^T,
// bfloat16 operands (both K-major, as activations and weights are stored), 32-bit accumulation in
// tensor memory, bfloat16 or 32-bit output, optionally with the SwiGLU activation fused into the
// epilogue.
//
// One CTA computes a 128 x 256 tile.  Lane 0 of warp 0 is the producer: it walks K in blocks of 64
// elements and fetches the A tile (128 x 64) and the W tile (256 x 64) of each block with two TMA
// loads (cp.async.bulk.tensor, 128-byte swizzle) into a 4-deep shared-memory ring, signalling an
// mbarrier per stage.  Lane 0 of warp 1 issues the MMAs: four tcgen05.mma (M=128, N=256, K=16) per
// stage, operands straight from shared memory through matrix descriptors, accumulator in 256
// columns of tensor memory; tcgen05.commit hands each stage back to the producer and, after the
// last block, tells the epilogue that the accumulator is complete.  Then all four warps read the
// accumulator with tcgen05.ld (warp w owns rows 32w..32w+31), convert and store.
//
// Every wait on an mbarrier is bounded: after TC_WAIT_LIMIT failed polls the thread records
// IMP_WAIT_TIMEOUT in the status word and leaves its loop; all threads then meet at the final
// barrier, tensor memory is freed and the CTA returns (its output is then undefined; the host
// sees the status).  The producer first waits, again bounded, for the copies it still has in
// flight.
//
// Reference counterpart: gemm() -> cublasLtMatmul with fp16 inputs and fp32 accumulation
// (src/compute/gemm.cu:303-445); the reference has no tensor-memory kernel of its own.
#include "common.cuh"

#include <cuda.h>

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64, TC_STAGES = 4, TC_UMMA_K = 16;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;   // 16 KiB
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;   // 32 KiB
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 20;   // polls of mbarrier.try_wait (each suspends for a while): about a second
constexpr int TC_TMEM_COLS = 256;

enum TcEpilogue : int { TC_OUT_BF16 = 0, TC_OUT_F32 = 1, TC_OUT_SWIGLU_BF16 = 2 };

// ---------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false (and a status report) when it runs out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    imp_report(status, IMP_WAIT_TIMEOUT);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile written by TMA with the 128-byte swizzle:
// rows of 128 bytes, groups of 8 rows 1024 bytes apart (stride byte offset), no leading offset.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);        // start address, 16-byte units
    d |= (uint64_t)(1024u >> 4) << 32;              // stride byte offset
    d |= (uint64_t)1 << 46;                         // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                         // layout: 128-byte swizzle
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M x N tile.
__device__ __forceinline__ uint32_t tc_instr_desc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators: lane i of the warp gets row (lane base + i).
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// ------------------------------------------------------------------------------------- kernel
template <int EPI>
__global__ void __launch_bounds__(128, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                         const __grid_constant__ CUtensorMap map_w, void* __restrict__ Cv,
                                                         int64_t ldc, int M, int N, int K, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ unsigned char tc_smem_raw[];
    // tiles must start on 1024-byte boundaries (8 rows of the 128-byte swizzle)
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TC_STAGES * TC_STAGE_BYTES);
    // bars[0..S) full, bars[S..2S) empty, bars[2S] accumulator ready; then the tensor-memory base address
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * TC_BN;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + TC_STAGES), accum_bar = smem_u32(bars + 2 * TC_STAGES);

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // one warp allocates the accumulator's columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------------ producer
        int issued = 0;
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
            const int s = kb % TC_STAGES;
            const uint32_t round = (uint32_t)(kb / TC_STAGES);
            ok = mbar_wait(empty0 + 8 * s, (round & 1u) ^ 1u, status);   // the slot's previous MMAs are done
            if (!ok) break;
            const uint32_t a_dst = smem_u32(tiles + s * TC_STAGE_BYTES), b_dst = a_dst + TC_A_BYTES;
            mbar_expect_tx(full0 + 8 * s, TC_STAGE_BYTES);
            tma_load_2d(a_dst, &map_a, kb * TC_BK, m0, full0 + 8 * s);
            tma_load_2d(b_dst, &map_w, kb * TC_BK, n0, full0 + 8 * s);
            issued = kb + 1;
        }
        if (!ok) {
            // give the copies still in flight a bounded chance to land before the CTA's memory is released
            for (int kb = issued > TC_STAGES ? issued - TC_STAGES : 0; kb < issued; ++kb)
                mbar_wait(full0 + 8 * (kb % TC_STAGES), (uint32_t)(kb / TC_STAGES) & 1u, nullptr);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------------- MMA issuer
        const uint32_t idesc = tc_instr_desc(TC_BM, TC_BN);
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
            const int s = kb % TC_STAGES;
            ok = mbar_wait(full0 + 8 * s, (uint32_t)(kb / TC_STAGES) & 1u, status);   // the stage's tiles have landed
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t a_addr = smem_u32(tiles + s * TC_STAGE_BYTES), b_addr = a_addr + TC_A_BYTES;
#pragma unroll
            for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)
                tc_mma(tmem_base, tc_smem_desc(a_addr + k * TC_UMMA_K * 2), tc_smem_desc(b_addr + k * TC_UMMA_K * 2), idesc,
                       (kb > 0 || k > 0) ? 1u : 0u);
            tc_commit(empty0 + 8 * s);   // the slot is free once these MMAs have read it
        }
        tc_commit(accum_bar);            // arrives when every MMA issued so far has completed
    }
    __syncwarp();

    // -------------------------------------------------------------------------- epilogue
    const bool acc_ok = __all_sync(0xffffffffu, mbar_wait(accum_bar, 0, status));   // the same verdict for the whole warp
    tc_fence_after_sync();
    if (acc_ok) {
        const int row = m0 + warp * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
        for (int c = 0; c < TC_BN / 32; ++c) {
            float v[32];
            tc_ld32(lane_base + (uint32_t)(c * 32), v);
            const int col0 = n0 + c * 32;
            if (row >= M || col0 >= N) continue;
            if (EPI == TC_OUT_F32) {
                float* dst = reinterpret_cast<float*>(Cv) + (int64_t)row * ldc + col0;
                if (col0 + 32 <= N && (ldc % 4) == 0) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                } else {
                    for (int i = 0; i < 32 && col0 + i < N; ++i) dst[i] = v[i];
                }
            } else if (EPI == TC_OUT_BF16) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cv) + (int64_t)row * ldc + col0;
                if (col0 + 32 <= N && (ldc % 8) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 o;
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * i], v[8 * i + 1]);
                        __nv_bfloat162 p1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
                        __nv_bfloat162 p3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
                        o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
                        o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
                        reinterpret_cast<uint4*>(dst)[i] = o;
                    }
                } else {
                    for (int i = 0; i < 32 && col0 + i < N; ++i) dst[i] = __float2bfloat16_rn(v[i]);
                }
            } else {
                // columns 16j..16j+7 are gate, 16j+8..16j+15 the matching up: 32 columns give 16 outputs
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cv) + (int64_t)row * ldc + (col0 >> 1);
                __nv_bfloat16 o[16];
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float gate = v[16 * j + i], up = v[16 * j + 8 + i];
                        o[8 * j + i] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
                    }
                if (col0 + 32 <= N && (ldc % 8) == 0) {
                    reinterpret_cast<uint4*>(dst)[0] = *reinterpret_cast<uint4*>(&o[0]);
                    reinterpret_cast<uint4*>(dst)[1] = *reinterpret_cast<uint4*>(&o[8]);
                } else {
                    for (int i = 0; i < 16 && col0 + 2 * i < N; ++i) dst[i] = o[i];
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TC_TMEM_COLS)
                     : "memory");
    }
}

// ------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld elements, fetched in boxes of box_rows x 64 elements.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int64_t ld, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        imp_set_error("gemm_tc: the driver does not provide cuTensorMapEncodeTiled");
        return IMP_ERR_UNSUPPORTED;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        imp_set_error("gemm_tc: cuTensorMapEncodeTiled failed with code %d (rows %d, K %d, ld %lld)", (int)r, rows, K,
                      (long long)ld);
        return IMP_ERR_ARG;
    }
    return 0;
}

template <int EPI>
static int launch_tc(void* C, int64_t ldc, const CUtensorMap& ma, const CUtensorMap& mw, int M, int N, int K, int* status,
                     cudaStream_t s) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (e != cudaSuccess) { imp_set_error("gemm_tc: %s", cudaGetErrorString(e)); return (int)e; }
        attr_set = true;
    }
    dim3 grid((M + TC_BM - 1) / TC_BM, (N + TC_BN - 1) / TC_BN);
    gemm_tc_kernel<EPI><<<grid, 128, TC_SMEM_BYTES, s>>>(ma, mw, C, ldc, M, N, K, status);
    IMP_RETURN_LAUNCH();
}

// epilogue: 0 = bfloat16 C[M,N]; 1 = float32 C[M,N]; 2 = bfloat16 C[M,N/2] = silu(gate) * up with
// gate and up rows of W interleaved in runs of 8.
// Returns IMP_ERR_UNSUPPORTED when the operands do not meet the alignment rules of the tensor copies
// (bases on 16-byte boundaries, row strides multiples of 8 elements): the caller uses another kernel.
IMP_API int imp_gemm_bf16_tc(void* C, int64_t ldc, int epilogue, const void* A, int64_t lda, const void* W, int64_t ldw,
                             int M, int N, int K, int* status, void* stream) {
    if (M == 0 || N == 0) return 0;
    IMP_CHECK_ARG(C && A && W && M > 0 && N > 0 && K > 0, "imp_gemm_bf16_tc: bad argument");
    IMP_CHECK_ARG(epilogue >= 0 && epilogue <= 2, "imp_gemm_bf16_tc: unknown epilogue %d", epilogue);
    IMP_CHECK_ARG(lda >= K && ldw >= K && ldc >= (epilogue == 2 ? N / 2 : N), "imp_gemm_bf16_tc: leading dimension too small");
    if (epilogue == 2) IMP_CHECK_ARG(N % 16 == 0, "imp_gemm_bf16_tc: %d interleaved rows are not a multiple of 16", N);
    if (K % 8 || lda % 8 || ldw % 8 || (uintptr_t)A % 16 || (uintptr_t)W % 16 || (uintptr_t)C % 16) return IMP_ERR_UNSUPPORTED;
    CUtensorMap ma, mw;
    if (int rc = make_map(&ma, A, M, K, lda, TC_BM)) return rc;
    if (int rc = make_map(&mw, W, N, K, ldw, TC_BN)) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == TC_OUT_BF16) return launch_tc<TC_OUT_BF16>(C, ldc, ma, mw, M, N, K, status, s);
    if (epilogue == TC_OUT_F32) return launch_tc<TC_OUT_F32>(C, ldc, ma, mw, M, N, K, status, s);
    return launch_tc<TC_OUT_SWIGLU_BF16>(C, ldc, ma, mw, M, N, K, status, s);
}
