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
#include "tc_common.cuh"

#include <cstdlib>

IMP_TL_DEFINE(gemm_tc)

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64, TC_STAGES = 4, TC_UMMA_K = 16;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;   // 16 KiB
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;   // 32 KiB
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int TC_TMEM_COLS = 256;

enum TcEpilogue : int { TC_OUT_BF16 = 0, TC_OUT_F32 = 1, TC_OUT_SWIGLU_BF16 = 2, TC_OUT_QKV_ROPE = 3 };

// Store 32 consecutive accumulator columns of one row (converted as the epilogue asks).
template <int EPI>
__device__ __forceinline__ void tc_store32(void* __restrict__ Cv, int64_t ldc, int row, int col0, int M, int N,
                                           const float (&v)[32]) {
    if (row >= M || col0 >= N) return;
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
        __align__(16) __nv_bfloat16 o[16];
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
            tc_store32<EPI>(Cv, ldc, row, n0 + c * 32, M, N, v);
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

// ------------------------------------------------------------------- persistent kernel
// One CTA per SM walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (M index fastest, so the CTAs
// running together share W tiles in L2).  Six warps: warp 0 produces (lane 0), warp 1 issues the
// MMAs (lane 0) and owns tensor memory, warps 2-5 are the epilogue.  Tensor memory holds two
// accumulators of 256 columns: while the epilogue warps drain one, the MMAs of the next tile fill
// the other, so the tensor cores do not wait for stores.
constexpr int TCP_THREADS = 192;
constexpr int TCP_TMEM_COLS = 512;

template <int EPI>
__global__ void __launch_bounds__(TCP_THREADS, 1) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                            const __grid_constant__ CUtensorMap map_w,
                                                                            void* __restrict__ Cv, int64_t ldc, int M, int N,
                                                                            int K, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TC_STAGES * TC_STAGE_BYTES);
    // bars: [0,S) full, [S,2S) empty, [2S,2S+2) accumulator full, [2S+2,2S+4) accumulator empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const int num_m = (M + TC_BM - 1) / TC_BM, num_n = (N + TC_BN - 1) / TC_BN;
    const int total = num_m * num_n;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + TC_STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * TC_STAGES), acce0 = smem_u32(bars + 2 * TC_STAGES + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, 4);     // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TCP_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // -------------------------------------------------------------- producer
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const int m0 = (t % num_m) * TC_BM, n0 = (t / num_m) * TC_BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % TC_STAGES;
                    ok = mbar_wait(empty0 + 8 * s, ((it / TC_STAGES) & 1u) ^ 1u, status);
                    if (!ok) break;
                    const uint32_t a_dst = smem_u32(tiles + s * TC_STAGE_BYTES), b_dst = a_dst + TC_A_BYTES;
                    mbar_expect_tx(full0 + 8 * s, TC_STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, kb * TC_BK, m0, full0 + 8 * s);
                    tma_load_2d(b_dst, &map_w, kb * TC_BK, n0, full0 + 8 * s);
                }
            }
            if (!ok) {   // a bounded chance for the copies still in flight to land before the memory is released
                for (uint32_t j = it > TC_STAGES ? it - TC_STAGES : 0; j < it; ++j)
                    mbar_wait(full0 + 8 * (j % TC_STAGES), (j / TC_STAGES) & 1u, nullptr);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ------------------------------------------------------------ MMA issuer
            const uint32_t idesc = tc_instr_desc(TC_BM, TC_BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++local) {
                const uint32_t buf = local & 1u;
                ok = mbar_wait(acce0 + 8 * buf, ((local >> 1) & 1u) ^ 1u, status);   // the epilogue has drained it
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * TC_BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % TC_STAGES;
                    ok = mbar_wait(full0 + 8 * s, (it / TC_STAGES) & 1u, status);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(tiles + s * TC_STAGE_BYTES), b_addr = a_addr + TC_A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)
                        tc_mma(d_tmem, tc_smem_desc(a_addr + k * TC_UMMA_K * 2), tc_smem_desc(b_addr + k * TC_UMMA_K * 2),
                               idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);
                }
                if (ok) tc_commit(accf0 + 8 * buf);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp & 3;                       // the 32 lanes of tensor memory this warp may read
        uint32_t local = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++local) {
            const uint32_t buf = local & 1u;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(accf0 + 8 * buf, (local >> 1) & 1u, status));
            if (!ok) break;
            tc_fence_after_sync();
            const int m0 = (t % num_m) * TC_BM, n0 = (t / num_m) * TC_BN;
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TC_BN;
#pragma unroll 1
            for (int c = 0; c < TC_BN / 32; ++c) {
                float v[32];
                tc_ld32(taddr + (uint32_t)(c * 32), v);
                tc_store32<EPI>(Cv, ldc, row, n0 + c * 32, M, N, v);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce0 + 8 * buf);    // this warp's quarter of the accumulator is free
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TCP_TMEM_COLS)
                     : "memory");
    }
}

// ------------------------------------------------ epilogue of the fused q,k,v projection
// With TC_OUT_QKV_ROPE the product's columns are the heads of q, then k, then v (head size 64 or 128, so
// a 256-column tile holds whole heads) and nothing is written as a [M, N] matrix: a thread, which owns a
// token's row of the accumulator, normalises each q and k head (RMSNorm over the head with one weight
// vector for q and one for k, 32-bit), rotates it by the token's position (pairs (i, i + Dh/2), cos / sin
// from a table) and writes q to its own buffer and k to the token's slot of the cache pages; v heads go
// to the pages as they are.  The values never round to bfloat16 in between.  Same math as
// qk_norm_rope_kv_kernel (rope_kv.cu), which runs after an unfused product.
struct QkvRopeArgs {
    const int* positions;        // [M]
    const int* seq_of_token;     // [M]
    const int* block_table;      // [n_seqs, bt_stride]
    const float* cos_tab;        // [max_pos, Dh / 2]
    const float* sin_tab;
    const float* q_norm_w;       // [Dh] or null (no norm)
    const float* k_norm_w;
    __nv_bfloat16* q_out;        // [M, q_stride], head h at column h * Dh
    __nv_bfloat16* k_cache;      // [num_pages, Hkv, page_size, Dh]
    __nv_bfloat16* v_cache;
    int64_t q_stride;
    float eps;
    int bt_stride, n_seqs, max_pos, Hq, Hkv, Dh, page_size, num_pages;
};

// The product as the other paths see it: rounded to bfloat16 before the per-head norm and the rotation, so that a
// token's cached key has the same bits whether its q,k,v came from this epilogue or from a product that wrote
// bfloat16 and a separate norm-and-rotation kernel.
__device__ __forceinline__ void round32_bf16(float (&v)[32]) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
}

__device__ __forceinline__ void store32_bf16(__nv_bfloat16* dst, const float (&v)[32]) {
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
}

// Output staging of the CTA-pair kernel: buffers of 128 rows x 128 bytes (64 bfloat16 columns), written row by row with
// the 128-byte swizzle and handed to TMA stores.
constexpr int TC2_OUT_BYTES = 128 * 128;
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y), "r"(src)
                 : "memory");
}
__device__ __forceinline__ uint4 tc2_pack8(const float* v) {
    uint4 o;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
    o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
    o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
    return o;
}
// Where the q part of the fused epilogue goes when it leaves through TMA stores (bufs == nullptr: every thread stores
// its own row): the two staging buffers, q's tensor map, whether this thread issues the stores, the thread's row in
// the CTA's half tile and that half tile's first row in q.
struct QkvStage {
    unsigned char* bufs;
    const CUtensorMap* map;
    bool storer;
    int r, m0;
};

// One accumulator row (token `row`, tensor-memory address `taddr` of its first column) of the tile that
// starts at column n0.  All 32 lanes of the warp call it together (the tensor-memory loads are collective);
// `live` says whether this lane's row exists.
__device__ __forceinline__ void qkv_rope_row(const QkvRopeArgs& a, uint32_t taddr, int row, int n0, int N, bool live,
                                             int* status, const QkvStage& stg) {
    const int Dh = a.Dh, half = Dh >> 1, chunks = Dh >> 5;          // 32-column chunks per head: 2 or 4
    int pos = 0;
    int64_t page_row = -1;
    if (live) {
        pos = a.positions[row];
        const int seq = a.seq_of_token[row];
        if (seq < 0 || seq >= a.n_seqs) {
            imp_report(status, IMP_BAD_SEQUENCE);
            live = false;
        } else if (pos < 0 || pos >= a.max_pos || pos / a.page_size >= a.bt_stride) {
            imp_report(status, IMP_TAGGED(IMP_BAD_POSITION, 5));
            live = false;
        } else {
            const int slot_page = pos / a.page_size;
            const int page = a.block_table[(int64_t)seq * a.bt_stride + slot_page];
            if (page < 0 || page >= a.num_pages) imp_report(status, IMP_BAD_PAGE);
            else page_row = (int64_t)page * a.Hkv * a.page_size + (pos - slot_page * a.page_size);
        }
    }
    const float* cs = a.cos_tab + (int64_t)pos * half;
    const float* sn = a.sin_tab + (int64_t)pos * half;
    for (int h0 = 0; h0 < 256; h0 += Dh) {
        const int col0 = n0 + h0;
        if (col0 >= N) break;                                       // uniform over the warp
        const int hh = col0 / Dh;
        const uint32_t thead = taddr + (uint32_t)h0;
        if (hh >= a.Hq + a.Hkv) {
            // ---- v: to the pages as it is
            __nv_bfloat16* dst = (live && page_row >= 0) ? a.v_cache + (page_row + (int64_t)(hh - a.Hq - a.Hkv) * a.page_size) * Dh
                                                         : nullptr;
            for (int c = 0; c < chunks; ++c) {
                float v[32];
                tc_ld32(thead + (uint32_t)(c * 32), v);
                if (dst) store32_bf16(dst + c * 32, v);
            }
            continue;
        }
        const bool is_q = hh < a.Hq;
        const float* nw = is_q ? a.q_norm_w : a.k_norm_w;
        float inv = 1.f;
        if (nw) {
            float ss = 0.f;
            for (int c = 0; c < chunks; ++c) {
                float v[32];
                tc_ld32(thead + (uint32_t)(c * 32), v);
                round32_bf16(v);
#pragma unroll
                for (int i = 0; i < 32; ++i) ss = fmaf(v[i], v[i], ss);
            }
            inv = rsqrtf(ss / (float)Dh + a.eps);
        }
        const bool staged = is_q && stg.bufs != nullptr;            // uniform over the CTA's epilogue warps
        __nv_bfloat16* dst = nullptr;
        if (live) {
            if (is_q) dst = a.q_out + (int64_t)row * a.q_stride + (int64_t)hh * Dh;
            else if (page_row >= 0) dst = a.k_cache + (page_row + (int64_t)(hh - a.Hq) * a.page_size) * Dh;
        }
        if (staged) {
            // both buffers are free once the stores of the head before have read them
            if (stg.storer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        for (int c = 0; c < chunks / 2; ++c) {                      // dims [32c, 32c+32) pair with [half + 32c, ...)
            float x[32], y[32];
            tc_ld32(thead + (uint32_t)(c * 32), x);
            tc_ld32(thead + (uint32_t)(half + c * 32), y);
            if (dst == nullptr && !staged) continue;                // (a staged row without a token writes what TMA clips)
            round32_bf16(x);
            round32_bf16(y);
            // the table row of this token is read 16 bytes at a time: 32 rows touch 32 sectors per load either
            // way, so fewer, wider loads keep the L1 out of the way
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
                const float4 co4 = *reinterpret_cast<const float4*>(cs + c * 32 + 4 * i4);
                const float4 si4 = *reinterpret_cast<const float4*>(sn + c * 32 + 4 * i4);
                const float co[4] = {co4.x, co4.y, co4.z, co4.w}, si[4] = {si4.x, si4.y, si4.z, si4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = 4 * i4 + j, d = c * 32 + i;
                    float xa = x[i] * inv, yb = y[i] * inv;
                    if (nw) { xa *= nw[d]; yb *= nw[d + half]; }
                    x[i] = xa * co[j] - yb * si[j];
                    y[i] = xa * si[j] + yb * co[j];
                }
            }
            if (staged) {
                // 32 dims = four 16-byte pieces of the row of the 64-column buffer they fall into
                const int dx = c * 32, dy = half + c * 32;
                unsigned char* rx = stg.bufs + (dx >> 6) * TC2_OUT_BYTES + stg.r * 128;
                unsigned char* ry = stg.bufs + (dy >> 6) * TC2_OUT_BYTES + stg.r * 128;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    *reinterpret_cast<uint4*>(rx + (((((dx & 63) >> 3) + i) ^ (stg.r & 7)) << 4)) = tc2_pack8(x + 8 * i);
                    *reinterpret_cast<uint4*>(ry + (((((dy & 63) >> 3) + i) ^ (stg.r & 7)) << 4)) = tc2_pack8(y + 8 * i);
                }
            } else {
                store32_bf16(dst + c * 32, x);
                store32_bf16(dst + half + c * 32, y);
            }
        }
        if (staged) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (stg.storer) {
                for (int sub = 0; sub < Dh / 64; ++sub)
                    tma_store_2d(stg.map, smem_u32(stg.bufs + sub * TC2_OUT_BYTES), hh * Dh + sub * 64, stg.m0);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
    }
}

// ------------------------------------------------------------ pairs of CTAs (cta_group::2)
// Two CTAs of a cluster, on neighbouring SMs, compute one 256 x 256 tile together.  Each of them loads
// its own 128 rows of A and its own half (128 rows) of the W tile, so a k-block costs an SM 32 KiB of
// shared-memory fill instead of 48; the MMA (M = 256, N = 256, issued by the even CTA for both) reads
// W from both CTAs' shared memory, and each CTA's tensor memory receives the accumulator of its own 128
// rows.  Protocol, per stage s of the six-deep ring (barriers live at the same offsets in both CTAs):
//   full[s]   in the even CTA only: its producer announces the bytes of both CTAs' copies, all four TMA
//             loads (cta_group::2) complete on it;
//   empty[s]  in both: the MMA's commit arrives on both at once (multicast), each producer waits its own;
//   accumulator full: the commit after a tile's last MMA, again on both; accumulator empty: in the even
//   CTA, eight arrivals (four epilogue warps of each CTA, the odd CTA's through the cluster's shared
//   window).
// Both CTAs pass a cluster barrier after initialising their barriers and before they leave.
constexpr int TC2_STAGES = 6;
constexpr int TC2_HALF_BYTES = 128 * TC_BK * 2;                 // 16 KiB: 128 rows of A, or of W
constexpr int TC2_STAGE_BYTES = 2 * TC2_HALF_BYTES;
// Output staging for the bfloat16 epilogues: two buffers of 128 rows x 128 bytes (64 output columns), written row by
// row with the 128-byte swizzle and handed to TMA stores.  (Each thread storing 16 bytes to its own row of C cost a
// 2,048 x 4,096 x 4,096 product 8 % of its time and one of 512 rows 12 %.)
constexpr int TC2_RING_BYTES = TC2_STAGES * TC2_STAGE_BYTES;
constexpr int TC2_SMEM_BYTES = TC2_RING_BYTES + 2 * TC2_OUT_BYTES + 1024 + 256;
static_assert(TC2_SMEM_BYTES <= 227 * 1024, "the pair kernel's shared memory");


constexpr int TC2_BM = 256, TC2_BN = 256;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of `addr` (an address in this CTA's shared memory) in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: the copy lands in this CTA's shared memory, its bytes count on `bar`,
// which may be the partner's barrier (an address in the cluster's shared window).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The barrier at this offset in both CTAs of the pair gets an arrival when the MMAs issued so far are done.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TCP_THREADS, 1)
    gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        void* __restrict__ Cv, int64_t ldc, int M, int N, int K, int* status,
                        const __grid_constant__ QkvRopeArgs qkv, int splits, int kb_per_split, int64_t split_stride,
                        const __grid_constant__ CUtensorMap map_c, int tma_store) {
    // tma_store (bfloat16 and SwiGLU epilogues): C goes out through shared memory and TMA stores described by map_c
    // (boxes of 128 rows x 64 columns, clipped at the matrix edges) instead of 16-byte stores from every thread.
    // splits > 1 (32-bit output only): the K range is cut into `splits` parts, each (tile, part) is a unit of work of its
    // own and writes its partial product split_stride elements after the part before; the caller adds the parts in order.
    IMP_TL_BEGIN(20 + EPI)
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* out_stage = tiles + TC2_RING_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + 2 * TC2_OUT_BYTES);
    // bars: [0,S) full, [S,2S) empty, [2S,2S+2) accumulator full, [2S+2,2S+4) accumulator empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC2_STAGES + 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const int num_m = (M + TC2_BM - 1) / TC2_BM, num_n = (N + TC2_BN - 1) / TC2_BN;
    const int n_tiles = num_m * num_n;
    const int total = n_tiles * splits;            // units: all tiles of part 0, then all of part 1, ...
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + TC2_STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * TC2_STAGES), acce0 = smem_u32(bars + 2 * TC2_STAGES + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC2_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, 8);     // four epilogue warps of each CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // the same warp of both CTAs, the same slot offset
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TCP_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();        // the partner's barriers are initialised before anything can arrive on them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Up to here nothing read or wrote what an earlier kernel of the stream may still be working on.
    pdl_wait();
    IMP_TL_WAITED()
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------ producer (one per CTA, for its own halves)
            uint32_t it = 0;
            bool ok = true;
            for (int u = pair; u < total && ok; u += n_pairs) {
                const int t = u % n_tiles, z = u / n_tiles;
                const int kb_lo = z * kb_per_split, kb_hi = min(k_blocks, kb_lo + kb_per_split);
                const int m0 = (t % num_m) * TC2_BM + (int)rank * 128, n0 = (t / num_m) * TC2_BN + (int)rank * 128;
                for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
                    const uint32_t s = it % TC2_STAGES;
                    ok = mbar_wait(empty0 + 8 * s, ((it / TC2_STAGES) & 1u) ^ 1u, status);
                    if (!ok) break;
                    const uint32_t a_dst = smem_u32(tiles + s * TC2_STAGE_BYTES), b_dst = a_dst + TC2_HALF_BYTES;
                    const uint32_t full_even = cluster_map(full0 + 8 * s, 0);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * TC2_STAGE_BYTES);   // both CTAs' copies
                    tma_load_2d_pair(a_dst, &map_a, kb * TC_BK, m0, full_even);
                    tma_load_2d_pair(b_dst, &map_w, kb * TC_BK, n0, full_even);
                }
            }
            if (!ok && rank == 0) {   // a bounded chance for the copies still in flight to land
                for (uint32_t j = it > TC2_STAGES ? it - TC2_STAGES : 0; j < it; ++j)
                    mbar_wait(full0 + 8 * (j % TC2_STAGES), (j / TC2_STAGES) & 1u, nullptr);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ------------------------------------------------------------ MMA issuer (even CTA)
            const uint32_t idesc = tc_instr_desc(TC2_BM, TC2_BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int u = pair; u < total && ok; u += n_pairs, ++local) {
                const int z = u / n_tiles;
                const int kb_lo = z * kb_per_split, kb_hi = min(k_blocks, kb_lo + kb_per_split);
                const uint32_t buf = local & 1u;
                ok = mbar_wait(acce0 + 8 * buf, ((local >> 1) & 1u) ^ 1u, status);   // both epilogues have drained it
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * TC2_BN;
                for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
                    const uint32_t s = it % TC2_STAGES;
                    ok = mbar_wait(full0 + 8 * s, (it / TC2_STAGES) & 1u, status);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(tiles + s * TC2_STAGE_BYTES), b_addr = a_addr + TC2_HALF_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)
                        tc_mma_pair(d_tmem, tc_smem_desc(a_addr + k * TC_UMMA_K * 2), tc_smem_desc(b_addr + k * TC_UMMA_K * 2),
                                    idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
                    tc_commit_pair(empty0 + 8 * s);
                }
                if (ok) tc_commit_pair(accf0 + 8 * buf);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const int quarter = warp & 3;
        const uint32_t acce_even0 = cluster_map(acce0, 0);
        const bool storer = warp == 2 && lane == 0;      // issues the TMA stores and waits for them
        uint32_t out_n = 0;                              // staging buffers used so far
        uint32_t local = 0;
        for (int u = pair; u < total; u += n_pairs, ++local) {
            const int t = u % n_tiles, z = u / n_tiles;
            const uint32_t buf = local & 1u;
            bool ok = __all_sync(0xffffffffu, mbar_wait(accf0 + 8 * buf, (local >> 1) & 1u, status));
            if (EPI != TC_OUT_F32 && tma_store) {
                // the four warps meet at barriers below: they go on, or give up, together
                uint32_t all;
                asm volatile(
                    "{\n"
                    ".reg .pred p, q;\n"
                    "setp.ne.u32 p, %1, 0;\n"
                    "bar.red.and.pred q, 2, 128, p;\n"
                    "selp.u32 %0, 1, 0, q;\n"
                    "}\n"
                    : "=r"(all)
                    : "r"((uint32_t)ok)
                    : "memory");
                ok = all != 0;
            }
            if (!ok) break;
            tc_fence_after_sync();
            const int m0 = (t % num_m) * TC2_BM + (int)rank * 128, n0 = (t / num_m) * TC2_BN;
            void* Cz = EPI == TC_OUT_F32 ? (void*)(reinterpret_cast<float*>(Cv) + (int64_t)z * split_stride) : Cv;
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TC2_BN;
            // TMA stores only for a CTA's 128 rows that all lie inside C (and whole 64-column pieces): a store that the
            // tensor map clips measured far slower than the threads' own stores (2048 x 24576 outputs cut at 320 rows:
            // 97 us against 78), so the last, partly filled row block of a matrix takes the plain path.
            const bool whole = m0 + 128 <= M && n0 + TC2_BN <= N;
            if (EPI == TC_OUT_QKV_ROPE) {
                const QkvStage stg{tma_store && m0 + 128 <= M ? out_stage : nullptr, &map_c, storer, quarter * 32 + lane, m0};
                qkv_rope_row(qkv, taddr, row, n0, N, row < M, status, stg);
            } else if ((EPI == TC_OUT_BF16 || EPI == TC_OUT_SWIGLU_BF16) && tma_store && whole) {
                constexpr int SUBS = EPI == TC_OUT_SWIGLU_BF16 ? 2 : 4;     // sub-tiles of 64 output columns
                const int x0 = EPI == TC_OUT_SWIGLU_BF16 ? n0 >> 1 : n0;
                const int r = quarter * 32 + lane;                          // row in the CTA's half of the tile
#pragma unroll 1
                for (int j = 0; j < SUBS; ++j, ++out_n) {
                    unsigned char* buf = out_stage + (out_n & 1u) * TC2_OUT_BYTES;
                    // the store that read this buffer two sub-tiles ago has finished reading it
                    if (storer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    uint4 q[8];
                    if (EPI == TC_OUT_BF16) {
#pragma unroll
                        for (int cc = 0; cc < 2; ++cc) {
                            float v[32];
                            tc_ld32(taddr + (uint32_t)((2 * j + cc) * 32), v);
#pragma unroll
                            for (int i = 0; i < 4; ++i) q[4 * cc + i] = tc2_pack8(v + 8 * i);
                        }
                    } else {
                        // 32 accumulator columns = gate (8), up (8), gate (8), up (8): 16 outputs
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) {
                            float v[32], o[16];
                            tc_ld32(taddr + (uint32_t)((4 * j + cc) * 32), v);
#pragma unroll
                            for (int h = 0; h < 2; ++h)
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    const float gate = v[16 * h + i], up = v[16 * h + 8 + i];
                                    o[8 * h + i] = gate / (1.f + expf(-gate)) * up;
                                }
                            q[2 * cc] = tc2_pack8(o);
                            q[2 * cc + 1] = tc2_pack8(o + 8);
                        }
                    }
                    unsigned char* rowp = buf + r * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(rowp + ((c ^ (r & 7)) << 4)) = q[c];
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (storer) {
                        tma_store_2d(&map_c, smem_u32(buf), x0 + j * 64, m0);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < TC2_BN / 32; ++c) {
                    float v[32];
                    tc_ld32(taddr + (uint32_t)(c * 32), v);
                    tc_store32<EPI == TC_OUT_QKV_ROPE ? TC_OUT_BF16 : EPI>(Cz, ldc, row, n0 + c * 32, M, N, v);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acce_even0 + 8 * buf);
        }
        if (storer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // C is written before the CTA leaves
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();        // neither CTA leaves while the other may still read its memory or signal its barriers
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TCP_TMEM_COLS)
                     : "memory");
    }
    IMP_TL_END()
}

// ------------------------------------------------------- few rows: weights on the M side
// For up to 128 activation rows the product is turned round, as in the decode kernel of
// gemm_stream.cu: up to 128 weight rows are the M side of the MMA (one accumulator lane per weight row),
// the activation rows its N side (BN = 32, 64 or 128 columns of tensor memory).  A CTA streams its
// weight rows through a TMA ring; with few weight-row tiles the K range is cut into
// `splits` parts (grid.z) so that every SM pulls on the memory, each part writing a 32-bit partial
// result that gemm_tc_reduce_kernel adds up in split order.
// Epilogue: lane r of the accumulator is output column n0 + r, column t is token t, so consecutive
// lanes write consecutive addresses of C[t, :].  With interleaved gate/up weight rows (SwiGLU,
// splits == 1) lanes r and r + 8 of every 16 hold gate and up of one output column.
constexpr int TCS_W_BYTES = 128 * TC_BK * 2;   // 16 KiB

// For the test of the give-up paths only (imp_gemm_tc_test_hooks), handed to gemm_tc_swap_kernel with its parameters:
// the poll limit of its waits, and the K block whose stage the producer leaves unfilled, so that the waits behind it
// cannot succeed.  TC_WAIT_LIMIT and -1 in every other run.
static uint32_t g_tcs_wait_limit = TC_WAIT_LIMIT;
static int g_tcs_skip_kb = -1;

// Ring depth.  Up to 32 tokens: five stages of 20 KiB; up to 64: four of 24 KiB; more: three of 32 KiB; all so that
// two CTAs share an SM (and its memory pipes).  (Five stages measured 0.7 % faster than four on the whole decode step
// at 8 to 32 rows; six would leave room for one CTA only.  At 65 to 128 tokens six stages and one CTA an SM put gate/up
// of the 8B shape in two waves of 128-row tiles: 64 to 73 us; three stages and 256 resident tiles of 96 rows: 45 to 51,
// whole decode steps at batch 128 10.47 -> 9.95 ms.  The same product on CTA pairs (cta_group::2, each CTA loading
// half of the activation tile) gained nothing beyond that, and with two CTAs an SM its paired tensor-memory
// allocations, each holding its SM's permit while waiting for its partner, hung a step once: it was taken out.)
#ifndef IMP_TCS_STAGES32
#define IMP_TCS_STAGES32 5
#endif
#ifndef IMP_TCS_STAGES128
#define IMP_TCS_STAGES128 3
#endif
template <int BN> constexpr int tcs_stages() { return BN <= 32 ? IMP_TCS_STAGES32 : (BN <= 64 ? 4 : IMP_TCS_STAGES128); }
template <int BN> constexpr int tcs_stage_bytes() { return TCS_W_BYTES + BN * TC_BK * 2; }
template <int BN> constexpr int tcs_smem_bytes() { return tcs_stages<BN>() * tcs_stage_bytes<BN>() + 1024 + 256; }
// WROWS < 128: the kernel is built for tiles of that many weight rows, whose stages are smaller, so that the same
// 100 KiB hold more of them (96 rows and 64 tokens: five stages of 20 KiB instead of four of 24).  A stage still spans
// the 16 KiB that the MMA reads from its start.
template <int BN, int WROWS> constexpr int tcs_rows_stage_bytes() { return WROWS * TC_BK * 2 + BN * TC_BK * 2; }
template <int BN, int WROWS> constexpr int tcs_rows_stages() {
    return WROWS == 128 ? tcs_stages<BN>() : (100 * 1024 / tcs_rows_stage_bytes<BN, WROWS>() < 8 ? 100 * 1024 / tcs_rows_stage_bytes<BN, WROWS>() : 8);
}
template <int BN, int WROWS> constexpr int tcs_rows_smem_bytes() { return tcs_rows_stages<BN, WROWS>() * tcs_rows_stage_bytes<BN, WROWS>() + 1024 + 256; }

// EPI: 0 = bfloat16 C[M,N], 1 = float32 C[M,N] (also the split partials), 2 = SwiGLU bfloat16 C[M,N/2]
template <int BN, int EPI, int WROWS = 128>
__global__ void __launch_bounds__(128, 1) gemm_tc_swap_kernel(const __grid_constant__ CUtensorMap map_w,
                                                              const __grid_constant__ CUtensorMap map_x, void* __restrict__ Cv,
                                                              int64_t ldc, int64_t split_stride, int M, int N, int K,
                                                              int kb_per_split, int tile_rows, int* status,
                                                              uint32_t wait_limit, int skip_kb) {
    constexpr int TCS_STAGES = tcs_rows_stages<BN, WROWS>();
    static_assert(tcs_rows_stage_bytes<BN, WROWS>() >= TCS_W_BYTES && tcs_rows_stage_bytes<BN, WROWS>() % 1024 == 0, "a stage spans what the MMA reads");
    IMP_TL_BEGIN(10 + EPI)
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int STAGE = tcs_rows_stage_bytes<BN, WROWS>();
    constexpr int W_BYTES = WROWS * TC_BK * 2;      // where the activation tile starts in a stage
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TCS_STAGES * STAGE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TCS_STAGES + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // A CTA owns tile_rows (<= 128, a multiple of 16) weight rows: map_w's box has that many rows, the MMA still
    // spans 128 and works on whatever the stage holds beyond them; those accumulator lanes are never stored.
    const int n0 = blockIdx.x * tile_rows;
    const uint32_t stage_tx = (uint32_t)(tile_rows + BN) * (TC_BK * 2);   // bytes the two boxes of a stage bring
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    const int kb_lo = blockIdx.z * kb_per_split;
    const int kb_hi = min(total_kb, kb_lo + kb_per_split);
    const int k_blocks = max(kb_hi - kb_lo, 0);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + TCS_STAGES), accum_bar = smem_u32(bars + 2 * TCS_STAGES);

    // Nothing before pdl_wait() reads or writes what an earlier kernel of the stream may still be
    // working on: barriers, tensor memory and the weight tiles of the first stages only.
    if (threadIdx.x == 0) {
        for (int s = 0; s < TCS_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        int issued = 0;
        bool ok = true;
        // the weights of the first stages do not depend on the kernel before this one
        const int early = k_blocks < TCS_STAGES ? k_blocks : TCS_STAGES;
        for (int i = 0; i < early; ++i) {
            mbar_expect_tx(full0 + 8 * i, stage_tx);
            tma_load_2d(smem_u32(tiles + i * STAGE), &map_w, (kb_lo + i) * TC_BK, n0, full0 + 8 * i);
        }
        pdl_wait();
        IMP_TL_WAITED()
        for (int i = 0; i < early; ++i)
            tma_load_2d(smem_u32(tiles + i * STAGE) + W_BYTES, &map_x, (kb_lo + i) * TC_BK, 0, full0 + 8 * i);
        issued = early;
        for (int i = early; i < k_blocks; ++i) {
            const int s = i % TCS_STAGES;
            ok = mbar_wait(empty0 + 8 * s, ((uint32_t)(i / TCS_STAGES) & 1u) ^ 1u, status, wait_limit);
            if (!ok) break;
            if (i == skip_kb) { issued = i + 1; continue; }
            const uint32_t w_dst = smem_u32(tiles + s * STAGE), x_dst = w_dst + W_BYTES;
            mbar_expect_tx(full0 + 8 * s, stage_tx);
            tma_load_2d(w_dst, &map_w, (kb_lo + i) * TC_BK, n0, full0 + 8 * s);
            tma_load_2d(x_dst, &map_x, (kb_lo + i) * TC_BK, 0, full0 + 8 * s);
            issued = i + 1;
        }
        if (!ok)
            for (int i = issued > TCS_STAGES ? issued - TCS_STAGES : 0; i < issued; ++i)
                mbar_wait(full0 + 8 * (i % TCS_STAGES), (uint32_t)(i / TCS_STAGES) & 1u, nullptr, wait_limit);
    } else {
        pdl_wait();
    }
    if (warp == 1 && lane == 0) {
        const uint32_t idesc = tc_instr_desc(128, BN);
        bool ok = true;
        for (int i = 0; i < k_blocks && ok; ++i) {
            const int s = i % TCS_STAGES;
            ok = mbar_wait(full0 + 8 * s, (uint32_t)(i / TCS_STAGES) & 1u, status, wait_limit);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t w_addr = smem_u32(tiles + s * STAGE), x_addr = w_addr + W_BYTES;
#pragma unroll
            for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)
                tc_mma(tmem_base, tc_smem_desc(w_addr + k * TC_UMMA_K * 2), tc_smem_desc(x_addr + k * TC_UMMA_K * 2), idesc,
                       (i > 0 || k > 0) ? 1u : 0u);
            tc_commit(empty0 + 8 * s);
        }
        tc_commit(accum_bar);
    }
    __syncwarp();

    const bool acc_ok = __all_sync(0xffffffffu, mbar_wait(accum_bar, 0, status, wait_limit));
    tc_fence_after_sync();
    if (acc_ok) {
        const int r = warp * 32 + lane;             // accumulator lane = weight row of the tile
        const int col = n0 + r;                     // output column
        const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            float v[32];
            if (k_blocks > 0) {
                tc_ld32(lane_base + (uint32_t)(c * 32), v);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0.f;   // an empty K range contributes nothing
            }
            if (EPI == TC_OUT_SWIGLU_BF16) {
                __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(Cv);
                const bool is_gate = (r & 8) == 0;
                const int ocol = (col >> 4) * 8 + (r & 7);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float up = __shfl_xor_sync(0xffffffffu, v[i], 8);   // lane r + 8 holds the matching up row
                    const int tok = c * 32 + i;
                    if (is_gate && tok < M && col + 8 < N && r < tile_rows)
                        base[(int64_t)tok * ldc + ocol] = __float2bfloat16_rn(v[i] / (1.f + expf(-v[i])) * up);
                }
            } else if (col < N && r < tile_rows) {
                if (EPI == TC_OUT_F32) {
                    float* base = reinterpret_cast<float*>(Cv) + (int64_t)blockIdx.z * split_stride;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int tok = c * 32 + i;
                        if (tok < M) base[(int64_t)tok * ldc + col] = v[i];
                    }
                } else {
                    __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(Cv);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int tok = c * 32 + i;
                        if (tok < M) base[(int64_t)tok * ldc + col] = __float2bfloat16_rn(v[i]);
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
    IMP_TL_END()
}

// out[m, n] = sum over splits of part[s, m, n], in split order.
template <typename TO>
__global__ void gemm_tc_reduce_kernel(TO* __restrict__ out, int64_t ldc, const float* __restrict__ part, int64_t split_stride,
                                      int M, int N, int splits) {
    IMP_TL_BEGIN(2)
    pdl_wait();
    IMP_TL_WAITED()
    pdl_launch_dependents();
    const int64_t total = (int64_t)M * N;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / N;
        const int n = (int)(i - m * N);
        float acc = 0.f;
        for (int s0 = 0; s0 < splits; s0 += 8) {      // eight parts requested together, added in split order
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < splits) v[j] = part[(s0 + j) * split_stride + i];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < splits) acc += v[j];
        }
        out[m * ldc + n] = from_float<TO>(acc);
    }
    IMP_TL_END()
}

// The same sums (each element in split order) four columns at a time, for the partial products of many rows.
template <typename TO>
__global__ void gemm_tc_reduce4_kernel(TO* __restrict__ out, int64_t ldc, const float* __restrict__ part, int64_t split_stride,
                                       int M, int N, int splits) {
    pdl_wait();
    pdl_launch_dependents();
    const int n4 = N >> 2;
    const int64_t total = (int64_t)M * n4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / n4;
        const int n = (int)(i - m * n4) << 2;
        const float* src = part + m * N + n;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < splits; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(src + s * split_stride);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        TO* dst = out + m * ldc + n;
        if constexpr (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(dst) = acc;
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&lo);
            o.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst) = o;
        }
    }
}

// ------------------------------------------------------------------------------------- host
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
static int launch_tc(void* C, int64_t ldc, const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mw128, int M,
                     int N, int K, int* status, cudaStream_t s) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (e != cudaSuccess) { imp_set_error("gemm_tc: %s", cudaGetErrorString(e)); return (int)e; }
        attr_set = true;
    }
    static int mode = -1, sms = 0;   // IMP_B200_TC_SIMPLE=1 selects the one-tile-per-CTA kernel
    if (mode < 0) {
        mode = getenv("IMP_B200_TC_SIMPLE") ? 1 : 0;
        sms = imp_sm_count();
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (e != cudaSuccess) { imp_set_error("gemm_tc: %s", cudaGetErrorString(e)); mode = -1; return (int)e; }
    }
    // IMP_B200_TC_PAIR=0 keeps single CTAs; by default products of 256 rows and more run on CTA pairs.
    static int pair_mode = -1;
    if (pair_mode < 0) {
        const char* e = getenv("IMP_B200_TC_PAIR");
        pair_mode = e ? atoi(e) : 1;
        if (pair_mode) {
            cudaError_t e2 = cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC2_SMEM_BYTES);
            if (e2 != cudaSuccess) { imp_set_error("gemm_tc: %s", cudaGetErrorString(e2)); pair_mode = -1; return (int)e2; }
        }
    }
    static int pair_min_rows = -1;   // IMP_B200_TC_PAIR_ROWS: rows from which CTA pairs take the product (default 129)
    if (pair_min_rows < 0) { const char* e = getenv("IMP_B200_TC_PAIR_ROWS"); pair_min_rows = e ? atoi(e) : 129; }
    if (mode == 0 && pair_mode == 1 && M >= pair_min_rows) {
        const int tiles2 = ((M + TC2_BM - 1) / TC2_BM) * ((N + TC2_BN - 1) / TC2_BN);
        const int pairs = tiles2 < sms / 2 ? tiles2 : sms / 2;
        // bfloat16 outputs leave through TMA stores where C's rows allow them (16-byte strides)
        static int tma_out = -1;       // IMP_B200_TC_TMA_STORE=0: every thread stores its own row
        if (tma_out < 0) { const char* e = getenv("IMP_B200_TC_TMA_STORE"); tma_out = e ? atoi(e) : 1; }
        CUtensorMap mc{};
        int tma_store = 0;
        if (EPI != TC_OUT_F32 && tma_out && ldc % 8 == 0)
            tma_store = make_map(&mc, C, M, EPI == TC_OUT_SWIGLU_BF16 ? N / 2 : N, ldc, 128) == 0 ? 1 : 0;
        cudaError_t e = imp_launch(gemm_tc_pair_kernel<EPI>, dim3(2 * pairs), dim3(TCP_THREADS), (size_t)TC2_SMEM_BYTES, s, ma, mw128,
                                   C, ldc, M, N, K, status, QkvRopeArgs{}, 1, (K + TC_BK - 1) / TC_BK, (int64_t)0, mc, tma_store);
        if (e != cudaSuccess) { imp_set_error("gemm_tc: %s", cudaGetErrorString(e)); return (int)e; }
        return 0;
    }
    const int num_m = (M + TC_BM - 1) / TC_BM, num_n = (N + TC_BN - 1) / TC_BN;
    if (mode == 1) {
        gemm_tc_kernel<EPI><<<dim3(num_m, num_n), 128, TC_SMEM_BYTES, s>>>(ma, mw, C, ldc, M, N, K, status);
    } else {
        const int total = num_m * num_n;
        cudaError_t e = imp_launch(gemm_tc_persistent_kernel<EPI>, dim3(total < sms ? total : sms), dim3(TCP_THREADS),
                                   (size_t)TC_SMEM_BYTES, s, ma, mw, C, ldc, M, N, K, status);
        if (e != cudaSuccess) { imp_set_error("gemm_tc: %s", cudaGetErrorString(e)); return (int)e; }
        return 0;
    }
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
    CUtensorMap mw128;   // the W tile in halves of 128 rows, for CTA pairs
    if (int rc = make_map(&mw128, W, N, K, ldw, 128)) return rc;
    if (epilogue == TC_OUT_BF16) return launch_tc<TC_OUT_BF16>(C, ldc, ma, mw, mw128, M, N, K, status, s);
    if (epilogue == TC_OUT_F32) return launch_tc<TC_OUT_F32>(C, ldc, ma, mw, mw128, M, N, K, status, s);
    return launch_tc<TC_OUT_SWIGLU_BF16>(C, ldc, ma, mw, mw128, M, N, K, status, s);
}

// ---- many rows, few tiles: the K range in parts ------------------------------------------------------
// A portion of a prompt (256 to about a thousand rows) times a weight of a few thousand rows makes fewer 256 x 256
// tiles than the device has CTA pairs (512 x 4096: 32 tiles on 74 pairs).  Then the K range is cut so that
// tiles x parts fills the pairs, each part leaves a 32-bit partial product, and gemm_tc_reduce_kernel adds them in order.
#ifndef TC2_MIN_KB_PER_SPLIT
#define TC2_MIN_KB_PER_SPLIT 48    // blocks of K (3072 elements) a part has at least: a launch of the pair kernel costs about
#endif                             // 12 us before and after its MMAs, so parts of a short K gain less than their sum costs
#ifndef TC2_MAX_SPLITS
#define TC2_MAX_SPLITS 4
#endif
#ifndef TC2_SPLIT_MIN_ROWS
#define TC2_SPLIT_MIN_ROWS 129     // from where CTA pairs take the product (decode at 160 sequences: 12.87 -> 11.76 ms a step
#endif                             // once the down projection's 16 tiles are cut in four)
IMP_API int imp_gemm_bf16_tc_splits(int M, int N, int K) {
    static int enabled = -1;       // IMP_B200_TC_SPLIT=0: never
    if (enabled < 0) { const char* e = getenv("IMP_B200_TC_SPLIT"); enabled = e ? atoi(e) : 1; }
    const char* pair_env = getenv("IMP_B200_TC_PAIR");
    if (!enabled || M < TC2_SPLIT_MIN_ROWS || getenv("IMP_B200_TC_SIMPLE") || (pair_env && atoi(pair_env) == 0)) return 1;
    const int tiles2 = ((M + TC2_BM - 1) / TC2_BM) * ((N + TC2_BN - 1) / TC2_BN);
    const int pairs = imp_sm_count() / 2;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    int splits = pairs / (tiles2 > 0 ? tiles2 : 1);
    if (splits > k_blocks / TC2_MIN_KB_PER_SPLIT) splits = k_blocks / TC2_MIN_KB_PER_SPLIT;
    if (splits > TC2_MAX_SPLITS) splits = TC2_MAX_SPLITS;
    return splits < 1 ? 1 : splits;
}

// scratch[s][M, N] (32-bit, M * N floats apart) for s < imp_gemm_bf16_tc_splits(M, N, K): the parts of A W^T.
IMP_API int imp_gemm_bf16_tc_partials(float* scratch, const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N,
                                      int K, int* status, void* stream) {
    IMP_CHECK_ARG(scratch && A && W && M > 0 && N > 0 && K > 0 && lda >= K && ldw >= K, "imp_gemm_bf16_tc_partials: bad argument");
    const int splits = imp_gemm_bf16_tc_splits(M, N, K);
    if (splits < 2) return IMP_ERR_UNSUPPORTED;
    if (K % 8 || lda % 8 || ldw % 8 || N % 4 || (uintptr_t)A % 16 || (uintptr_t)W % 16 || (uintptr_t)scratch % 16) return IMP_ERR_UNSUPPORTED;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<TC_OUT_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC2_SMEM_BYTES);
        if (e != cudaSuccess) { imp_set_error("imp_gemm_bf16_tc_partials: %s", cudaGetErrorString(e)); return (int)e; }
        attr_set = true;
    }
    CUtensorMap ma, mw128;
    if (int rc = make_map(&ma, A, M, K, lda, TC_BM)) return rc;
    if (int rc = make_map(&mw128, W, N, K, ldw, 128)) return rc;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const int kb_per_split = (k_blocks + splits - 1) / splits;
    const int units = ((M + TC2_BM - 1) / TC2_BM) * ((N + TC2_BN - 1) / TC2_BN) * splits;
    const int sms = imp_sm_count();
    const int pairs = units < sms / 2 ? units : sms / 2;
    cudaError_t e = imp_launch(gemm_tc_pair_kernel<TC_OUT_F32>, dim3(2 * pairs), dim3(TCP_THREADS), (size_t)TC2_SMEM_BYTES,
                               (cudaStream_t)stream, ma, mw128, (void*)scratch, (int64_t)N, M, N, K, status, QkvRopeArgs{}, splits,
                               kb_per_split, (int64_t)M * N, CUtensorMap{}, 0);
    if (e != cudaSuccess) { imp_set_error("imp_gemm_bf16_tc_partials: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}

// ---- few rows (M <= 128) ----------------------------------------------------------------------------
// Number of K splits imp_gemm_bf16_tc_swap will use, and the floats of scratch it then needs.
#ifndef TCS_MIN_KB_PER_SPLIT
#define TCS_MIN_KB_PER_SPLIT 6     // blocks of K a split has at least
#endif
static int tcs_sms() { return imp_sm_count(); }
// CTAs resident at once: two an SM (the 128-token variant by its three stages of 32 KiB).
static int tcs_slots(int M) { (void)M; return 2 * tcs_sms(); }

// Weight rows of a CTA's tile when K is not split.  All CTAs are resident at once (two per SM up to 64 tokens),
// handed out round robin, so the SM with the most CTAs sets the time: 192 tiles of 128 rows put two tiles on 44 SMs
// and one on the others (256 rows at most per SM), 256 tiles of 96 rows put 192 at most.  Smaller tiles are
// taken while they lower that maximum; more CTAs than slots are left alone (several waves even out by themselves).
static int tcs_tile_rows(int M, int N, int splits) {
    static int fixed = -1;             // IMP_B200_TCS_ROWS=128 (or another multiple of 16): no choice
    if (fixed < 0) { const char* e = getenv("IMP_B200_TCS_ROWS"); fixed = e ? atoi(e) : 0; }
    if (fixed >= 16 && fixed <= 128 && fixed % 16 == 0) return fixed;
    if (splits > 1) return 128;
    const int sms = tcs_sms();
    const int slots = tcs_slots(M);
    int best = 128, best_load = -1;
    for (int rows = 128; rows >= 64; rows -= 16) {
        const int ctas = (N + rows - 1) / rows;
        if (ctas > slots) { if (rows == 128) return 128; break; }
        const int load = ((ctas + sms - 1) / sms) * rows;     // rows the busiest SM streams
        if (best_load < 0 || load < best_load) { best = rows; best_load = load; }
    }
    return best;
}

static int tcs_splits(int M, int N, int K, int epilogue) {
    if (epilogue == TC_OUT_SWIGLU_BF16) return 1;
    const int slots = tcs_slots(M);                      // resident CTAs
    const int tiles = (N + 127) / 128;
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    int splits = slots / tiles;                          // as many CTAs as fit in one wave
    const int max_splits = total_kb / TCS_MIN_KB_PER_SPLIT > 0 ? total_kb / TCS_MIN_KB_PER_SPLIT : 1;
    if (splits > max_splits) splits = max_splits;
    if (splits > 16) splits = 16;
    return splits < 1 ? 1 : splits;
}

IMP_API int64_t imp_gemm_bf16_tc_swap_scratch_floats(int M, int N, int K, int epilogue) {
    const int splits = tcs_splits(M, N, K, epilogue);
    return splits > 1 ? (int64_t)splits * M * N : 0;
}

template <int BN, int EPI, int WROWS = 128>
static int launch_tcs(void* C, int64_t ldc, int64_t split_stride, const CUtensorMap& mw, const CUtensorMap& mx, int M, int N,
                      int K, int splits, int kb_per_split, int tile_rows, int* status, cudaStream_t s) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_swap_kernel<BN, EPI, WROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             tcs_rows_smem_bytes<BN, WROWS>());
        if (e != cudaSuccess) { imp_set_error("gemm_tc_swap: %s", cudaGetErrorString(e)); return (int)e; }
        attr_set = true;
    }
    dim3 grid((N + tile_rows - 1) / tile_rows, 1, splits);
    cudaError_t e = imp_launch(gemm_tc_swap_kernel<BN, EPI, WROWS>, grid, dim3(128), (size_t)tcs_rows_smem_bytes<BN, WROWS>(), s, mw, mx,
                               C, ldc, split_stride, M, N, K, kb_per_split, tile_rows, status, g_tcs_wait_limit, g_tcs_skip_kb);
    if (e != cudaSuccess) { imp_set_error("gemm_tc_swap: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}

// C = A[M,K] * W[N,K]^T for 1 <= M <= 128 with the weights on the M side of the MMA.
// epilogue as for imp_gemm_bf16_tc.  `scratch` must hold imp_gemm_bf16_tc_swap_scratch_floats() floats.
static int gemm_bf16_tc_swap_impl(void* C, int64_t ldc, int epilogue, const void* A, int64_t lda, const void* W, int64_t ldw,
                                  int M, int N, int K, float* scratch, int* status, void* stream, bool partials_only) {
    if (M == 0 || N == 0) return 0;
    IMP_CHECK_ARG((C || partials_only) && A && W && M > 0 && N > 0 && K > 0, "imp_gemm_bf16_tc_swap: bad argument");
    IMP_CHECK_ARG(M <= 128, "imp_gemm_bf16_tc_swap: M %d exceeds 128", M);
    IMP_CHECK_ARG(epilogue >= 0 && epilogue <= 2, "imp_gemm_bf16_tc_swap: unknown epilogue %d", epilogue);
    if (epilogue == 2) IMP_CHECK_ARG(N % 16 == 0, "imp_gemm_bf16_tc_swap: %d interleaved rows are not a multiple of 16", N);
    IMP_CHECK_ARG(lda >= K && ldw >= K && ldc >= (epilogue == 2 ? N / 2 : N), "imp_gemm_bf16_tc_swap: leading dimension too small");
    if (K % 8 || lda % 8 || ldw % 8 || (uintptr_t)A % 16 || (uintptr_t)W % 16) return IMP_ERR_UNSUPPORTED;
    const int splits = tcs_splits(M, N, K, epilogue);
    IMP_CHECK_ARG(splits == 1 || scratch, "imp_gemm_bf16_tc_swap: %d splits of K need scratch memory", splits);
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    const int kb_per_split = (total_kb + splits - 1) / splits;
    static int bn32 = -1;                     // IMP_B200_TCS_BN32=0 keeps 64 columns for up to 32 rows (measurements)
    if (bn32 < 0) { const char* e = getenv("IMP_B200_TCS_BN32"); bn32 = e ? atoi(e) : 1; }
    const int BN = (M <= 32 && bn32) ? 32 : (M <= 64 ? 64 : 128);
    const int tile_rows = tcs_tile_rows(M, N, splits);
    CUtensorMap mw, mx;
    if (int rc = make_map(&mw, W, N, K, ldw, tile_rows)) return rc;
    if (int rc = make_map(&mx, A, M, K, lda, BN)) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    int rc = 0;
    if (splits > 1) {
        const int64_t split_stride = (int64_t)M * N;
        rc = BN == 32 ? launch_tcs<32, TC_OUT_F32>(scratch, N, split_stride, mw, mx, M, N, K, splits, kb_per_split, tile_rows, status, s)
           : BN == 64 ? launch_tcs<64, TC_OUT_F32>(scratch, N, split_stride, mw, mx, M, N, K, splits, kb_per_split, tile_rows, status, s)
                      : launch_tcs<128, TC_OUT_F32>(scratch, N, split_stride, mw, mx, M, N, K, splits, kb_per_split, tile_rows, status, s);
        if (rc) return rc;
        if (partials_only) IMP_RETURN_LAUNCH();
        const int64_t total = (int64_t)M * N;
        const int64_t cap = (int64_t)imp_sm_count() * 8;
        const int grid = (int)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
        cudaError_t e;
        if (epilogue == TC_OUT_F32)
            e = imp_launch(gemm_tc_reduce_kernel<float>, dim3(grid), dim3(256), 0, s, (float*)C, ldc, (const float*)scratch,
                           split_stride, M, N, splits);
        else
            e = imp_launch(gemm_tc_reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, (__nv_bfloat16*)C, ldc,
                           (const float*)scratch, split_stride, M, N, splits);
        if (e != cudaSuccess) { imp_set_error("gemm_tc_swap: %s", cudaGetErrorString(e)); return (int)e; }
    } else if (epilogue == TC_OUT_BF16) {
        rc = BN == 32 ? launch_tcs<32, TC_OUT_BF16>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s)
           : BN == 64 ? launch_tcs<64, TC_OUT_BF16>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s)
                      : launch_tcs<128, TC_OUT_BF16>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s);
    } else if (epilogue == TC_OUT_F32) {
        rc = BN == 32 ? launch_tcs<32, TC_OUT_F32>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s)
           : BN == 64 ? launch_tcs<64, TC_OUT_F32>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s)
                      : launch_tcs<128, TC_OUT_F32>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s);
    } else {
        static int rows96 = -1;        // IMP_B200_TCS_ROWS96: bit 0 the 64-token variant, bit 1 the 32-token one
        if (rows96 < 0) { const char* e = getenv("IMP_B200_TCS_ROWS96"); rows96 = e ? atoi(e) : 3; }
        // gate/up of the 8B shape (256 tiles of 96 rows): 42.3 -> 40.5 us at 64 tokens with five stages instead of four,
        // 34.8 -> 34.7 at 8 tokens with six instead of five; whole steps 0.2 to 0.5 % faster
        rc = (BN == 64 && tile_rows == 96 && (rows96 & 1))
                 ? launch_tcs<64, TC_OUT_SWIGLU_BF16, 96>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s)
           : (BN == 32 && tile_rows == 96 && (rows96 & 2))
                 ? launch_tcs<32, TC_OUT_SWIGLU_BF16, 96>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s)
           : BN == 32 ? launch_tcs<32, TC_OUT_SWIGLU_BF16>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s)
           : BN == 64 ? launch_tcs<64, TC_OUT_SWIGLU_BF16>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s)
                      : launch_tcs<128, TC_OUT_SWIGLU_BF16>(C, ldc, 0, mw, mx, M, N, K, 1, kb_per_split, tile_rows, status, s);
    }
    if (rc) return rc;
    IMP_RETURN_LAUNCH();
}

// Test hooks of the bounded waits.  `wait_limit` polls (0: the regular limit) bound every mbarrier wait of the
// few-rows kernel from its next launch on, and its producer leaves the stage of K block `skip_kb` unfilled (-1:
// none; blocks inside the first ring depth are never skipped), so that the MMA thread's wait for it, the producer's
// later wait for the slot and its wait for its own copies all run out.  The kernel then reports IMP_WAIT_TIMEOUT
// through the status word, frees its tensor memory and returns.  A test lowers the limit to a few thousand polls for
// one CTA and restores both values afterwards.  (Both travel as kernel parameters.)
IMP_API int imp_gemm_tc_test_hooks(unsigned wait_limit, int skip_kb) {
    g_tcs_wait_limit = wait_limit ? wait_limit : TC_WAIT_LIMIT;
    g_tcs_skip_kb = skip_kb;
    return 0;
}

IMP_API int imp_gemm_bf16_tc_swap(void* C, int64_t ldc, int epilogue, const void* A, int64_t lda, const void* W, int64_t ldw,
                                  int M, int N, int K, float* scratch, int* status, void* stream) {
    return gemm_bf16_tc_swap_impl(C, ldc, epilogue, A, lda, W, ldw, M, N, K, scratch, status, stream, false);
}

// How many partial results imp_gemm_bf16_tc_swap_partials leaves for this shape (1: it does not split, call the
// plain entry point instead).
IMP_API int imp_gemm_bf16_tc_swap_splits(int M, int N, int K) { return tcs_splits(M, N, K, TC_OUT_F32); }

// The product left unsummed: scratch[s][M, N] (32-bit, M * N floats apart) for s < imp_gemm_bf16_tc_swap_splits()
// holds the part of A W^T that split s of the contraction contributes.  Whoever reads the result next adds the
// parts in split order (the norm and rotary kernels have entry points that do), which saves the summing kernel.
IMP_API int imp_gemm_bf16_tc_swap_partials(float* scratch, const void* A, int64_t lda, const void* W, int64_t ldw, int M,
                                           int N, int K, int* status, void* stream) {
    IMP_CHECK_ARG(scratch, "imp_gemm_bf16_tc_swap_partials: no scratch memory");
    if (tcs_splits(M, N, K, TC_OUT_F32) < 2) return IMP_ERR_UNSUPPORTED;
    return gemm_bf16_tc_swap_impl(nullptr, N, TC_OUT_F32, A, lda, W, ldw, M, N, K, scratch, status, stream, true);
}

// C[M, N] (bfloat16 or float32, by `epilogue`) = the sum of the partial results, in split order.
IMP_API int imp_gemm_bf16_tc_swap_sum(void* C, int64_t ldc, int epilogue, const float* scratch, int M, int N, int splits,
                                      void* stream) {
    if (M == 0 || N == 0) return 0;
    IMP_CHECK_ARG(C && scratch && splits >= 1 && ldc >= N && (epilogue == TC_OUT_BF16 || epilogue == TC_OUT_F32),
                  "imp_gemm_bf16_tc_swap_sum: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t total = (int64_t)M * N;
    const int64_t cap = (int64_t)imp_sm_count() * 8;
    cudaError_t e;
    if (M > 128 && N % 4 == 0 && ldc % 4 == 0 && (uintptr_t)C % 16 == 0 && (uintptr_t)scratch % 16 == 0) {
        // many rows (the parts of a portion's product): four columns a thread
        const int64_t work = total / 4;
        const int grid = (int)((work + 255) / 256 < cap ? (work + 255) / 256 : cap);
        if (epilogue == TC_OUT_F32)
            e = imp_launch(gemm_tc_reduce4_kernel<float>, dim3(grid), dim3(256), 0, s, (float*)C, ldc, scratch, total, M, N, splits);
        else
            e = imp_launch(gemm_tc_reduce4_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, (__nv_bfloat16*)C, ldc, scratch,
                           total, M, N, splits);
    } else {
        const int grid = (int)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
        if (epilogue == TC_OUT_F32)
            e = imp_launch(gemm_tc_reduce_kernel<float>, dim3(grid), dim3(256), 0, s, (float*)C, ldc, scratch, total, M, N, splits);
        else
            e = imp_launch(gemm_tc_reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, (__nv_bfloat16*)C, ldc, scratch,
                           total, M, N, splits);
    }
    if (e != cudaSuccess) { imp_set_error("gemm_tc_swap_sum: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}

// q, k, v = A W^T with the per-head norm, the rotation and the cache write done in the product's epilogue
// (see QkvRopeArgs): A [M, K], W [(Hq + 2 Hkv) * Dh, K] with q heads first, then k, then v.  Needs at least
// 256 rows, head size 64 or 128 rotated over its whole width, CTA pairs enabled; returns IMP_ERR_UNSUPPORTED
// otherwise (the caller then runs the product and the rotary kernel one after the other).
IMP_API int imp_gemm_bf16_tc_qkv_rope(const void* A, int64_t lda, const void* W, int64_t ldw, int M, int K, int Hq, int Hkv,
                                      int Dh, const float* q_norm_w, const float* k_norm_w, float eps, const float* cos_tab,
                                      const float* sin_tab, int max_pos, const int* positions, const int* seq_of_token,
                                      const int* block_table, int bt_stride, int n_seqs, void* q_out, int64_t q_stride,
                                      void* k_cache, void* v_cache, int page_size, int num_pages, int* status, void* stream) {
    if (M == 0) return 0;
    IMP_CHECK_ARG(A && W && M > 0 && K > 0 && Hq > 0 && Hkv > 0, "imp_gemm_bf16_tc_qkv_rope: bad argument");
    IMP_CHECK_ARG(cos_tab && sin_tab && positions && seq_of_token && block_table && q_out && k_cache && v_cache,
                  "imp_gemm_bf16_tc_qkv_rope: null pointer");
    IMP_CHECK_ARG((q_norm_w == nullptr) == (k_norm_w == nullptr), "imp_gemm_bf16_tc_qkv_rope: q and k norm weights must both be set or both be null");
    IMP_CHECK_ARG(lda >= K && ldw >= K && q_stride >= (int64_t)Hq * Dh && page_size > 0 && num_pages > 0 && max_pos > 0,
                  "imp_gemm_bf16_tc_qkv_rope: bad geometry");
    const int N = (Hq + 2 * Hkv) * Dh;
    if (M < 256 || (Dh != 64 && Dh != 128)) return IMP_ERR_UNSUPPORTED;
    if (K % 8 || lda % 8 || ldw % 8 || q_stride % 8 || (uintptr_t)A % 16 || (uintptr_t)W % 16 || (uintptr_t)q_out % 16 ||
        (uintptr_t)k_cache % 16 || (uintptr_t)v_cache % 16)
        return IMP_ERR_UNSUPPORTED;
    static int ready = -1, sms = 2;
    if (ready < 0) {
        const char* e = getenv("IMP_B200_TC_PAIR");
        ready = (e == nullptr || atoi(e) != 0) && getenv("IMP_B200_TC_SIMPLE") == nullptr ? 1 : 0;
        if (ready) {
            sms = imp_sm_count() < 2 ? 2 : imp_sm_count();
            cudaError_t e2 = cudaFuncSetAttribute(gemm_tc_pair_kernel<TC_OUT_QKV_ROPE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  TC2_SMEM_BYTES);
            if (e2 != cudaSuccess) { imp_set_error("imp_gemm_bf16_tc_qkv_rope: %s", cudaGetErrorString(e2)); ready = -1; return (int)e2; }
        }
    }
    if (!ready) return IMP_ERR_UNSUPPORTED;
    CUtensorMap ma, mw128;
    if (int rc = make_map(&ma, A, M, K, lda, TC_BM)) return rc;
    if (int rc = make_map(&mw128, W, N, K, ldw, 128)) return rc;
    QkvRopeArgs a;
    a.positions = positions; a.seq_of_token = seq_of_token; a.block_table = block_table;
    a.cos_tab = cos_tab; a.sin_tab = sin_tab; a.q_norm_w = q_norm_w; a.k_norm_w = k_norm_w;
    a.q_out = (__nv_bfloat16*)q_out; a.k_cache = (__nv_bfloat16*)k_cache; a.v_cache = (__nv_bfloat16*)v_cache;
    a.q_stride = q_stride; a.eps = eps; a.bt_stride = bt_stride; a.n_seqs = n_seqs; a.max_pos = max_pos;
    a.Hq = Hq; a.Hkv = Hkv; a.Dh = Dh; a.page_size = page_size; a.num_pages = num_pages;
    const int tiles2 = ((M + TC2_BM - 1) / TC2_BM) * ((N + TC2_BN - 1) / TC2_BN);
    const int pairs = tiles2 < sms / 2 ? tiles2 : sms / 2;
    // q leaves through TMA stores (k and v go to their pages row by row)
    CUtensorMap mq{};
    int q_tma = 0;
    {
        const char* env = getenv("IMP_B200_TC_TMA_STORE");
        const char* env_q = getenv("IMP_B200_TC_TMA_Q");
        if (!(env && atoi(env) == 0) && !(env_q && atoi(env_q) == 0) && q_stride % 8 == 0)
            q_tma = make_map(&mq, q_out, M, Hq * Dh, q_stride, 128) == 0 ? 1 : 0;
    }
    cudaError_t e = imp_launch(gemm_tc_pair_kernel<TC_OUT_QKV_ROPE>, dim3(2 * pairs), dim3(TCP_THREADS), (size_t)TC2_SMEM_BYTES,
                               (cudaStream_t)stream, ma, mw128, (void*)nullptr, (int64_t)0, M, N, K, status, a, 1,
                               (K + TC_BK - 1) / TC_BK, (int64_t)0, mq, q_tma);
    if (e != cudaSuccess) { imp_set_error("imp_gemm_bf16_tc_qkv_rope: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}
