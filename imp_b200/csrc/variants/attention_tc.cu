// Paged prefill attention on the fifth-generation tensor cores (tcgen05 + tensor memory), bfloat16,
// compiled once per head size: -DIMP_ATTN_DH=64 or 128.
//
// A CTA owns one tile of up to 128 consecutive query tokens of one sequence and NQ (1 or 2) query
// heads that share a kv head, and walks the cached keys of the sequence in tiles of 128 from the
// window's start to the last token's position (keys come from the pages only; the new tokens'
// keys are already there).  Roles:
//   warp 0           producer.  Q tiles once, then per key tile the K pages and the V pages of the
//                    kv head with TMA (cp.async.bulk.tensor, 128-byte swizzle), one box per page
//                    and 64 head dimensions, into shared-memory rings; page ids come from the block
//                    table, pages that do not exist are fetched from beyond the tensor (zeros).
//   warp 1, lane 0   MMA issuer.  S_w = Q_w K^T (M=128 tokens, N=128 keys, K=head size) into tensor
//                    memory, and O_w += P_w V (M=128, N=head size, K=128 keys; P from tensor memory), V being read as an
//                    MN-major operand straight from its [key, dim] layout.  After P_w V of tile i
//                    it issues Q_w K^T of tile i+1, so while one head's softmax runs the tensor
//                    cores work on the other head.
//   warps 4..7 (head 0), 8..11 (head 1)   softmax.  A thread owns one query row: it reads its row of
//                    S from tensor memory, applies the causal / window mask on tiles that need it,
//                    keeps the running maximum and sum in 32-bit, writes P = exp2(s - m) as bfloat16
//                    pairs back into tensor memory over S, from where the MMA takes it as its A
//                    operand, and at the end divides its row of O by the sum and stores it.  O stays in tensor memory
//                    across key tiles; it is rescaled only when a row's maximum grew by more than
//                    2^8 since the last rescale (P then stays below 2^8, exact enough in bfloat16
//                    and 32-bit sums), the decision being taken per warp.
// Every mbarrier wait is bounded (TC_WAIT_LIMIT polls); a wait that runs out reports
// IMP_WAIT_TIMEOUT through the status word, the role leaves its loop, the producer waits (bounded)
// for its copies in flight, and the CTA frees its tensor memory and returns.
//
// Math as in the reference's prefill kernels (src/compute/attention.cu:158-216): s = scale * q.k,
// masked when key > query position or query position - key >= window, softmax with a running
// maximum, o = sum p v; query head h reads kv head h / (Hq / Hkv).
#include "../common.cuh"
#include "../tc_common.cuh"

#ifndef IMP_ATTN_DH
#error "compile with -DIMP_ATTN_DH=<head size>"
#endif

constexpr int DH = IMP_ATTN_DH;
static_assert(DH == 64 || DH == 128, "the tensor-memory prefill kernel is built for head sizes 64 and 128");

constexpr int FA_BM = 128;                       // query rows per tile (the MMA's M)
constexpr int FA_BN = 128;                       // keys per tile
constexpr int FA_KB = DH / 64;                   // 64-wide blocks of the head dimension
constexpr int FA_BLOCK_BYTES = 128 * 128;        // 128 rows of 128 bytes: one swizzled block
constexpr int FA_Q_BYTES = FA_KB * FA_BLOCK_BYTES;          // one head's Q tile
constexpr int FA_KV_BYTES = FA_KB * FA_BLOCK_BYTES;         // one K or V tile
constexpr float FA_RESCALE_STEP = 8.f;           // log2 of the growth of a row maximum that forces a rescale

template <int NQ> struct FaCfg {
    static constexpr int K_STAGES = 2;
    static constexpr int V_STAGES = 2;
    static constexpr int THREADS = 128 + 128 * NQ;        // warps 0-3: producer, MMA issuer, two idle; then 4 per head
    static constexpr int TMEM_COLS = 256 * NQ;
    static constexpr int TILE_BYTES = NQ * FA_Q_BYTES + (K_STAGES + V_STAGES) * FA_KV_BYTES;
    static constexpr int N_BARS = 1 + 2 * K_STAGES + 2 * V_STAGES + 3 * NQ;
    static constexpr int SMEM_BYTES = TILE_BYTES + 1024 /* alignment slack */ + 256 /* barriers, tmem slot */;
};

// V as the B operand of O = P V: [key, dim] rows of 128 bytes per 64-dim block, i.e. MN-major with
// the 128-byte swizzle: 8-key groups 1024 bytes apart (stride offset), 64-dim blocks one block
// apart (leading offset).
__device__ __forceinline__ uint64_t fa_v_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((uint32_t)FA_BLOCK_BYTES >> 4) << 16;   // leading byte offset
    d |= (uint64_t)(1024u >> 4) << 32;                      // stride byte offset
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// D += A B with A (bfloat16, two consecutive K elements per 32-bit column, one row per lane) in tensor memory.
__device__ __forceinline__ void fa_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ float fa_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t fa_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int NQ>
__global__ void __launch_bounds__(FaCfg<NQ>::THREADS, 1) attn_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int64_t out_stride,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ seq_of_token,
    const int* __restrict__ positions, const int* __restrict__ tile_tok0, const int* __restrict__ tile_rows, int n_tiles,
    int n_seqs, int Hq, int Hkv, int P, int num_pages, float scale_log2, int window, int* status) {
    using Cfg = FaCfg<NQ>;
    constexpr int KS = Cfg::K_STAGES, VS = Cfg::V_STAGES;
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ unsigned char fa_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = tiles;                                   // [NQ][FA_Q_BYTES]
    unsigned char* k_s = q_s + NQ * FA_Q_BYTES;                   // [KS][FA_KV_BYTES]
    unsigned char* v_s = k_s + KS * FA_KV_BYTES;                  // [VS][FA_KV_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + Cfg::TILE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::N_BARS);
    const uint32_t q_full = smem_u32(bars);
    const uint32_t k_full0 = q_full + 8, k_empty0 = k_full0 + 8 * KS;
    const uint32_t v_full0 = k_empty0 + 8 * KS, v_empty0 = v_full0 + 8 * VS;
    const uint32_t s_full0 = v_empty0 + 8 * VS, p_ready0 = s_full0 + 8 * NQ, o_done0 = p_ready0 + 8 * NQ;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = Hq / Hkv, units_per_kv = G / NQ, units = Hkv * units_per_kv;
    // heavy tiles first: within a sequence later tiles see more keys
    const int tile = n_tiles - 1 - (int)(blockIdx.x / units);
    const int unit = blockIdx.x % units;
    const int hk = unit / units_per_kv;
    const int head0 = hk * G + (unit % units_per_kv) * NQ;
    const int tok0 = tile_tok0[tile];
    const int rows = tile_rows[tile];
    const int seq = seq_of_token[tok0];
    const int pos0 = positions[tok0];
    const int pos_last = pos0 + rows - 1;
    const bool geometry_ok = seq >= 0 && seq < n_seqs && pos0 >= 0 && rows >= 1 && rows <= FA_BM &&
                             pos_last / P < bt_stride;
    if (!geometry_ok && threadIdx.x == 0)
        imp_report(status, seq < 0 || seq >= n_seqs ? IMP_BAD_SEQUENCE : IMP_BAD_POSITION);
    // key tiles [kt_lo, kt_hi]: from the window's start of the first row to the last row's own key
    const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int kt_lo = first_key / FA_BN;
    const int kt_hi = geometry_ok ? pos_last / FA_BN : kt_lo - 1;
    const int n_kt = kt_hi - kt_lo + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < KS; ++s) { mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1); }
        for (int s = 0; s < VS; ++s) { mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1); }
        for (int w = 0; w < NQ; ++w) {
            mbar_init(s_full0 + 8 * w, 1);
            mbar_init(p_ready0 + 8 * w, 4);      // one arrival per softmax warp
            mbar_init(o_done0 + 8 * w, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)Cfg::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // With two heads the 384 threads start with 168 registers each; the softmax threads hold a whole row of S
    // (128 values) and take registers over from the first warpgroup, which needs few.
    if (warp < 4) {
    if (NQ == 2) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
    if (warp == 0) {
        if (n_kt > 0) {
            // ------------------------------------------------------------------ producer (whole warp)
            // Lane 0 waits for a free stage and announces the bytes; then every lane fetches boxes: box b of a tile is
            // page b / FA_KB, head-dimension block b % FA_KB.  Page ids are read before the wait, so the table lookup
            // overlaps it.
            if (lane == 0) {
                mbar_expect_tx(q_full, NQ * FA_Q_BYTES);
                for (int w = 0; w < NQ; ++w)
                    for (int kb = 0; kb < FA_KB; ++kb)
                        tma_load_2d(smem_u32(q_s + w * FA_Q_BYTES + kb * FA_BLOCK_BYTES), &map_q, (head0 + w) * DH + kb * 64,
                                    tok0, q_full);
            }
            const int* bt = block_table + (int64_t)seq * bt_stride;
            const int pages_per_tile = FA_BN / P;
            const int boxes = pages_per_tile * FA_KB;         // at most 32: page sizes start at 8
            const int oob_row = num_pages * Hkv * P;          // a box that starts here is all zeros
            const int my_pg = lane / FA_KB, my_kb = lane % FA_KB;
            bool ok = true;
            int k_issued = 0, v_issued = 0;
            for (int i = 0; i < n_kt && ok; ++i) {
                int y = oob_row;
                if (lane < boxes) {
                    const int idx = (kt_lo + i) * pages_per_tile + my_pg;
                    const int page = idx < bt_stride ? bt[idx] : -1;
                    if (page >= 0 && page < num_pages) {
                        y = (page * Hkv + hk) * P;
                    } else if (idx * P <= pos_last && idx * P + P - 1 >= first_key) {
                        // some row of this tile reads the page: it starts at or before the last position and ends inside
                        // the first row's window
                        imp_report(status, IMP_BAD_PAGE);
                    }
                }
                for (int kv = 0; kv < 2 && ok; ++kv) {
                    const int stages = kv == 0 ? KS : VS;
                    const int s = i % stages;
                    const uint32_t full = (kv == 0 ? k_full0 : v_full0) + 8 * s;
                    const uint32_t empty = (kv == 0 ? k_empty0 : v_empty0) + 8 * s;
                    if (lane == 0) {
                        ok = mbar_wait(empty, ((uint32_t)(i / stages) & 1u) ^ 1u, status);
                        if (ok) mbar_expect_tx(full, FA_KV_BYTES);
                    }
                    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                    if (!ok) break;
                    unsigned char* dst = (kv == 0 ? k_s : v_s) + s * FA_KV_BYTES;
                    if (lane < boxes)
                        tma_load_2d(smem_u32(dst + my_kb * FA_BLOCK_BYTES + my_pg * P * 128), kv == 0 ? &map_k : &map_v,
                                    my_kb * 64, y, full);
                    if (kv == 0) k_issued = i + 1; else v_issued = i + 1;
                }
            }
            if (!ok && lane == 0) {   // let the copies in flight land before the CTA's shared memory is released
                mbar_wait(q_full, 0, nullptr);
                for (int i = k_issued > KS ? k_issued - KS : 0; i < k_issued; ++i)
                    mbar_wait(k_full0 + 8 * (i % KS), (uint32_t)(i / KS) & 1u, nullptr);
                for (int i = v_issued > VS ? v_issued - VS : 0; i < v_issued; ++i)
                    mbar_wait(v_full0 + 8 * (i % VS), (uint32_t)(i / VS) & 1u, nullptr);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_kt > 0) {
            // ---------------------------------------------------------------- MMA issuer
            const uint32_t idesc_s = tc_instr_desc(FA_BM, FA_BN);
            const uint32_t idesc_o = tc_instr_desc(FA_BM, DH) | (1u << 16);   // B (= V) is MN-major
            bool ok = mbar_wait(q_full, 0, status);
            auto issue_qk = [&](int w, int i) {
                const uint32_t q_addr = smem_u32(q_s + w * FA_Q_BYTES), k_addr = smem_u32(k_s + (i % KS) * FA_KV_BYTES);
#pragma unroll
                for (int kb = 0; kb < FA_KB; ++kb)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        tc_mma(tmem_base + (uint32_t)(w * 256), tc_smem_desc(q_addr + kb * FA_BLOCK_BYTES + kk * 32),
                               tc_smem_desc(k_addr + kb * FA_BLOCK_BYTES + kk * 32), idesc_s, (kb > 0 || kk > 0) ? 1u : 0u);
                tc_commit(s_full0 + 8 * w);
            };
            if (ok) ok = mbar_wait(k_full0, 0, status);
            if (ok) {
                tc_fence_after_sync();
                for (int w = 0; w < NQ; ++w) issue_qk(w, 0);
                tc_commit(k_empty0);
            }
            for (int i = 0; i < n_kt && ok; ++i) {
                for (int w = 0; w < NQ && ok; ++w) {
                    ok = mbar_wait(p_ready0 + 8 * w, (uint32_t)i & 1u, status);
                    if (ok && w == 0) ok = mbar_wait(v_full0 + 8 * (i % VS), (uint32_t)(i / VS) & 1u, status);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t v_addr = smem_u32(v_s + (i % VS) * FA_KV_BYTES);
                    // P is the A operand straight from tensor memory: 16 keys = 8 columns of bfloat16 pairs per step
#pragma unroll
                    for (int t = 0; t < FA_BN / 16; ++t)
                        fa_mma_ts(tmem_base + (uint32_t)(w * 256 + 128), tmem_base + (uint32_t)(w * 256 + t * 8),
                                  fa_v_desc(v_addr + t * 2048), idesc_o, (i > 0 || t > 0) ? 1u : 0u);
                    tc_commit(o_done0 + 8 * w);
                    if (w == NQ - 1) tc_commit(v_empty0 + 8 * (i % VS));
                    if (i + 1 < n_kt) {
                        if (w == 0) {
                            ok = mbar_wait(k_full0 + 8 * ((i + 1) % KS), (uint32_t)((i + 1) / KS) & 1u, status);
                            if (!ok) break;
                            tc_fence_after_sync();
                        }
                        issue_qk(w, i + 1);
                        if (w == NQ - 1) tc_commit(k_empty0 + 8 * ((i + 1) % KS));
                    }
                }
            }
        }
    }
    } else {
        // -------------------------------------------------------------------- softmax
        if (NQ == 2) asm volatile("setmaxnreg.inc.sync.aligned.u32 224;" ::: "memory");
        const int w = (warp - 4) >> 2;                       // which head of the CTA
        const int row = (warp & 3) * 32 + lane;              // tensor-memory lane = query row of the tile
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_tmem = lane_base + (uint32_t)(w * 256), o_tmem = s_tmem + 128u;
        const int p = pos0 + (row < rows ? row : rows - 1);  // padding rows repeat the last real row
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_kt && ok; ++i) {
            const int k0 = (kt_lo + i) * FA_BN;
            ok = __all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * w, (uint32_t)i & 1u, status));
            if (!ok) break;
            tc_fence_after_sync();
            // a tile needs the mask when a key of it lies behind the first row's position or before the last row's window
            const bool masked = (k0 + FA_BN - 1 > pos0) || (window > 0 && pos0 + FA_BM - 1 - k0 >= window);
            const int hi = p - k0;                                        // columns <= hi are not in the future
            const int lo = window > 0 ? p - window + 1 - k0 : -(1 << 30); // columns >= lo are inside the window
            // the whole row of S: four loads in flight, one wait
            uint32_t sr[FA_BN / 32][32];
#pragma unroll
            for (int c = 0; c < FA_BN / 32; ++c) tc_ld32_issue(s_tmem + (uint32_t)(c * 32), sr[c]);
            tc_wait_ld_pin<true>(sr[0]);
#pragma unroll
            for (int c = 1; c < FA_BN / 32; ++c) tc_wait_ld_pin<false>(sr[c]);
            // four independent maxima: one chain of 128 dependent comparisons would sit on the critical path
            float tm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (masked) {
#pragma unroll
                for (int c = 0; c < FA_BN / 32; ++c)
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = c * 32 + j;
                        if (!(col <= hi && col >= lo)) sr[c][j] = 0xff800000u;   // -inf
                        tm[j & 3] = fmaxf(tm[j & 3], __uint_as_float(sr[c][j]));
                    }
            } else {
#pragma unroll
                for (int c = 0; c < FA_BN / 32; ++c)
#pragma unroll
                    for (int j = 0; j < 32; ++j) tm[j & 3] = fmaxf(tm[j & 3], __uint_as_float(sr[c][j]));
            }
            float tmax = fmaxf(fmaxf(tm[0], tm[1]), fmaxf(tm[2], tm[3]));
            tmax *= scale_log2;                                           // scale > 0: the order is kept
            const bool grow = tmax > m_used + FA_RESCALE_STEP;            // also true for the first finite maximum
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = fmaxf(m_used, tmax);
                const float alpha = (m_used == -INFINITY) ? 0.f : fa_exp2(m_used - m_new);
                l *= alpha;
                if (i > 0) {
                    // P V of tile i-1 has completed: S of this tile was committed after it
#pragma unroll 1
                    for (int c = 0; c < DH / 32; ++c) {
                        float o[32];
                        tc_ld32(o_tmem + (uint32_t)(c * 32), o);
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[j] *= alpha;
                        tc_st32(o_tmem + (uint32_t)(c * 32), o);
                    }
                    tc_wait_st();
                }
                m_used = m_new;
            }
            const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;    // a row with nothing visible yet
            float ls[4] = {0.f, 0.f, 0.f, 0.f};                             // four partial sums, added in a fixed order
            // P = exp2(s - m) as bfloat16 pairs, written over the first 64 columns of S (this thread's own row):
            // keys 2j, 2j+1 share column j, the lower key in the lower half
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                float pk[32];
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int c = 2 * hlf + cc;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float e0 = fa_exp2(fmaf(__uint_as_float(sr[c][j]), scale_log2, -m_sub));   // exp2(-inf) = 0: masked
                        const float e1 = fa_exp2(fmaf(__uint_as_float(sr[c][j + 1]), scale_log2, -m_sub));
                        ls[(j >> 1) & 3] += e0 + e1;
                        pk[cc * 16 + (j >> 1)] = __uint_as_float(fa_pack(e0, e1));
                    }
                }
                tc_st32(s_tmem + (uint32_t)(hlf * 32), pk);
            }
            l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
            tc_wait_st();
            tc_fence_before_sync();                                       // this row's reads and writes of tensor memory
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready0 + 8 * w);
        }
        if (ok && n_kt > 0) ok = __all_sync(0xffffffffu, mbar_wait(o_done0 + 8 * w, (uint32_t)(n_kt - 1) & 1u, status));
        if (ok && n_kt > 0) {
            tc_fence_after_sync();
            const float inv_l = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* o_row = out + (int64_t)(tok0 + row) * out_stride + (int64_t)(head0 + w) * DH;
#pragma unroll 1
            for (int c = 0; c < DH / 32; ++c) {
                float o[32];
                tc_ld32(o_tmem + (uint32_t)(c * 32), o);
                if (row < rows) {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        uint4 u;
                        u.x = fa_pack(o[8 * t] * inv_l, o[8 * t + 1] * inv_l);
                        u.y = fa_pack(o[8 * t + 2] * inv_l, o[8 * t + 3] * inv_l);
                        u.z = fa_pack(o[8 * t + 4] * inv_l, o[8 * t + 5] * inv_l);
                        u.w = fa_pack(o[8 * t + 6] * inv_l, o[8 * t + 7] * inv_l);
                        *reinterpret_cast<uint4*>(o_row + c * 32 + t * 8) = u;
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                     : "memory");
    }
}

// ------------------------------------------------------------------------------------- host
// A [rows, cols] bfloat16 matrix with row stride ld elements, fetched in boxes of box_rows x 64 elements.
static int fa_make_map(CUtensorMap* map, const void* base, int64_t rows, int cols, int64_t ld, int box_rows, const char* what) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        imp_set_error("imp_attn_prefill_tc: the driver does not provide cuTensorMapEncodeTiled");
        return IMP_ERR_UNSUPPORTED;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        imp_set_error("imp_attn_prefill_tc: cuTensorMapEncodeTiled failed with code %d for %s (rows %lld, cols %d, ld %lld)",
                      (int)r, what, (long long)rows, cols, (long long)ld);
        return IMP_ERR_ARG;
    }
    return 0;
}

IMP_API int imp_attn_tc_head_dim(void) { return DH; }
IMP_API int imp_attn_prefill_tc_tile_tokens(void) { return FA_BM; }

// 1 when the kernel takes this geometry (the caller then uses another kernel): page sizes that tile 128 keys
// and are whole 8-row swizzle groups, 16-byte aligned rows.
IMP_API int imp_attn_prefill_tc_supported(int64_t q_stride, int64_t out_stride, int page_size) {
    return (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128) &&
           q_stride % 8 == 0 && out_stride % 8 == 0;
}

template <int NQ>
static int fa_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, __nv_bfloat16* out, int64_t out_stride,
                     const int* block_table, int bt_stride, const int* seq_of_token, const int* positions,
                     const int* tile_tok0, const int* tile_rows, int n_tiles, int n_seqs, int Hq, int Hkv, int P,
                     int num_pages, float scale_log2, int window, int* status, cudaStream_t s) {
    using Cfg = FaCfg<NQ>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Cfg::SMEM_BYTES);
        if (e != cudaSuccess) { imp_set_error("imp_attn_prefill_tc: %s", cudaGetErrorString(e)); return (int)e; }
        attr_set = true;
    }
    const int64_t grid = (int64_t)n_tiles * Hkv * ((Hq / Hkv) / NQ);
    IMP_CHECK_ARG(grid <= 0x7fffffff, "imp_attn_prefill_tc: too many tiles");
    cudaError_t e = imp_launch(attn_prefill_tc_kernel<NQ>, dim3((unsigned)grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, s, mq, mk,
                               mv, out, out_stride, block_table, bt_stride, seq_of_token, positions, tile_tok0, tile_rows,
                               n_tiles, n_seqs, Hq, Hkv, P, num_pages, scale_log2, window, status);
    if (e != cudaSuccess) { imp_set_error("imp_attn_prefill_tc: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}

// out, q: [n_tokens, stride] bfloat16 (head h at column h*DH).  kc, vc: [num_pages, Hkv, P, DH] of one layer.
// tile_tok0 / tile_rows: tiles of up to 128 consecutive tokens of one sequence (first row in q/out, row count).
IMP_API int imp_attn_prefill_tc(void* out, int64_t out_stride, const void* q, int64_t q_stride, int n_tokens, const void* kc,
                                const void* vc, const int* block_table, int bt_stride, const int* seq_of_token,
                                const int* positions, const int* tile_tok0, const int* tile_rows, int n_tiles, int n_seqs,
                                int Hq, int Hkv, int P, int num_pages, float scale, int window, int* status, void* stream) {
    if (n_tiles == 0) return 0;
    IMP_CHECK_ARG(out && q && kc && vc && block_table && seq_of_token && positions && tile_tok0 && tile_rows,
                  "imp_attn_prefill_tc: null pointer");
    IMP_CHECK_ARG(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "imp_attn_prefill_tc: %d query heads are not a multiple of %d kv heads",
                  Hq, Hkv);
    IMP_CHECK_ARG(imp_attn_prefill_tc_supported(q_stride, out_stride, P),
                  "imp_attn_prefill_tc: page size %d or strides %lld / %lld not supported by this kernel", P,
                  (long long)q_stride, (long long)out_stride);
    IMP_CHECK_ARG(q_stride >= (int64_t)Hq * DH && out_stride >= (int64_t)Hq * DH && n_tokens > 0 && num_pages > 0 &&
                      window >= 0 && scale > 0.f,
                  "imp_attn_prefill_tc: bad geometry");
    IMP_CHECK_ARG(((uintptr_t)q % 16) == 0 && ((uintptr_t)kc % 16) == 0 && ((uintptr_t)vc % 16) == 0 && ((uintptr_t)out % 16) == 0,
                  "imp_attn_prefill_tc: pointers must be 16-byte aligned");
    CUtensorMap mq, mk, mv;
    if (int rc = fa_make_map(&mq, q, n_tokens, Hq * DH, q_stride, FA_BM, "q")) return rc;
    const int64_t kv_rows = (int64_t)num_pages * Hkv * P;
    if (int rc = fa_make_map(&mk, kc, kv_rows, DH, DH, P, "k")) return rc;
    if (int rc = fa_make_map(&mv, vc, kv_rows, DH, DH, P, "v")) return rc;
    const float scale_log2 = scale * 1.4426950408889634f;
    cudaStream_t s = (cudaStream_t)stream;
#define FA_ARGS mq, mk, mv, (__nv_bfloat16*)out, out_stride, block_table, bt_stride, seq_of_token, positions, tile_tok0, tile_rows, \
                n_tiles, n_seqs, Hq, Hkv, P, num_pages, scale_log2, window, status, s
    if ((Hq / Hkv) % 2 == 0) return fa_launch<2>(FA_ARGS);
    return fa_launch<1>(FA_ARGS);
#undef FA_ARGS
}
