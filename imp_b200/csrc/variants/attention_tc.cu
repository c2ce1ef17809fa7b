// Paged prefill attention on the fifth-generation tensor cores (tcgen05 + tensor memory), bfloat16,
// compiled once per head size: -DIMP_ATTN_DH=64 or 128.
//
// A work item is one tile of up to 128 consecutive query tokens of one sequence and NQ (1 or 2) query
// heads that share a kv head; it walks the cached keys of the sequence in tiles of 128 from the
// window's start to the last token's position (keys come from the pages only; the new tokens'
// keys are already there).  One CTA per SM (a CTA holds all of an SM's tensor memory) works through
// several items: the list has the heavy tiles first and the CTAs walk it forth and back, so that the
// sums per CTA come out nearly equal, and barriers, tensor memory and the pipeline are set up once.
// While the softmax warps store one item's result, the Q tiles of the next are already loaded and its
// first S is on the tensor cores.  Roles:
//   warp 0           producer.  Per item the Q tiles, then per key tile the K pages and the V pages of the
//                    kv head with TMA (cp.async.bulk.tensor, 128-byte swizzle), one box per page
//                    and 64 head dimensions, into shared-memory rings; page ids come from the block
//                    table, pages that do not exist are fetched from beyond the tensor (zeros).
//   warp 1           MMA issuer.  S_w = Q_w K^T (M=128 tokens, N=128 keys, K=head size) into tensor
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

#include <cstdlib>

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
    static constexpr int OUT_BYTES = 128 * 128;           // per head: 128 rows x 64 dims of O on their way to a TMA store
    static constexpr int TILE_BYTES = NQ * FA_Q_BYTES + (K_STAGES + V_STAGES) * FA_KV_BYTES + NQ * OUT_BYTES;
    static constexpr int N_BARS = 2 + 2 * K_STAGES + 2 * V_STAGES + 4 * NQ;
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

// The MMAs of one S tile (S = Q K^T over the whole head size) and of one O update (O += P V over 128 keys) as one
// block of instructions each: descriptors advance by constants inside the block, one lane of the (converged) warp is
// elected once and issues all of them.  Written out because the issuing thread is on the critical path of every tile:
// with the descriptors built per MMA in C++ a tile's sixteen MMAs took about 1,500 cycles to issue, more than the 1,024
// the tensor cores need to run them.
// Q and K tiles: 64-wide blocks of the head dimension 16 KiB apart (descriptor units of 16 bytes: 1024), K steps of
// 16 elements = 32 bytes (2 units).
#define FA_QK_STEP(a_off, b_off, pred)                                         \
    "add.u64 a, %1, " #a_off ";\n"                                             \
    "add.u64 b, %2, " #b_off ";\n"                                             \
    "@e tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, " #pred ";\n"
__device__ __forceinline__ void fa_issue_qk(uint32_t d_tmem, uint64_t q_desc, uint64_t k_desc, uint32_t idesc) {
    asm volatile(
        "{\n"
        ".reg .pred e, yes, no;\n"
        ".reg .b64 a, b;\n"
        "elect.sync _|e, 0xffffffff;\n"
        "setp.eq.u32 yes, 0, 0;\n"
        "setp.ne.u32 no, 0, 0;\n"
        FA_QK_STEP(0, 0, no) FA_QK_STEP(2, 2, yes) FA_QK_STEP(4, 4, yes) FA_QK_STEP(6, 6, yes)
#if IMP_ATTN_DH == 128
        FA_QK_STEP(1024, 1024, yes) FA_QK_STEP(1026, 1026, yes) FA_QK_STEP(1028, 1028, yes) FA_QK_STEP(1030, 1030, yes)
#endif
        "}\n" ::"r"(d_tmem), "l"(q_desc), "l"(k_desc), "r"(idesc)
        : "memory");
}
#undef FA_QK_STEP
// P (tensor memory, 8 columns of bfloat16 pairs per 16 keys) times V (16 keys = 2 swizzle groups of 1024 bytes: 128
// descriptor units per step) for one half of a tile (64 keys); the first MMA overwrites O unless `accumulate`.
#define FA_PV_STEP(t, pred)                                                    \
    "add.u32 pa, %1, " #t " * 8;\n"                                            \
    "add.u64 b, %2, " #t " * 128;\n"                                           \
    "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], b, %3, " #pred ";\n"
__device__ __forceinline__ void fa_issue_pv(uint32_t o_tmem, uint32_t p_tmem, uint64_t v_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred e, yes, first;\n"
        ".reg .b64 b;\n"
        ".reg .b32 pa;\n"
        "elect.sync _|e, 0xffffffff;\n"
        "setp.eq.u32 yes, 0, 0;\n"
        "setp.ne.u32 first, %4, 0;\n"
        FA_PV_STEP(0, first) FA_PV_STEP(1, yes) FA_PV_STEP(2, yes) FA_PV_STEP(3, yes)
        "}\n" ::"r"(o_tmem), "r"(p_tmem), "l"(v_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
#undef FA_PV_STEP

__device__ __forceinline__ float fa_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The softmax warps are bound by the number of instructions they issue (a share of the exponentials computed on the
// FMA pipe instead of the special-function unit made them slower), so the arithmetic around the exponentials uses
// the two-wide 32-bit instructions and the three-input maximum of this architecture.
__device__ __forceinline__ float fa_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// (x0, x1) = (a0, a1) * s + t
__device__ __forceinline__ void fa_fma2(float& x0, float& x1, float a0, float a1, float s, float t) {
    asm("{\n"
        ".reg .b64 a, b, c, d;\n"
        "mov.b64 a, {%2, %3};\n"
        "mov.b64 b, {%4, %4};\n"
        "mov.b64 c, {%5, %5};\n"
        "fma.rn.f32x2 d, a, b, c;\n"
        "mov.b64 {%0, %1}, d;\n"
        "}\n"
        : "=f"(x0), "=f"(x1)
        : "f"(a0), "f"(a1), "f"(s), "f"(t));
}
// (s0, s1) += (a0, a1)
__device__ __forceinline__ void fa_add2(float& s0, float& s1, float a0, float a1) {
    asm("{\n"
        ".reg .b64 a, b, d;\n"
        "mov.b64 a, {%0, %1};\n"
        "mov.b64 b, {%2, %3};\n"
        "add.rn.f32x2 d, a, b;\n"
        "mov.b64 {%0, %1}, d;\n"
        "}\n"
        : "+f"(s0), "+f"(s1)
        : "f"(a0), "f"(a1));
}

__device__ __forceinline__ uint32_t fa_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// -DFA_TRACE: CTA 0 records SM clock values at the hand-overs of its pipeline (for reading a timeline; never in a
// product build).  Slot layout: role * 1024 + event index; roles 0: MMA issuer, 1: softmax head 0, 2: softmax head 1.
#ifdef FA_TRACE
__device__ long long fa_trace_buf[3 * 1024];
#define FA_TR(role, idx) do { if (blockIdx.x == 0 && (idx) < 1024) fa_trace_buf[(role) * 1024 + (idx)] = clock64(); } while (0)
IMP_API int imp_attn_tc_trace(long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, fa_trace_buf, sizeof(long long) * (size_t)(n < 3072 ? n : 3072));
}
#else
#define FA_TR(role, idx) do {} while (0)
#endif

// Geometry of one work item: one tile of query tokens and NQ query heads of one kv head.
struct FaItem {
    int hk, head0, tok0, rows, seq, pos0, pos_last, first_key, kt_lo, n_kt;
    bool geometry_ok;
};

template <int NQ>
__global__ void __launch_bounds__(FaCfg<NQ>::THREADS, 1) attn_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, int out_tma,
    __nv_bfloat16* __restrict__ out, int64_t out_stride,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ seq_of_token,
    const int* __restrict__ positions, const int* __restrict__ tile_tok0, const int* __restrict__ tile_rows, int n_tiles,
    int n_seqs, int Hq, int Hkv, int P, int num_pages, float scale_log2, int window, int* status) {
    using Cfg = FaCfg<NQ>;
    constexpr int KS = Cfg::K_STAGES, VS = Cfg::V_STAGES;
    extern __shared__ unsigned char fa_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = tiles;                                   // [NQ][FA_Q_BYTES]
    unsigned char* k_s = q_s + NQ * FA_Q_BYTES;                   // [KS][FA_KV_BYTES]
    unsigned char* v_s = k_s + KS * FA_KV_BYTES;                  // [VS][FA_KV_BYTES]
    unsigned char* o_s = v_s + VS * FA_KV_BYTES;                  // [NQ][OUT_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + Cfg::TILE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::N_BARS);
    const uint32_t q_full = smem_u32(bars), q_empty = q_full + 8;
    const uint32_t k_full0 = q_empty + 8, k_empty0 = k_full0 + 8 * KS;
    const uint32_t v_full0 = k_empty0 + 8 * KS, v_empty0 = v_full0 + 8 * VS;
    // p_ready: per head two barriers, one for each half (64 keys) of P
    const uint32_t s_full0 = v_empty0 + 8 * VS, p_ready0 = s_full0 + 8 * NQ, o_done0 = p_ready0 + 16 * NQ;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = Hq / Hkv, units_per_kv = G / NQ, units = Hkv * units_per_kv;
    const int n_items = n_tiles * units;

    // Nothing up to pdl_wait() touches what an earlier kernel of the stream may still write.
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int s = 0; s < KS; ++s) { mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1); }
        for (int s = 0; s < VS; ++s) { mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1); }
        for (int w = 0; w < NQ; ++w) {
            mbar_init(s_full0 + 8 * w, 1);
            mbar_init(p_ready0 + 16 * w, 4);     // one arrival per softmax warp
            mbar_init(p_ready0 + 16 * w + 8, 4);
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
    pdl_wait();
    pdl_launch_dependents();

    // The CTA's item in pass p.  The list has the heavy tiles first (within a sequence later tiles see more keys), and
    // the passes walk it forth and back: the CTA that got the heaviest item of one pass gets the lightest of the next.
    // Every role walks the same items in the same order; an item without keys (or with a broken geometry) is skipped by
    // all of them.
    auto load_item = [&](int pass, FaItem& it) -> bool {
        const int grid = (int)gridDim.x;
        const int k = pass * grid + ((pass & 1) ? grid - 1 - (int)blockIdx.x : (int)blockIdx.x);
        if (k >= n_items) return false;
        const int tile = n_tiles - 1 - k / units, unit = k % units;
        it.hk = unit / units_per_kv;
        it.head0 = it.hk * G + (unit % units_per_kv) * NQ;
        it.tok0 = tile_tok0[tile];
        it.rows = tile_rows[tile];
        it.seq = seq_of_token[it.tok0];
        it.pos0 = positions[it.tok0];
        it.pos_last = it.pos0 + it.rows - 1;
        it.geometry_ok = it.seq >= 0 && it.seq < n_seqs && it.pos0 >= 0 && it.rows >= 1 && it.rows <= FA_BM &&
                         it.pos_last / P < bt_stride;
        // key tiles [kt_lo, kt_hi]: from the window's start of the first row to the last row's own key
        it.first_key = (window > 0 && it.pos0 - window + 1 > 0) ? it.pos0 - window + 1 : 0;
        it.kt_lo = it.first_key / FA_BN;
        const int kt_hi = it.geometry_ok ? it.pos_last / FA_BN : it.kt_lo - 1;
        it.n_kt = kt_hi - it.kt_lo + 1;
        return true;
    };

    // With two heads the 384 threads start with 168 registers each; the softmax threads hold a whole row of S
    // (128 values) and take registers over from the first warpgroup, which needs few.
    if (warp < 4) {
    if (NQ == 2) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
    if (warp == 0) {
        // ------------------------------------------------------------------ producer (whole warp)
        // Lane 0 waits for a free stage and announces the bytes; then every lane fetches boxes: box b of a tile is
        // page b / FA_KB, head-dimension block b % FA_KB.  Page ids are read before the wait, so the table lookup
        // overlaps it.  K and V tiles are numbered through all items of the CTA (kv_n); an item's Q tiles follow its
        // first K tile, once the MMAs of the item before have read theirs (q_empty).
        const int pages_per_tile = FA_BN / P;
        const int boxes = pages_per_tile * FA_KB;         // at most 32: page sizes start at 8
        const int oob_row = num_pages * Hkv * P;          // a box that starts here is all zeros
        const int my_pg = lane / FA_KB, my_kb = lane % FA_KB;
        bool ok = true;
        int k_n = 0, v_n = 0, q_n = 0;                    // K tiles, V tiles and Q loads issued so far
        FaItem it;
        for (int pass = 0; ok && load_item(pass, it); ++pass) {
            if (!it.geometry_ok && lane == 0)
                imp_report(status, it.seq < 0 || it.seq >= n_seqs ? IMP_TAGGED(IMP_BAD_SEQUENCE, 4) : IMP_TAGGED(IMP_BAD_POSITION, 4));
            if (it.n_kt <= 0) continue;
            const int* bt = block_table + (int64_t)it.seq * bt_stride;
            for (int i = 0; i < it.n_kt && ok; ++i) {
                int y = oob_row;
                if (lane < boxes) {
                    const int idx = (it.kt_lo + i) * pages_per_tile + my_pg;
                    const int page = idx < bt_stride ? bt[idx] : -1;
                    if (page >= 0 && page < num_pages) {
                        y = (page * Hkv + it.hk) * P;
                    } else if (idx * P <= it.pos_last && idx * P + P - 1 >= it.first_key) {
                        // some row of this tile reads the page: it starts at or before the last position and ends inside
                        // the first row's window
                        imp_report(status, IMP_BAD_PAGE);
                    }
                }
                for (int kv = 0; kv < 2 && ok; ++kv) {
                    const int stages = kv == 0 ? KS : VS;
                    const int n = kv == 0 ? k_n : v_n;
                    const int s = n % stages;
                    const uint32_t full = (kv == 0 ? k_full0 : v_full0) + 8 * s;
                    const uint32_t empty = (kv == 0 ? k_empty0 : v_empty0) + 8 * s;
                    if (lane == 0) {
                        ok = mbar_wait(empty, ((uint32_t)(n / stages) & 1u) ^ 1u, status);
                        if (ok) mbar_expect_tx(full, FA_KV_BYTES);
                    }
                    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                    if (!ok) break;
                    unsigned char* dst = (kv == 0 ? k_s : v_s) + s * FA_KV_BYTES;
                    if (lane < boxes)
                        tma_load_2d(smem_u32(dst + my_kb * FA_BLOCK_BYTES + my_pg * P * 128), kv == 0 ? &map_k : &map_v,
                                    my_kb * 64, y, full);
                    if (kv == 0) ++k_n; else ++v_n;
                    if (kv == 0 && i == 0) {
                        if (lane == 0) {
                            if (q_n > 0) ok = mbar_wait(q_empty, (uint32_t)(q_n - 1) & 1u, status);
                            if (ok) {
                                mbar_expect_tx(q_full, NQ * FA_Q_BYTES);
                                for (int w = 0; w < NQ; ++w)
                                    for (int kb = 0; kb < FA_KB; ++kb)
                                        tma_load_2d(smem_u32(q_s + w * FA_Q_BYTES + kb * FA_BLOCK_BYTES), &map_q,
                                                    (it.head0 + w) * DH + kb * 64, it.tok0, q_full);
                            }
                        }
                        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                        if (ok) ++q_n;
                    }
                }
            }
        }
        if (!ok && lane == 0) {   // let the copies in flight land before the CTA's shared memory is released
            if (q_n > 0) mbar_wait(q_full, (uint32_t)(q_n - 1) & 1u, nullptr);
            for (int n = k_n > KS ? k_n - KS : 0; n < k_n; ++n)
                mbar_wait(k_full0 + 8 * (n % KS), (uint32_t)(n / KS) & 1u, nullptr);
            for (int n = v_n > VS ? v_n - VS : 0; n < v_n; ++n)
                mbar_wait(v_full0 + 8 * (n % VS), (uint32_t)(n / VS) & 1u, nullptr);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (whole warp)
        // All lanes run this code with the same values, so that addresses and descriptors stay in uniform registers;
        // each MMA and each commit is then issued by one elected lane.  (A single lane running the loop alone spent
        // about 100 cycles per MMA, more than the 64 the tensor cores need for it.)
        // Per key tile and head: O_w += P_w V once the softmax has written P_w, then S_w = Q_w K^T of the next tile,
        // so while one head's softmax runs the tensor cores work on the other head.  After the last tile of an item
        // both heads' S of the next item's first tile follow at once: the softmax warps find them ready when they
        // come back from storing the item's result.
#ifdef FA_EXP_N64   // timing experiment only (wrong results): S tiles of 64 keys, to see whether issue or execution sets the pace
        const uint32_t idesc_s = tc_instr_desc(FA_BM, 64);
#else
        const uint32_t idesc_s = tc_instr_desc(FA_BM, FA_BN);
#endif
        const uint32_t idesc_o = tc_instr_desc(FA_BM, DH) | (1u << 16);   // B (= V) is MN-major
        bool ok = true;
        int kv_n = 0;                 // number of the current K / V tile among all of the CTA's
        int t_n = 0;                  // tiles finished: the phase of s_full, p_ready, o_done
        int item_n = 0;               // items started: the phase of q_full
        int pass = 0;
        auto wait_all = [&](uint32_t bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, status)) != 0; };
        auto next_n_kt = [&]() -> int {   // key tiles of the CTA's next item with work; 0: none left
            FaItem it;
            while (load_item(pass++, it))
                if (it.n_kt > 0) return it.n_kt;
            return 0;
        };
        static_assert(FA_BN == 128, "fa_issue_pv is written for halves of tiles of 128 keys");
        const uint64_t q_desc0 = tc_smem_desc(smem_u32(q_s)), k_desc0 = tc_smem_desc(smem_u32(k_s)), v_desc0 = fa_v_desc(smem_u32(v_s));
        auto issue_qk = [&](int w, int n) {      // S_w = Q_w K^T with K tile number n
            fa_issue_qk(tmem_base + (uint32_t)(w * 256), q_desc0 + (uint64_t)(w * (FA_Q_BYTES >> 4)),
                        k_desc0 + (uint64_t)((n % KS) * (FA_KV_BYTES >> 4)), idesc_s);
            if (tc_elect_one()) tc_commit(s_full0 + 8 * w);
        };
        // S of an item's first tile, both heads: its Q tiles and K tile number n
        auto first_qk = [&](int n, int n_kt) {
            ok = wait_all(q_full, (uint32_t)item_n & 1u);
            if (ok) ok = wait_all(k_full0 + 8 * (n % KS), (uint32_t)(n / KS) & 1u);
            if (!ok) return;
            tc_fence_after_sync();
            for (int w = 0; w < NQ; ++w) issue_qk(w, n);
            if (tc_elect_one()) {
                tc_commit(k_empty0 + 8 * (n % KS));
                if (n_kt == 1) tc_commit(q_empty);      // the item's only use of Q
            }
            ++item_n;
        };
        int n_kt = next_n_kt();
        if (n_kt > 0) first_qk(0, n_kt);
        while (n_kt > 0 && ok) {
            const int n_kt_next = next_n_kt();
            for (int i = 0; i < n_kt && ok; ++i, ++kv_n, ++t_n) {
                const bool last = i + 1 == n_kt;
                for (int w = 0; w < NQ && ok; ++w) {
                    if (lane == 0) FA_TR(0, (t_n * 2 + w) * 4 + 0);
                    // the first 64 keys of P are there while the softmax still works on the other 64
                    ok = wait_all(p_ready0 + 16 * w, (uint32_t)t_n & 1u);
                    if (lane == 0) FA_TR(0, (t_n * 2 + w) * 4 + 1);
                    if (ok && w == 0) ok = wait_all(v_full0 + 8 * (kv_n % VS), (uint32_t)(kv_n / VS) & 1u);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t v_desc = v_desc0 + (uint64_t)((kv_n % VS) * (FA_KV_BYTES >> 4));
                    fa_issue_pv(tmem_base + (uint32_t)(w * 256 + 128), tmem_base + (uint32_t)(w * 256), v_desc, idesc_o, i > 0 ? 1u : 0u);
                    ok = wait_all(p_ready0 + 16 * w + 8, (uint32_t)t_n & 1u);
                    if (!ok) break;
                    tc_fence_after_sync();
                    fa_issue_pv(tmem_base + (uint32_t)(w * 256 + 128), tmem_base + (uint32_t)(w * 256 + 32), v_desc + 4 * 128, idesc_o, 1u);
                    if (tc_elect_one()) {
                        tc_commit(o_done0 + 8 * w);
                        if (w == NQ - 1) tc_commit(v_empty0 + 8 * (kv_n % VS));
                    }
                    if (lane == 0) FA_TR(0, (t_n * 2 + w) * 4 + 2);
                    if (!last) {
                        if (w == 0) {
                            ok = wait_all(k_full0 + 8 * ((kv_n + 1) % KS), (uint32_t)((kv_n + 1) / KS) & 1u);
                            if (!ok) break;
                            tc_fence_after_sync();
                        }
                        issue_qk(w, kv_n + 1);
                        if (lane == 0) FA_TR(0, (t_n * 2 + w) * 4 + 3);
                        if (w == NQ - 1 && tc_elect_one()) {
                            tc_commit(k_empty0 + 8 * ((kv_n + 1) % KS));
                            if (i + 2 == n_kt) tc_commit(q_empty);   // that was the item's last use of Q
                        }
                    }
                }
                if (last && ok && n_kt_next > 0) first_qk(kv_n + 1, n_kt_next);
            }
            n_kt = n_kt_next;
        }
    }
    } else {
        // -------------------------------------------------------------------- softmax
        if (NQ == 2) asm volatile("setmaxnreg.inc.sync.aligned.u32 224;" ::: "memory");
        const int w = (warp - 4) >> 2;                       // which head of the CTA
        const int row = (warp & 3) * 32 + lane;              // tensor-memory lane = query row of the tile
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_tmem = lane_base + (uint32_t)(w * 256), o_tmem = s_tmem + 128u;
        bool ok = true;
        int t_n = 0;                                         // tiles finished: the phase of s_full and o_done
        FaItem it;
        for (int pass = 0; ok && load_item(pass, it); ++pass) {
        if (it.n_kt <= 0) continue;
        const int n_kt = it.n_kt, pos0 = it.pos0, rows = it.rows;
        const int p = pos0 + (row < rows ? row : rows - 1);  // padding rows repeat the last real row
        float m_used = -INFINITY, l = 0.f;
        for (int i = 0; i < n_kt && ok; ++i, ++t_n) {
            const int k0 = (it.kt_lo + i) * FA_BN;
            if ((warp & 3) == 0 && lane == 0) FA_TR(1 + w, t_n * 6 + 0);
            ok = __all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * w, (uint32_t)t_n & 1u, status));
            if (!ok) break;
            tc_fence_after_sync();
            if ((warp & 3) == 0 && lane == 0) FA_TR(1 + w, t_n * 6 + 1);
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
            if ((warp & 3) == 0 && lane == 0) FA_TR(1 + w, t_n * 6 + 2);
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
                    for (int j = 0; j < 32; j += 2)
                        tm[(j >> 1) & 3] = fa_max3(tm[(j >> 1) & 3], __uint_as_float(sr[c][j]), __uint_as_float(sr[c][j + 1]));
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
            if ((warp & 3) == 0 && lane == 0) FA_TR(1 + w, t_n * 6 + 3);
            const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;    // a row with nothing visible yet
            float ls[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};         // eight partial sums, added in a fixed order
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
                        float x0, x1;
                        fa_fma2(x0, x1, __uint_as_float(sr[c][j]), __uint_as_float(sr[c][j + 1]), scale_log2, -m_sub);
                        const float e0 = fa_exp2(x0), e1 = fa_exp2(x1);                  // exp2(-inf) = 0: masked
                        fa_add2(ls[j & 6], ls[(j & 6) + 1], e0, e1);
                        pk[cc * 16 + (j >> 1)] = __uint_as_float(fa_pack(e0, e1));
                    }
                }
                tc_st32(s_tmem + (uint32_t)(hlf * 32), pk);
                // each half is handed over by itself: the MMAs of the first run while the second is computed
                if (hlf == 1) {
                    l += ((ls[0] + ls[1]) + (ls[2] + ls[3])) + ((ls[4] + ls[5]) + (ls[6] + ls[7]));
                    if ((warp & 3) == 0 && lane == 0) FA_TR(1 + w, t_n * 6 + 4);
                }
                tc_wait_st();
                tc_fence_before_sync();                                   // this row's reads and writes of tensor memory
                __syncwarp();
                if (lane == 0) mbar_arrive(p_ready0 + 16 * w + 8 * hlf);
            }
            if ((warp & 3) == 0 && lane == 0) FA_TR(1 + w, t_n * 6 + 5);
        }
        // The item's result.  The loads of O are complete (tc_ld32 waits) before this warp signals its next P, and the
        // first P V of the next item, which overwrites O, waits for that signal of all four warps.
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_done0 + 8 * w, (uint32_t)(t_n - 1) & 1u, status));
        if (out_tma) {
            // the head's four warps meet at barriers below: they go on, or give up, together (a warp that gave up
            // inside the item arrives here too, the others after their own waits have run out)
            uint32_t all;
            asm volatile(
                "{\n"
                ".reg .pred p, q;\n"
                "setp.ne.u32 p, %1, 0;\n"
                "bar.red.and.pred q, %2, 128, p;\n"
                "selp.u32 %0, 1, 0, q;\n"
                "}\n"
                : "=r"(all)
                : "r"((uint32_t)ok), "r"(1 + w)
                : "memory");
            ok = all != 0;
        }
        if (ok && out_tma && rows == FA_BM) {
            // A full tile leaves through shared memory and TMA stores, 64 dims at a time: every thread storing 16 bytes
            // to its own row of `out` (rows 8 KB apart) took about 3 us per item.  (A ragged tile keeps the stores below:
            // a box of 128 rows would run into the next sequence's tokens.)
            tc_fence_after_sync();
            const float inv_l = l > 0.f ? 1.f / l : 0.f;
            unsigned char* buf = o_s + w * Cfg::OUT_BYTES;
            const bool storer = (warp & 3) == 0 && lane == 0;
#pragma unroll 1
            for (int sub = 0; sub < DH / 64; ++sub) {
                if (storer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the buffer's last store has read it
                asm volatile("bar.sync %0, 128;" ::"r"(1 + w) : "memory");
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    float o[32];
                    tc_ld32(o_tmem + (uint32_t)((2 * sub + cc) * 32), o);
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        uint4 u;
                        u.x = fa_pack(o[8 * t] * inv_l, o[8 * t + 1] * inv_l);
                        u.y = fa_pack(o[8 * t + 2] * inv_l, o[8 * t + 3] * inv_l);
                        u.z = fa_pack(o[8 * t + 4] * inv_l, o[8 * t + 5] * inv_l);
                        u.w = fa_pack(o[8 * t + 6] * inv_l, o[8 * t + 7] * inv_l);
                        *reinterpret_cast<uint4*>(buf + row * 128 + (((4 * cc + t) ^ (row & 7)) << 4)) = u;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync %0, 128;" ::"r"(1 + w) : "memory");
                if (storer) {
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&map_o),
                                 "r"((it.head0 + w) * DH + sub * 64), "r"(it.tok0), "r"(smem_u32(buf))
                                 : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
            tc_fence_before_sync();
        } else if (ok) {
            tc_fence_after_sync();
            const float inv_l = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* o_row = out + (int64_t)(it.tok0 + row) * out_stride + (int64_t)(it.head0 + w) * DH;
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
            tc_fence_before_sync();
        }
        }
        if (out_tma && (warp & 3) == 0 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // `out` is written
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
static int fa_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, int out_tma,
                     __nv_bfloat16* out, int64_t out_stride,
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
    const int64_t items = (int64_t)n_tiles * Hkv * ((Hq / Hkv) / NQ);
    IMP_CHECK_ARG(items <= 0x7fffffff, "imp_attn_prefill_tc: too many tiles");
    static int sms = 0;                 // one CTA fits an SM (all of its tensor memory); the CTAs share out the items
    if (sms <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 1;
    }
    const int64_t grid = items < sms ? items : sms;
    cudaError_t e = imp_launch(attn_prefill_tc_kernel<NQ>, dim3((unsigned)grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, s, mq, mk,
                               mv, mo, out_tma, out, out_stride, block_table, bt_stride, seq_of_token, positions, tile_tok0, tile_rows,
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
    // full tiles of the result leave through TMA stores (boxes of 128 rows x 64 dims of `out`)
    CUtensorMap mo{};
    int out_tma = 0;
    {
        const char* env = getenv("IMP_B200_ATTN_TMA_STORE");
        if (!(env && atoi(env) == 0)) out_tma = fa_make_map(&mo, out, n_tokens, Hq * DH, out_stride, FA_BM, "out") == 0 ? 1 : 0;
    }
#define FA_ARGS mq, mk, mv, mo, out_tma, (__nv_bfloat16*)out, out_stride, block_table, bt_stride, seq_of_token, positions, tile_tok0, tile_rows, \
                n_tiles, n_seqs, Hq, Hkv, P, num_pages, scale_log2, window, status, s
    // Two heads per item halve the K / V traffic; one head per item gives twice as many, half as long items.  With
    // fewer two-head items than half the SMs (a portion of a prompt late in a long sequence: few tiles, each with many
    // keys) the longest item sets the time, so the heads are shared out one by one.
    static int pair_min_items = -1;       // IMP_B200_ATTN_PAIR_MIN: two heads per item from this many items on
    if (pair_min_items < 0) {
        const char* e = getenv("IMP_B200_ATTN_PAIR_MIN");
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 0;
        pair_min_items = e ? atoi(e) : sms / 2 + 1;
    }
    const int64_t pair_items = (int64_t)n_tiles * Hkv * ((Hq / Hkv) / 2);
    if ((Hq / Hkv) % 2 == 0 && pair_items >= pair_min_items) return fa_launch<2>(FA_ARGS);
    return fa_launch<1>(FA_ARGS);
#undef FA_ARGS
}
