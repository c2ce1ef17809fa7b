// Paged flash attention on warp-level tensor-core MMAs (bfloat16 in, 32-bit softmax and
// accumulation), compiled once per head size: -DIMP_ATTN_DH=<multiple of 16, at most 256>.
//
// Two entry points over the same inner loop:
//   decode : one query token per sequence.  A CTA owns (token, kv head, split of the keys); its
//            16-row tile holds the query heads that share the kv head, so every key and value
//            byte is read once per group.  Splits write unnormalised partial results to scratch
//            and a second kernel merges them.  Launch shape depends on the batch size only and
//            key ranges are read from device memory, so a captured graph serves any context.
//   prefill: a CTA owns up to 32 consecutive query tokens of one sequence and up to 4 query heads
//            of one kv head (a warp: 16 tokens of one head); its warps share every staged key and
//            value tile while they walk the cached keys from the window's start to the last
//            token's position.
// In the prefill kernel keys and values travel from the pages to shared memory through a cp.async
// ring (rows padded so that fragment reads are free of bank conflicts) and are shared by the CTA's
// warps; in the decode kernel every warp reads its own keys straight from the pages.  Either way
// fragments are filled with 16-byte loads and no ldmatrix: the contraction index of each product is permuted so that what a lane
// reads contiguously is what its fragment needs.  For S = Q K^T the head dimension is permuted
// (the same permutation on Q's fragments), for O = P V the value columns are permuted and
// un-permuted when the result is written.
//
// Math as in the reference's kernels (src/compute/attention.cu:158-216 prefill,
// src/compute/attention_paged.cu:904-1195 split-K decode + reduce): s = scale * q.k, causal and
// window masks, running max and sum, o = sum p v; the reference's kernels are half-precision
// WMMA / CUDA-core code over the call's own K,V (prefill) or one query per sequence (decode).
#include "../common.cuh"

#include <cstdlib>

IMP_TL_DEFINE(attention_mma)

#ifndef IMP_ATTN_DH
#error "compile with -DIMP_ATTN_DH=<head size>"
#endif

constexpr int DH = IMP_ATTN_DH;
static_assert(DH % 16 == 0 && DH >= 16 && DH <= 256, "head size must be a multiple of 16 in [16, 256]");
constexpr int KSTEPS = DH / 16;       // k-steps of the QK^T product
constexpr int NTILES = DH / 8;        // 8-wide output tiles of the PV product
constexpr int WARPS = 4;          // decode: warps per CTA, taking 16-key steps in turn

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Dimension permutation of the QK^T contraction.  The head dimension is cut into blocks of 32
// (plus one block of 16 when DH % 32 == 16).  In a 32-block, lane t (= lane & 3) loads the 8
// contiguous elements [8t, 8t+8) of a row; k-step s (0 or 1) of the block takes elements
// 4s..4s+3 of them as (k=2t,2t+1) and (k=2t+8,2t+9).  In a 16-block lane t loads [4t, 4t+4).
template <typename Row>
__device__ __forceinline__ void load_row_frags(uint32_t (&f)[KSTEPS][2], const Row* __restrict__ row, int t) {
#pragma unroll
    for (int b = 0; b < DH / 32; ++b) {
        const uint4 v = *reinterpret_cast<const uint4*>(row + b * 32 + 8 * t);
        f[2 * b][0] = v.x; f[2 * b][1] = v.y; f[2 * b + 1][0] = v.z; f[2 * b + 1][1] = v.w;
    }
    if (DH % 32) {
        const uint2 v = *reinterpret_cast<const uint2*>(row + (DH / 32) * 32 + 4 * t);
        f[KSTEPS - 1][0] = v.x; f[KSTEPS - 1][1] = v.y;
    }
}

// Value columns are cut into blocks of 64, then 32, then 16.  In a block of NT tiles (NT = 8, 4, 2)
// lane g (= lane >> 2) loads the NT contiguous elements [NT*g, NT*g + NT) of a value row; element i
// is column g of output tile i.  So accumulator (tile i, column c) of the block holds dimension
// base + NT*c + i.
struct VBlocks {
    static constexpr int N64 = DH / 64;
    static constexpr int HAS32 = (DH % 64) >= 32;
    static constexpr int HAS16 = (DH % 32) == 16;
};

// One row of the tile as this lane sees it.
struct RowInfo {
    int limit;   // last key position the row may see (its own position); -1 = row unused
    int first;   // first key position (window), 0 without a window
};

struct TileState {
    float o[NTILES][4];   // [tile][c0,c1 (row g), c2,c3 (row g+8)]
    float m[2], l[2];     // running max (log2 domain) and lane-partial sum for rows g and g+8
};

__device__ __forceinline__ void tile_init(TileState& s) {
#pragma unroll
    for (int i = 0; i < NTILES; ++i) { s.o[i][0] = s.o[i][1] = s.o[i][2] = s.o[i][3] = 0.f; }
    s.m[0] = s.m[1] = -INFINITY;
    s.l[0] = s.l[1] = 0.f;
}

// Row offset (in elements) of key j of kv head hk in a layer's cache.  j is first brought into
// [j_min, j_max], the keys some row of the tile can see: keys outside are masked anyway, and their
// pages may already have gone back to the pool.  A bad page id is reported and replaced by page 0.
__device__ __forceinline__ int64_t key_row_offset(int j, int j_min, int j_max, const int* __restrict__ bt, int P,
                                                  int Hkv, int hk, int num_pages, int* status) {
    j = max(j_min, min(j, j_max));
    const int lp = j / P;
    int page = bt[lp];
    if (page < 0 || page >= num_pages) {
        imp_report(status, IMP_BAD_PAGE);
        page = 0;
    }
    return (((int64_t)page * Hkv + hk) * P + (j - lp * P)) * DH;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));   // ex2(-inf) = +0
    return y;
}

// ---- decode: 16 keys at a time, straight from the pages into fragments ------------------------------
// NR = 2: the tile's 16 rows are all in use (rows g and g+8 of every lane).  NR = 1: at most 8 query
// heads share the kv head, rows g+8 do not exist; their half of every fragment is zero and their half
// of the accumulator is not kept, which frees registers for more loads in flight.
template <int NR> struct DecState {
    float o[NTILES][2 * NR];
    float m[NR], l[NR];     // running max (scaled, log2 domain) and lane-partial sum
};
struct DecLoads {
    uint32_t kb0[KSTEPS][2], kb1[KSTEPS][2];   // key fragments of the two 8-key tiles
    int64_t v_off[4];                          // rows of keys 2t, 2t+1, 2t+8, 2t+9 in the value cache
};

// Look the 16 keys' rows up and request their key fragments (the loads stay in flight until used).
__device__ __forceinline__ void dec_fetch(DecLoads& L, const __nv_bfloat16* __restrict__ kc, const int* __restrict__ bt,
                                          int P, int Hkv, int hk, int num_pages, int j0, int j_min, int j_max, int lane,
                                          int* status) {
    const int g = lane >> 2, t = lane & 3;
    // Lanes 0..15 look up the row of key j0 + lane; the others copy what they need.
    const int64_t my_off = key_row_offset(j0 + (lane & 15), j_min, j_max, bt, P, Hkv, hk, num_pages, status);
    const int64_t k_off0 = __shfl_sync(0xffffffffu, my_off, g);
    const int64_t k_off1 = __shfl_sync(0xffffffffu, my_off, g + 8);
    L.v_off[0] = __shfl_sync(0xffffffffu, my_off, 2 * t);
    L.v_off[1] = __shfl_sync(0xffffffffu, my_off, 2 * t + 1);
    L.v_off[2] = __shfl_sync(0xffffffffu, my_off, 2 * t + 8);
    L.v_off[3] = __shfl_sync(0xffffffffu, my_off, 2 * t + 9);
    load_row_frags(L.kb0, kc + k_off0, t);
    load_row_frags(L.kb1, kc + k_off1, t);
}

template <int NR>
__device__ __forceinline__ void dec_mma(float (&acc)[2 * NR], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    if (NR == 2) {
        float c[4] = {acc[0], acc[1], acc[2 * NR - 2], acc[2 * NR - 1]};
        mma_16816(c, a0, a1, a2, a3, b0, b1);
        acc[0] = c[0]; acc[1] = c[1]; acc[2 * NR - 2] = c[2]; acc[2 * NR - 1] = c[3];
    } else {
        float c[4] = {acc[0], acc[1], 0.f, 0.f};
        mma_16816(c, a0, 0u, a2, 0u, b0, b1);
        acc[0] = c[0]; acc[1] = c[1];
    }
}

// Scores, softmax update and P V for the 16 keys j0 .. j0+15 whose loads `L` holds.
template <int NR>
__device__ __forceinline__ void dec_compute(DecState<NR>& st, const uint32_t (&qa)[KSTEPS][4], const RowInfo (&rows)[2],
                                            const DecLoads& L, const __nv_bfloat16* __restrict__ vc, int j0,
                                            float scale_log2, int lane) {
    const int g = lane >> 2, t = lane & 3;
    // the value rows are requested first: they travel while the scores are computed
    uint4 vr[VBlocks::N64 > 0 ? VBlocks::N64 : 1][4];
#pragma unroll
    for (int b = 0; b < VBlocks::N64; ++b)
#pragma unroll
        for (int k = 0; k < 4; ++k) vr[b][k] = *reinterpret_cast<const uint4*>(vc + L.v_off[k] + b * 64 + 8 * g);

    float s0[2 * NR], s1[2 * NR];
#pragma unroll
    for (int i = 0; i < 2 * NR; ++i) s0[i] = s1[i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        dec_mma<NR>(s0, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], L.kb0[ks][0], L.kb0[ks][1]);
        dec_mma<NR>(s1, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], L.kb1[ks][0], L.kb1[ks][1]);
    }
    uint32_t pa[2][NR];    // [8-key tile][row] packed probabilities of keys 2t, 2t+1
    float corr[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        float v[4] = {s0[2 * r] * scale_log2, s0[2 * r + 1] * scale_log2, s1[2 * r] * scale_log2, s1[2 * r + 1] * scale_log2};
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = j0 + 8 * (e >> 1) + 2 * t + (e & 1);
            if (j > rows[r].limit || j < rows[r].first) v[e] = -INFINITY;
            mx = fmaxf(mx, v[e]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(st.m[r], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        corr[r] = fast_exp2(st.m[r] - m_use);
        const float p0 = fast_exp2(v[0] - m_use), p1 = fast_exp2(v[1] - m_use);
        const float p2 = fast_exp2(v[2] - m_use), p3 = fast_exp2(v[3] - m_use);
        st.l[r] = st.l[r] * corr[r] + (p0 + p1) + (p2 + p3);
        st.m[r] = m_new;
        pa[0][r] = pack_bf16(p0, p1);
        pa[1][r] = pack_bf16(p2, p3);
    }
    bool rescale = corr[0] != 1.f;
    if (NR == 2) rescale = rescale || corr[NR - 1] != 1.f;
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int i = 0; i < NTILES; ++i)
#pragma unroll
            for (int c = 0; c < 2 * NR; ++c) st.o[i][c] *= corr[c >> 1];
    }
    const uint32_t pa0 = pa[0][0], pa2 = pa[1][0];
    const uint32_t pa1 = NR == 2 ? pa[0][NR - 1] : 0u, pa3 = NR == 2 ? pa[1][NR - 1] : 0u;
    int tile = 0;
#pragma unroll
    for (int b = 0; b < VBlocks::N64; ++b) {
        const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&vr[b][0]);
        const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&vr[b][1]);
        const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&vr[b][2]);
        const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&vr[b][3]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
            dec_mma<NR>(st.o[tile + i], pa0, pa1, pa2, pa3, __byte_perm(w0[i >> 1], w1[i >> 1], sel),
                        __byte_perm(w2[i >> 1], w3[i >> 1], sel));
        }
        tile += 8;
    }
    if (VBlocks::HAS32) {
        const int base = VBlocks::N64 * 64;
        uint2 r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) r[k] = *reinterpret_cast<const uint2*>(vc + L.v_off[k] + base + 4 * g);
        const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&r[0]);
        const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&r[1]);
        const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&r[2]);
        const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&r[3]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
            dec_mma<NR>(st.o[tile + i], pa0, pa1, pa2, pa3, __byte_perm(w0[i >> 1], w1[i >> 1], sel),
                        __byte_perm(w2[i >> 1], w3[i >> 1], sel));
        }
        tile += 4;
    }
    if (VBlocks::HAS16) {
        const int base = VBlocks::N64 * 64 + VBlocks::HAS32 * 32;
        uint32_t r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) r[k] = *reinterpret_cast<const uint32_t*>(vc + L.v_off[k] + base + 2 * g);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
            dec_mma<NR>(st.o[tile + i], pa0, pa1, pa2, pa3, __byte_perm(r[0], r[1], sel), __byte_perm(r[2], r[3], sel));
        }
    }
}

// ---------------------------------------------------------------------------- staging
// Row strides in shared memory.  Keys: lanes (g, t) read 16 bytes at row g, byte 16t of a 64-byte
// block, so consecutive rows must fall into the two halves of a 128-byte bank line: stride = 64
// (mod 128).  Values: lanes (g, t) read 16 bytes at rows 2t.., byte 16g of a 128-byte block, so rows
// two apart must be 32 bytes apart (mod 128): stride = 16 (mod 64).
constexpr int SK = DH * 2 + ((64 - (DH * 2) % 128) + 128) % 128;
constexpr int SV = DH * 2 + ((16 - (DH * 2) % 64) + 64) % 64;
static_assert(SK % 128 == 64 && SV % 64 == 16 && SK % 16 == 0 && SV % 16 == 0, "padding");
constexpr int CHUNKS_PER_ROW = DH / 8;   // 16-byte chunks of a key or value row

template <int KEYS> struct StageGeom {
    static constexpr int K_BYTES = KEYS * SK;
    static constexpr int BYTES = KEYS * (SK + SV);
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// All THREADS threads of the CTA copy keys and values j0 .. j0+KEYS-1 of kv head hk into one stage.
// Keys outside [j_min, j_max] (masked for every row of the CTA; their pages may be gone) become zeros.
// A bad page id is reported and the row zero-filled.
template <int KEYS, int THREADS>
__device__ __forceinline__ void load_stage(uint32_t stage_addr, const __nv_bfloat16* __restrict__ kc,
                                           const __nv_bfloat16* __restrict__ vc, const int* __restrict__ bt, int P,
                                           int Hkv, int hk, int num_pages, int j0, int j_min, int j_max, int tid,
                                           int* status) {
    constexpr int TOTAL = 2 * KEYS * CHUNKS_PER_ROW;
#pragma unroll
    for (int c0 = 0; c0 < TOTAL; c0 += THREADS) {
        const int c = c0 + tid;
        if (TOTAL % THREADS != 0 && c >= TOTAL) break;
        const bool is_v = c >= KEYS * CHUNKS_PER_ROW;
        const int cc = is_v ? c - KEYS * CHUNKS_PER_ROW : c;
        const int row = cc / CHUNKS_PER_ROW, col = cc - row * CHUNKS_PER_ROW;
        const int j = j0 + row;
        bool ok = j >= j_min && j <= j_max;
        int64_t off = 0;
        if (ok) {
            const int lp = j / P;
            const int page = bt[lp];
            if (page < 0 || page >= num_pages) {
                imp_report(status, IMP_BAD_PAGE);
                ok = false;
            } else {
                off = (((int64_t)page * Hkv + hk) * P + (j - lp * P)) * DH;
            }
        }
        const uint32_t dst = stage_addr + (is_v ? KEYS * SK + row * SV : row * SK) + col * 16;
        cp_async16(dst, (is_v ? vc : kc) + off + col * 8, ok ? 16 : 0);
    }
}

// Fragments of one key row from shared memory (same permutation as load_row_frags).
__device__ __forceinline__ void load_k_frags(uint32_t (&f)[KSTEPS][2], const unsigned char* row, int t) {
#pragma unroll
    for (int b = 0; b < DH / 32; ++b) {
        const uint4 v = *reinterpret_cast<const uint4*>(row + b * 64 + 16 * t);
        f[2 * b][0] = v.x; f[2 * b][1] = v.y; f[2 * b + 1][0] = v.z; f[2 * b + 1][1] = v.w;
    }
    if (DH % 32) {
        const uint2 v = *reinterpret_cast<const uint2*>(row + (DH / 32) * 64 + 8 * t);
        f[KSTEPS - 1][0] = v.x; f[KSTEPS - 1][1] = v.y;
    }
}


// Process the 32 keys j0 .. j0+31, staged at rows 0 .. 31 of a stage, for a 16-row tile: scores
// of all 32 keys first, one softmax update (one rescale of the accumulator), then two P V steps.
// Scores stay unscaled; the scale (times log2 e) enters as the factor of a fused multiply-add in
// front of ex2.  `need_mask` (warp-uniform) is false when every key is visible to every row.
__device__ __forceinline__ void process_stage32(TileState& st, const uint32_t (&qa)[KSTEPS][4], const RowInfo (&rows)[2],
                                                const unsigned char* __restrict__ ksm, const unsigned char* __restrict__ vsm,
                                                int j0, float scale_log2, bool need_mask, int lane) {
    const int g = lane >> 2, t = lane & 3;
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    // The four 8-key tiles are independent accumulation chains: walk the head dimension in the outer
    // loop so that consecutive MMAs never wait for one another.
#pragma unroll
    for (int b = 0; b < DH / 32; ++b) {
        uint4 v[4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) v[nt] = *reinterpret_cast<const uint4*>(ksm + (8 * nt + g) * SK + b * 64 + 16 * t);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
            mma_16816(s[nt], qa[2 * b][0], qa[2 * b][1], qa[2 * b][2], qa[2 * b][3], v[nt].x, v[nt].y);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
            mma_16816(s[nt], qa[2 * b + 1][0], qa[2 * b + 1][1], qa[2 * b + 1][2], qa[2 * b + 1][3], v[nt].z, v[nt].w);
    }
    if (DH % 32) {
        uint2 v[4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) v[nt] = *reinterpret_cast<const uint2*>(ksm + (8 * nt + g) * SK + (DH / 32) * 64 + 8 * t);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
            mma_16816(s[nt], qa[KSTEPS - 1][0], qa[KSTEPS - 1][1], qa[KSTEPS - 1][2], qa[KSTEPS - 1][3], v[nt].x, v[nt].y);
    }
    if (need_mask) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = j0 + 8 * nt + 2 * t + e;
                    if (j > rows[r].limit || j < rows[r].first) s[nt][2 * r + e] = -INFINITY;
                }
    }
    float corr[2];
    uint32_t pa[4][2];   // [n-tile][row g / row g+8] packed probabilities of keys 2t, 2t+1 of the tile
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(st.m[r], mx);                     // unscaled running max
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;    // a row with nothing to see yet
        const float neg = -m_use * scale_log2;
        corr[r] = fast_exp2(fmaf(st.m[r], scale_log2, neg));      // st.m = -inf -> 0
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float p0 = fast_exp2(fmaf(s[nt][2 * r], scale_log2, neg));
            const float p1 = fast_exp2(fmaf(s[nt][2 * r + 1], scale_log2, neg));
            sum += p0 + p1;
            pa[nt][r] = pack_bf16(p0, p1);
        }
        st.l[r] = st.l[r] * corr[r] + sum;
        st.m[r] = m_new;
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // the maxima seldom move after the first tiles
#pragma unroll
        for (int i = 0; i < NTILES; ++i) {
            st.o[i][0] *= corr[0]; st.o[i][1] *= corr[0];
            st.o[i][2] *= corr[1]; st.o[i][3] *= corr[1];
        }
    }
    // ---- O += P V, 16 keys at a time ---------------------------------------------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t pa0 = pa[2 * h][0], pa1 = pa[2 * h][1], pa2 = pa[2 * h + 1][0], pa3 = pa[2 * h + 1][1];
        const int r0 = 16 * h;
        const unsigned char* vr[4] = {vsm + (r0 + 2 * t) * SV, vsm + (r0 + 2 * t + 1) * SV, vsm + (r0 + 2 * t + 8) * SV,
                                      vsm + (r0 + 2 * t + 9) * SV};
        int tile = 0;
#pragma unroll
        for (int b = 0; b < VBlocks::N64; ++b) {
            uint4 r[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) r[k] = *reinterpret_cast<const uint4*>(vr[k] + b * 128 + 16 * g);
            const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&r[0]);
            const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&r[1]);
            const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&r[2]);
            const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&r[3]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
                mma_16816(st.o[tile + i], pa0, pa1, pa2, pa3, __byte_perm(w0[i >> 1], w1[i >> 1], sel),
                          __byte_perm(w2[i >> 1], w3[i >> 1], sel));
            }
            tile += 8;
        }
        if (VBlocks::HAS32) {
            const int base = VBlocks::N64 * 128;
            uint2 r[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) r[k] = *reinterpret_cast<const uint2*>(vr[k] + base + 8 * g);
            const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&r[0]);
            const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&r[1]);
            const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&r[2]);
            const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&r[3]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
                mma_16816(st.o[tile + i], pa0, pa1, pa2, pa3, __byte_perm(w0[i >> 1], w1[i >> 1], sel),
                          __byte_perm(w2[i >> 1], w3[i >> 1], sel));
            }
            tile += 4;
        }
        if (VBlocks::HAS16) {
            const int base = VBlocks::N64 * 128 + VBlocks::HAS32 * 64;
            uint32_t r[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) r[k] = *reinterpret_cast<const uint32_t*>(vr[k] + base + 4 * g);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
                mma_16816(st.o[tile + i], pa0, pa1, pa2, pa3, __byte_perm(r[0], r[1], sel), __byte_perm(r[2], r[3], sel));
            }
        }
    }
}

// Dimension held by accumulator (tile, column c) -- the inverse of the value-column permutation.
__device__ __forceinline__ int dim_of(int tile, int c) {
    if (tile < VBlocks::N64 * 8) return (tile >> 3) * 64 + 8 * c + (tile & 7);
    tile -= VBlocks::N64 * 8;
    int base = VBlocks::N64 * 64;
    if (VBlocks::HAS32) {
        if (tile < 4) return base + 4 * c + tile;
        tile -= 4;
        base += 32;
    }
    return base + 2 * c + tile;
}

// Query fragments of rows g and g+8 (null pointer = unused row -> zeros).
__device__ __forceinline__ void load_q(uint32_t (&qa)[KSTEPS][4], const __nv_bfloat16* q0, const __nv_bfloat16* q1, int t) {
    uint32_t f0[KSTEPS][2], f1[KSTEPS][2];
    if (q0) load_row_frags(f0, q0, t);
    if (q1) load_row_frags(f1, q1, t);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        qa[ks][0] = q0 ? f0[ks][0] : 0u;   // row g,   k = 2t, 2t+1
        qa[ks][1] = q1 ? f1[ks][0] : 0u;   // row g+8, k = 2t, 2t+1
        qa[ks][2] = q0 ? f0[ks][1] : 0u;   // row g,   k = 2t+8, 2t+9
        qa[ks][3] = q1 ? f1[ks][1] : 0u;   // row g+8
    }
}

// ================================================================================== decode
// grid (n_splits, Hkv * tiles_per_group, n_tokens), block 128.  Each warp takes every fourth 16-key
// step of the CTA's split; several CTAs per SM keep enough loads in flight.
// part_o: [n_tokens, Hq, n_splits, DH] float, part_ml: [n_tokens, Hq, n_splits, 2] float (used when n_splits > 1).
template <int NR>
__global__ void __launch_bounds__(WARPS * 32, NR == 1 ? 4 : 2) attn_decode_kernel(
    __nv_bfloat16* __restrict__ out, int64_t out_stride, const __nv_bfloat16* __restrict__ q, int64_t q_stride,
    const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ seq_of_token, const int* __restrict__ positions, int n_seqs, int Hq,
    int Hkv, int P, int num_pages, float scale_log2, int window, int n_splits, float* __restrict__ part_o,
    float* __restrict__ part_ml, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float smem[];   // (WARPS-1) x (NTILES*2*NR + 2*NR) x 32 floats
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int G = Hq / Hkv;
    const int tiles_per_group = (G + 15) / 16;
    const int split = blockIdx.x;
    const int hk = blockIdx.y / tiles_per_group;
    const int row0 = (blockIdx.y % tiles_per_group) * 16;   // first head of the group in this tile
    const int tok = blockIdx.z;
    const int seq = seq_of_token[tok];
    const int pos = positions[tok];
    if (seq < 0 || seq >= n_seqs || pos < 0 || pos / P >= bt_stride) {
        if (threadIdx.x == 0) imp_report(status, seq < 0 || seq >= n_seqs ? IMP_TAGGED(IMP_BAD_SEQUENCE, 1) : IMP_TAGGED(IMP_BAD_POSITION, 1));
        return;
    }
    const int* bt = block_table + (int64_t)seq * bt_stride;
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first16 = first & ~15;
    const int total_steps = (pos - first16) / 16 + 1;
    // balanced ranges: every split gets floor or ceil of total / n_splits steps, none is left empty while others hold two
    const int step_lo = (int)((int64_t)split * total_steps / n_splits);
    const int step_hi = (int)((int64_t)(split + 1) * total_steps / n_splits);

    RowInfo rows[2];
    const __nv_bfloat16* qrow[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int hr = row0 + g + 8 * r;
        const bool used = r < NR && hr < G;
        rows[r].limit = used ? pos : -1;
        rows[r].first = first;
        qrow[r] = used ? q + (int64_t)tok * q_stride + (int64_t)(hk * G + hr) * DH : nullptr;
    }
    int s = step_lo + warp;
    uint32_t qa[KSTEPS][4];
    load_q(qa, qrow[0], qrow[1], t4);
    DecState<NR> st;
#pragma unroll
    for (int i = 0; i < NTILES; ++i)
#pragma unroll
        for (int c = 0; c < 2 * NR; ++c) st.o[i][c] = 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) { st.m[r] = -INFINITY; st.l[r] = 0.f; }
    for (; s < step_hi; s += WARPS) {
        DecLoads cur;
        dec_fetch(cur, kc, bt, P, Hkv, hk, num_pages, first16 + 16 * s, first, pos, lane, status);
        dec_compute<NR>(st, qa, rows, cur, vc, first16 + 16 * s, scale_log2, lane);
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
    // ---- merge the four warps (fragment-wise, through shared memory) ---------------------------------
    constexpr int NACC = NTILES * 2 * NR;
    constexpr int PER_WARP = NACC + 2 * NR;
    if (warp > 0) {
        float* dst = smem + (size_t)(warp - 1) * PER_WARP * 32;
#pragma unroll
        for (int i = 0; i < NTILES; ++i)
#pragma unroll
            for (int c = 0; c < 2 * NR; ++c) dst[(i * 2 * NR + c) * 32 + lane] = st.o[i][c];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            dst[(NACC + r) * 32 + lane] = st.m[r];
            dst[(NACC + NR + r) * 32 + lane] = st.l[r];
        }
    }
    __syncthreads();
    if (warp != 0) return;
    for (int w = 1; w < WARPS; ++w) {
        const float* src = smem + (size_t)(w - 1) * PER_WARP * 32;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const float mo = src[(NACC + r) * 32 + lane];
            const float lo = src[(NACC + NR + r) * 32 + lane];
            const float m_new = fmaxf(st.m[r], mo);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float ca = exp2f(st.m[r] - m_use), cb = exp2f(mo - m_use);
            st.l[r] = st.l[r] * ca + lo * cb;
            st.m[r] = m_new;
#pragma unroll
            for (int i = 0; i < NTILES; ++i) {
                st.o[i][2 * r] = st.o[i][2 * r] * ca + src[(i * 2 * NR + 2 * r) * 32 + lane] * cb;
                st.o[i][2 * r + 1] = st.o[i][2 * r + 1] * ca + src[(i * 2 * NR + 2 * r + 1) * 32 + lane] * cb;
            }
        }
    }
    // ---- write: final output, or this split's partial ---------------------------------------------
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int hr = row0 + g + 8 * r;
        if (hr >= G) continue;
        const int head = hk * G + hr;
        if (n_splits == 1) {
            const float inv = st.l[r] > 0.f ? 1.f / st.l[r] : 0.f;
            __nv_bfloat16* o = out + (int64_t)tok * out_stride + (int64_t)head * DH;
#pragma unroll
            for (int i = 0; i < NTILES; ++i) {
                o[dim_of(i, 2 * t4)] = __float2bfloat16_rn(st.o[i][2 * r] * inv);
                o[dim_of(i, 2 * t4 + 1)] = __float2bfloat16_rn(st.o[i][2 * r + 1] * inv);
            }
        } else {
            const int64_t slot = ((int64_t)tok * Hq + head) * n_splits + split;
            float* o = part_o + slot * DH;
#pragma unroll
            for (int i = 0; i < NTILES; ++i) {
                o[dim_of(i, 2 * t4)] = st.o[i][2 * r];
                o[dim_of(i, 2 * t4 + 1)] = st.o[i][2 * r + 1];
            }
            if (t4 == 0) {
                part_ml[slot * 2] = st.m[r];
                part_ml[slot * 2 + 1] = st.l[r];
            }
        }
    }
}

// One block per (token, head): out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
// Warp 0 turns the splits' (m, l) into weights in shared memory; then every thread sums its
// dimensions over the splits in split order with independent loads.
constexpr int MERGE_MAX_SPLITS = 256;

__global__ void __launch_bounds__(128) attn_merge_kernel(__nv_bfloat16* __restrict__ out, int64_t out_stride,
                                                         const float* __restrict__ part_o,
                                                         const float* __restrict__ part_ml, int Hq, int n_splits) {
    IMP_TL_BEGIN(7)
    pdl_wait();
    IMP_TL_WAITED()
    pdl_launch_dependents();
    __shared__ float w_s[MERGE_MAX_SPLITS];
    __shared__ float inv_s;
    const int unit = blockIdx.x;
    const int tok = unit / Hq, head = unit - tok * Hq;
    const float* ml = part_ml + (int64_t)unit * n_splits * 2;
    const float* po = part_o + (int64_t)unit * n_splits * DH;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float M = -INFINITY;
        for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, ml[2 * s]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float L = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 32) {        // fixed order: chunks of 32 splits, tree inside a chunk
            const int s = s0 + lane;
            float w = 0.f, l = 0.f;
            if (s < n_splits) {
                const float m = ml[2 * s];
                w = (m == -INFINITY) ? 0.f : exp2f(m - M);
                l = ml[2 * s + 1] * w;
                w_s[s] = w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            L += l;
        }
        if (lane == 0) inv_s = L > 0.f ? 1.f / L : 0.f;
    }
    // The partial outputs do not depend on the weights: every thread asks for its dimension of the first 32 splits
    // before the barrier, so that they arrive while warp 0 works; further chunks (and dimensions) follow in the loop.
    constexpr int MB = 32;
    float v[MB];
    if (threadIdx.x < DH) {
#pragma unroll
        for (int j = 0; j < MB; ++j)
            if (j < n_splits) v[j] = po[(int64_t)j * DH + threadIdx.x];
    }
    __syncthreads();
    const float inv = inv_s;
    __nv_bfloat16* o = out + (int64_t)tok * out_stride + (int64_t)head * DH;
    for (int d = threadIdx.x; d < DH; d += 128) {
        float acc = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += MB) {          // split order
            if (s0 > 0 || d != (int)threadIdx.x) {
#pragma unroll
                for (int j = 0; j < MB; ++j)
                    if (s0 + j < n_splits) v[j] = po[(int64_t)(s0 + j) * DH + d];
            }
#pragma unroll
            for (int j = 0; j < MB; ++j)
                if (s0 + j < n_splits) acc += v[j] * w_s[s0 + j];
        }
        o[d] = __float2bfloat16_rn(acc * inv);
    }
    IMP_TL_END()
}

static int check_common(const void* out, const void* q, const void* kc, const void* vc, const int* bt,
                        int64_t out_stride, int64_t q_stride, int Hq, int Hkv, int P, int num_pages) {
    IMP_CHECK_ARG(out && q && kc && vc && bt, "attention: null pointer");
    IMP_CHECK_ARG(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: %d query heads are not a multiple of %d kv heads", Hq, Hkv);
    IMP_CHECK_ARG(P > 0 && num_pages > 0, "attention: bad cache geometry");
    IMP_CHECK_ARG(q_stride % 8 == 0 && out_stride % 2 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)kc % 16 == 0 &&
                      (uintptr_t)vc % 16 == 0,
                  "attention: q, k and v rows must start on 16-byte boundaries");
    IMP_CHECK_ARG((int64_t)num_pages * Hkv * P * DH < ((int64_t)1 << 40), "attention: cache too large");
    return 0;
}

IMP_API int imp_attn_head_dim(void) { return DH; }

// Scratch floats needed by imp_attn_decode for n_splits > 1: part_o then part_ml.
IMP_API int64_t imp_attn_decode_scratch_floats(int n_tokens, int Hq, int n_splits) {
    return n_splits > 1 ? (int64_t)n_tokens * Hq * n_splits * (DH + 2) : 0;
}

// ------------------------------------------------------------------ decode, bulk-copy ring
// The same split-key decode for page sizes that are multiples of 16: the 16 keys of a step then lie
// in one page, 16 consecutive rows of a kv head = one contiguous run of 32*DH bytes for keys and one
// for values.  A fifth warp is the producer: per stage of 64 keys its lanes 0..7 issue one cp.async.bulk
// copy each (global -> shared, completion counted in bytes on the stage's mbarrier; keys and values of
// the four steps, fewer and larger copies where 2 or 4 steps share a page) into a three-deep ring; the
// page ids come from one coalesced read of the block table per eight stages, one id a lane.  The four
// consumer warps each take one 16-key step of the stage from shared memory and hand the stage back
// through a second mbarrier.  A CTA so keeps two stages (up to 64 x DH x 4 bytes each) in flight without
// holding them in registers.  Measured: the copies of a stage issued by one thread, and that thread
// reading the block table stage by stage, held a CTA to about 19 GB/s whatever the ring's depth (4.7-5.0
// TB/s for the device at two CTAs per SM); issued side by side the same ring reaches 6.1-6.7 TB/s.  Copies
// cost per piece, not per byte: 32 copies of 1 KB a stage were as slow as the single thread.  Every wait
// is bounded (IMP_WAIT_TIMEOUT in the status word, then the CTA drains and leaves).
#ifndef IMP_DT_STAGES
#define IMP_DT_STAGES 3
#endif
constexpr int DT_KEYS = 64, DT_STAGES = IMP_DT_STAGES, DT_CONSUMERS = 4;
constexpr int DT_RUN_BYTES = 16 * DH * 2;                 // keys (or values) of one step
constexpr int DT_STAGE_BYTES = 2 * DT_CONSUMERS * DT_RUN_BYTES;
constexpr uint32_t DT_WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ bool dt_wait(uint32_t bar, uint32_t parity, int* status) {
    for (uint32_t i = 0; i < DT_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    imp_report(status, IMP_WAIT_TIMEOUT);
    return false;
}

// Scores, softmax update and P V for 16 keys whose rows lie at `ksm` / `vsm` (16 rows of DH bfloat16).
template <int NR>
__device__ __forceinline__ void dec_compute_smem(DecState<NR>& st, const uint32_t (&qa)[KSTEPS][4], const RowInfo (&rows)[2],
                                                 const unsigned char* __restrict__ ksm, const unsigned char* __restrict__ vsm,
                                                 int j0, float scale_log2, int lane) {
    const int g = lane >> 2, t = lane & 3;
    constexpr int RB = DH * 2;   // bytes per row
    float s0[2 * NR], s1[2 * NR];
#pragma unroll
    for (int i = 0; i < 2 * NR; ++i) s0[i] = s1[i] = 0.f;
    {
        uint32_t k0[KSTEPS][2], k1[KSTEPS][2];
        load_row_frags(k0, reinterpret_cast<const __nv_bfloat16*>(ksm + g * RB), t);
        load_row_frags(k1, reinterpret_cast<const __nv_bfloat16*>(ksm + (g + 8) * RB), t);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            dec_mma<NR>(s0, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], k0[ks][0], k0[ks][1]);
            dec_mma<NR>(s1, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], k1[ks][0], k1[ks][1]);
        }
    }
    uint32_t pa[2][NR];
    float corr[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        float v[4] = {s0[2 * r] * scale_log2, s0[2 * r + 1] * scale_log2, s1[2 * r] * scale_log2, s1[2 * r + 1] * scale_log2};
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = j0 + 8 * (e >> 1) + 2 * t + (e & 1);
            if (j > rows[r].limit || j < rows[r].first) v[e] = -INFINITY;
            mx = fmaxf(mx, v[e]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(st.m[r], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        corr[r] = fast_exp2(st.m[r] - m_use);
        const float p0 = fast_exp2(v[0] - m_use), p1 = fast_exp2(v[1] - m_use);
        const float p2 = fast_exp2(v[2] - m_use), p3 = fast_exp2(v[3] - m_use);
        st.l[r] = st.l[r] * corr[r] + (p0 + p1) + (p2 + p3);
        st.m[r] = m_new;
        pa[0][r] = pack_bf16(p0, p1);
        pa[1][r] = pack_bf16(p2, p3);
    }
    bool rescale = corr[0] != 1.f;
    if (NR == 2) rescale = rescale || corr[NR - 1] != 1.f;
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int i = 0; i < NTILES; ++i)
#pragma unroll
            for (int c = 0; c < 2 * NR; ++c) st.o[i][c] *= corr[c >> 1];
    }
    const uint32_t pa0 = pa[0][0], pa2 = pa[1][0];
    const uint32_t pa1 = NR == 2 ? pa[0][NR - 1] : 0u, pa3 = NR == 2 ? pa[1][NR - 1] : 0u;
    const unsigned char* vr[4] = {vsm + (2 * t) * RB, vsm + (2 * t + 1) * RB, vsm + (2 * t + 8) * RB, vsm + (2 * t + 9) * RB};
    int tile = 0;
#pragma unroll
    for (int b = 0; b < VBlocks::N64; ++b) {
        uint4 r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) r[k] = *reinterpret_cast<const uint4*>(vr[k] + b * 128 + 16 * g);
        const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&r[0]);
        const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&r[1]);
        const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&r[2]);
        const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&r[3]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
            dec_mma<NR>(st.o[tile + i], pa0, pa1, pa2, pa3, __byte_perm(w0[i >> 1], w1[i >> 1], sel),
                        __byte_perm(w2[i >> 1], w3[i >> 1], sel));
        }
        tile += 8;
    }
    if (VBlocks::HAS32) {
        const int base = VBlocks::N64 * 128;
        uint2 r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) r[k] = *reinterpret_cast<const uint2*>(vr[k] + base + 8 * g);
        const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&r[0]);
        const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&r[1]);
        const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&r[2]);
        const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&r[3]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
            dec_mma<NR>(st.o[tile + i], pa0, pa1, pa2, pa3, __byte_perm(w0[i >> 1], w1[i >> 1], sel),
                        __byte_perm(w2[i >> 1], w3[i >> 1], sel));
        }
        tile += 4;
    }
    if (VBlocks::HAS16) {
        const int base = VBlocks::N64 * 128 + VBlocks::HAS32 * 64;
        uint32_t r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) r[k] = *reinterpret_cast<const uint32_t*>(vr[k] + base + 4 * g);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
            dec_mma<NR>(st.o[tile + i], pa0, pa1, pa2, pa3, __byte_perm(r[0], r[1], sel), __byte_perm(r[2], r[3], sel));
        }
    }
}

// The decode step straight from the projection: with `qkv` set, q is read raw from the fused q|k|v rows
// (q heads first, then k heads, then v heads) and normalised and rotated here, and the CTA whose keys include
// the token's own position does the same for the new key, writes key and value into their page and into its
// own copy of the page in shared memory (the producer fetched that row as it was).  This is the work of the
// rotary kernel (csrc/rope_kv.cu, same formulas and roundings), saved as a launch.  Head sizes that are
// multiples of 64, rotated over their whole width: a lane then holds both elements of every rotary pair.
struct DecFused {
    const __nv_bfloat16* qkv;      // null: q is ready and the pages hold this step's key and value
    int64_t stride;                // elements between rows of qkv
    const float* q_norm_w;         // [DH] or null
    const float* k_norm_w;
    const float* cos_tab;          // [max_pos, DH / 2]
    const float* sin_tab;
    __nv_bfloat16* k_pages;        // the caches again, to write
    __nv_bfloat16* v_pages;
    float eps;
    int max_pos;
};

__device__ __forceinline__ float2 unpack_bf16(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}

// Query fragments (see load_row_frags for which dimensions a lane holds): per-head RMSNorm, then rotation of the
// pairs (d, d + DH/2).  k-step ks < KSTEPS/2 holds d = 32 (ks / 2) + 8 t + 4 (ks % 2) + {0,1} and {2,3}; its
// partner is k-step ks + KSTEPS/2.  The four lanes t of a row share the sum of squares.
template <int NR>
__device__ __forceinline__ void dec_q_norm_rope(uint32_t (&qa)[KSTEPS][4], const DecFused& fz, int pos, int t) {
    constexpr int HALF = DH / 2, HK = KSTEPS / 2;
    const float* cs = fz.cos_tab + (int64_t)pos * HALF;
    const float* sn = fz.sin_tab + (int64_t)pos * HALF;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        float ss = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float2 v = unpack_bf16(qa[ks][2 * j + r]);
                ss += v.x * v.x + v.y * v.y;
            }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        const float inv = fz.q_norm_w ? rsqrtf(ss / (float)DH + fz.eps) : 1.f;
#pragma unroll
        for (int ks = 0; ks < HK; ++ks)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int d = 32 * (ks >> 1) + 8 * t + 4 * (ks & 1) + 2 * j;
                float2 a = unpack_bf16(qa[ks][2 * j + r]), b = unpack_bf16(qa[ks + HK][2 * j + r]);
                a.x *= inv; a.y *= inv; b.x *= inv; b.y *= inv;
                if (fz.q_norm_w) {
                    a.x *= fz.q_norm_w[d]; a.y *= fz.q_norm_w[d + 1];
                    b.x *= fz.q_norm_w[d + HALF]; b.y *= fz.q_norm_w[d + 1 + HALF];
                }
                const float2 c = *reinterpret_cast<const float2*>(cs + d), sv = *reinterpret_cast<const float2*>(sn + d);
                qa[ks][2 * j + r] = pack_bf16(a.x * c.x - b.x * sv.x, a.y * c.y - b.y * sv.y);
                qa[ks + HK][2 * j + r] = pack_bf16(a.x * sv.x + b.x * c.x, a.y * sv.y + b.y * c.y);
            }
    }
}

// The token's own key and value: k normalised and rotated, both written to row `pos` of their page at once (dec_make_own_key,
// before the warp's loop over the stages, so that the trip for the raw rows runs beside the one for q) and, once the
// stage that holds the row has landed, to the rows `ksm_row` / `vsm_row` of this warp's copy of the page in shared memory
// (dec_patch_own_key; the producer fetched that row as it was).  One warp; lane l holds the pairs (2l, 2l+1) of both rotary
// halves (and the next 64 dimensions for head sizes above 128), as the rotary kernel does.
struct OwnKey {
    uint32_t lo[2], hi[2];     // rotated key: first and second half of the head, pairs lane and lane + 32
    uint2 v[2];                // value: dimensions 4 lane .. 4 lane + 3, and the same 128 further on
};

__device__ __forceinline__ void dec_make_own_key(OwnKey& own, const DecFused& fz, const __nv_bfloat16* __restrict__ kraw,
                                                 const __nv_bfloat16* __restrict__ vraw, int64_t page_row_off, int pos, int lane) {
    constexpr int HALF = DH / 2;
    const float* cs = fz.cos_tab + (int64_t)pos * HALF;
    const float* sn = fz.sin_tab + (int64_t)pos * HALF;
    float2 a[2], b[2];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int j = lane + 32 * r;
        a[r] = b[r] = make_float2(0.f, 0.f);
        if (2 * j < HALF) {
            a[r] = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(kraw)[j]);
            b[r] = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(kraw + HALF)[j]);
            ss += a[r].x * a[r].x + a[r].y * a[r].y + b[r].x * b[r].x + b[r].y * b[r].y;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = lane * 4 + 128 * r;
        own.v[r] = i < DH ? *reinterpret_cast<const uint2*>(vraw + i) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = fz.k_norm_w ? rsqrtf(ss / (float)DH + fz.eps) : 1.f;
    __nv_bfloat16* kdst = fz.k_pages + page_row_off;
    __nv_bfloat16* vdst = fz.v_pages + page_row_off;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int j = lane + 32 * r;
        own.lo[r] = own.hi[r] = 0u;
        if (2 * j >= HALF) continue;
        float2 av = make_float2(a[r].x * inv, a[r].y * inv), bv = make_float2(b[r].x * inv, b[r].y * inv);
        if (fz.k_norm_w) {
            av.x *= fz.k_norm_w[2 * j]; av.y *= fz.k_norm_w[2 * j + 1];
            bv.x *= fz.k_norm_w[2 * j + HALF]; bv.y *= fz.k_norm_w[2 * j + 1 + HALF];
        }
        const float2 c = *reinterpret_cast<const float2*>(cs + 2 * j), sv = *reinterpret_cast<const float2*>(sn + 2 * j);
        own.lo[r] = pack_bf16(av.x * c.x - bv.x * sv.x, av.y * c.y - bv.y * sv.y);
        own.hi[r] = pack_bf16(av.x * sv.x + bv.x * c.x, av.y * sv.y + bv.y * c.y);
        reinterpret_cast<uint32_t*>(kdst)[j] = own.lo[r];
        reinterpret_cast<uint32_t*>(kdst + HALF)[j] = own.hi[r];
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = lane * 4 + 128 * r;
        if (i < DH) *reinterpret_cast<uint2*>(vdst + i) = own.v[r];
    }
}

__device__ __forceinline__ void dec_patch_own_key(const OwnKey& own, unsigned char* ksm_row, unsigned char* vsm_row, int lane) {
    constexpr int HALF = DH / 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int j = lane + 32 * r;
        if (2 * j < HALF) {
            reinterpret_cast<uint32_t*>(ksm_row)[j] = own.lo[r];
            reinterpret_cast<uint32_t*>(ksm_row + HALF * 2)[j] = own.hi[r];
        }
        const int i = lane * 4 + 128 * r;
        if (i < DH) *reinterpret_cast<uint2*>(vsm_row + 2 * i) = own.v[r];
    }
    // the slot is refilled by a bulk copy later: order these ordinary stores before it
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
}

template <int NR>
__global__ void __launch_bounds__((DT_CONSUMERS + 1) * 32) attn_decode_tma_kernel(
    __nv_bfloat16* __restrict__ out, int64_t out_stride, const __nv_bfloat16* __restrict__ q, int64_t q_stride,
    const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ seq_of_token, const int* __restrict__ positions, int n_seqs, int Hq,
    int Hkv, int P, int num_pages, float scale_log2, int window, int n_splits, float* __restrict__ part_o,
    float* __restrict__ part_ml, int* status, const DecFused fz, int cluster_merge) {
    // cluster_merge: the CTAs of the key splits of one (token, kv head) form a cluster (grid.x == cluster size) and
    // merge their results in the first CTA's shared memory: no partial results in global memory, no merge kernel.
    // pdl_wait() comes later: the batch arrays and the keys before this step's position do not depend on the
    // kernel before this one, so the first stages are requested while it still runs.
    IMP_TL_BEGIN(3)
    extern __shared__ __align__(128) unsigned char dt_smem[];
    __shared__ __align__(8) uint64_t dt_bars[2 * DT_STAGES];     // [0,S) full, [S,2S) empty
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int G = Hq / Hkv;
    const int tiles_per_group = (G + 15) / 16;
    const int split = blockIdx.x;
    const int hk = blockIdx.y / tiles_per_group;
    const int row0 = (blockIdx.y % tiles_per_group) * 16;
    const int tok = blockIdx.z;
    const int seq = seq_of_token[tok];
    const int pos = positions[tok];
    if (seq < 0 || seq >= n_seqs || pos < 0 || pos / P >= bt_stride || (fz.qkv && pos >= fz.max_pos)) {
        if (tid == 0) imp_report(status, seq < 0 || seq >= n_seqs ? IMP_TAGGED(IMP_BAD_SEQUENCE, 2) : IMP_TAGGED(IMP_BAD_POSITION, 2));
        return;
    }
    const int* bt = block_table + (int64_t)seq * bt_stride;
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first_al = first & ~(DT_KEYS - 1);
    const int total_stages = (pos - first_al) / DT_KEYS + 1;
    // balanced ranges: every split gets floor or ceil of total / n_splits stages
    const int stage_lo = (int)((int64_t)split * total_stages / n_splits);
    const int stage_hi = (int)((int64_t)(split + 1) * total_stages / n_splits);
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dt_smem);
    const uint32_t full0 = (uint32_t)__cvta_generic_to_shared(dt_bars), empty0 = full0 + 8 * DT_STAGES;
    if (tid == 0) {
        for (int i = 0; i < DT_STAGES; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full0 + 8 * i), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty0 + 8 * i), "r"(DT_CONSUMERS) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    DecState<NR> st;
#pragma unroll
    for (int i = 0; i < NTILES; ++i)
#pragma unroll
        for (int c = 0; c < 2 * NR; ++c) st.o[i][c] = 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) { st.m[r] = -INFINITY; st.l[r] = 0.f; }

    if (warp == DT_CONSUMERS) {
        // ---------------------------------------------------------------------- producer
        // The whole warp runs the loop: every lane keeps the page id of one 16-key step (32 steps = 8 stages,
        // one coalesced read of the block table), lane 0 waits for the slot, lanes 0..7 issue.
        constexpr int STAGES_PER_FILL = 32 / DT_CONSUMERS;
        static_assert(DT_CONSUMERS == 4, "the grouping of steps into copies assumes four steps a stage");
        // steps of a stage that one copy may cover: the 64 keys of a stage start at a multiple of 64
        const int run_steps = P % 64 == 0 ? 4 : (P % 32 == 0 ? 2 : 1);
        bool ok = true;
        int issued = 0;
        int page_reg = -1, fill_base = -(1 << 30);
        auto issue_stage = [&](int s) {
            if (s < fill_base || s >= fill_base + STAGES_PER_FILL) {
                const int j0 = first_al + DT_KEYS * s + 16 * lane;
                page_reg = (j0 <= pos && j0 + 15 >= first) ? bt[j0 / P] : -1;    // pos / P < bt_stride was checked above
                fill_base = s;
            }
            // Lane kind * C + step requests the keys (kind 0) or values (kind 1) of one step, so that a stage's copies
            // go out together: one thread issuing them one after the other held a CTA to about 20 GB/s.  Where the page
            // size allows, 2 or 4 steps that lie in one page travel as one copy (copies cost per piece, not per byte).
            const int it = s - stage_lo, slot = it % DT_STAGES;
            const int w = lane % DT_CONSUMERS;
            const int j0 = first_al + DT_KEYS * s + 16 * w;
            const int page = __shfl_sync(0xffffffffu, page_reg, (s - fill_base) * DT_CONSUMERS + w);
            const bool wanted = j0 <= pos && j0 + 15 >= first;          // else every key of the step is masked: not fetched
            const bool good = wanted && page >= 0 && page < num_pages;
            if (wanted && !good && lane < DT_CONSUMERS) imp_report(status, IMP_BAD_PAGE);
            const uint32_t steps = __ballot_sync(0xffffffffu, good) & ((1u << DT_CONSUMERS) - 1u);
            // the steps of this lane's group (run_steps consecutive steps in one page) that are fetched
            const uint32_t group = (steps >> (w & ~(run_steps - 1))) & ((1u << run_steps) - 1u);
            const int lead = __ffs(group) - 1;                          // first fetched step of the group
            const int n_run = 32 - __clz(group) - lead;                 // up to its last one (the steps between come along)
            uint32_t bytes = 0;
            if (lane < 2 * DT_CONSUMERS && group && (w & (run_steps - 1)) == lead) bytes = (uint32_t)n_run * DT_RUN_BYTES;
            uint32_t total = bytes;
#pragma unroll
            for (int o = 1; o < 2 * DT_CONSUMERS; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
            if (lane == 0)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full0 + 8 * slot), "r"(total) : "memory");
            __syncwarp();
            if (bytes) {
                const bool is_v = lane >= DT_CONSUMERS;
                const int64_t off = (((int64_t)page * Hkv + hk) * P + (j0 % P)) * DH;
                const uint32_t dst = ring + slot * DT_STAGE_BYTES + ((is_v ? DT_CONSUMERS : 0) + w) * DT_RUN_BYTES;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(dst), "l"((is_v ? vc : kc) + off), "r"(bytes), "r"(full0 + 8 * slot) : "memory");
            }
            issued = it + 1;
        };
        // stages that end before this step's own position hold keys of earlier steps only
        for (int s = stage_lo; s < stage_hi && s - stage_lo < DT_STAGES; ++s) {
            if (first_al + DT_KEYS * s + DT_KEYS - 1 >= pos) break;
            issue_stage(s);
        }
        pdl_wait();
        for (int s = stage_lo + issued; s < stage_hi; ++s) {
            const int it = s - stage_lo, slot = it % DT_STAGES;
            if (lane == 0) ok = dt_wait(empty0 + 8 * slot, ((uint32_t)(it / DT_STAGES) & 1u) ^ 1u, status);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            if (!ok) break;
            issue_stage(s);
        }
        if (!ok && lane == 0) {   // a bounded chance for the copies in flight to land before the memory is released
            for (int it = issued > DT_STAGES ? issued - DT_STAGES : 0; it < issued; ++it)
                dt_wait(full0 + 8 * (it % DT_STAGES), (uint32_t)(it / DT_STAGES) & 1u, nullptr);
        }
    } else {
        // -------------------------------------------------------------------- consumers
        pdl_wait();
        IMP_TL_WAITED()
        RowInfo rows[2];
        const __nv_bfloat16* qrow[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int hr = row0 + g + 8 * r;
            const bool used = r < NR && hr < G;
            rows[r].limit = used ? pos : -1;
            rows[r].first = first;
            qrow[r] = used ? q + (int64_t)tok * q_stride + (int64_t)(hk * G + hr) * DH : nullptr;
        }
        uint32_t qa[KSTEPS][4];
        load_q(qa, qrow[0], qrow[1], t4);
        if constexpr (DH % 64 == 0) {
            if (fz.qkv) dec_q_norm_rope<NR>(qa, fz, pos, t4);
        }
        // The warp whose 16 keys include the token's own makes that key and value now and writes them to their page
        // (the raw rows travel beside q); the stage's copy in shared memory is patched when it has landed.
        OwnKey own;
        int own_stage = -1;
        if constexpr (DH % 64 == 0) {
            const int s_own = (pos - first_al) / DT_KEYS;
            if (fz.qkv && s_own >= stage_lo && s_own < stage_hi && ((pos - first_al) % DT_KEYS) / 16 == warp) {
                const int page = bt[pos / P];
                if (page >= 0 && page < num_pages) {     // else the producer reports it
                    const __nv_bfloat16* kraw = fz.qkv + (int64_t)tok * fz.stride + (int64_t)(Hq + hk) * DH;
                    dec_make_own_key(own, fz, kraw, kraw + (int64_t)Hkv * DH, (((int64_t)page * Hkv + hk) * P + (pos % P)) * DH,
                                     pos, lane);
                    own_stage = s_own;
                }
            }
        }
        for (int s = stage_lo; s < stage_hi; ++s) {
            const int it = s - stage_lo, slot = it % DT_STAGES;
            const bool ok = __all_sync(0xffffffffu, dt_wait(full0 + 8 * slot, (uint32_t)(it / DT_STAGES) & 1u, status));
            if (!ok) break;
            const int j0 = first_al + DT_KEYS * s + 16 * warp;
            if constexpr (DH % 64 == 0) {
                if (s == own_stage) {
                    unsigned char* sb = dt_smem + slot * DT_STAGE_BYTES;
                    dec_patch_own_key(own, sb + warp * DT_RUN_BYTES + (pos - j0) * DH * 2,
                                      sb + (DT_CONSUMERS + warp) * DT_RUN_BYTES + (pos - j0) * DH * 2, lane);
                }
            }
            if (j0 <= pos && j0 + 15 >= first) {
                const unsigned char* sb = dt_smem + slot * DT_STAGE_BYTES;
                dec_compute_smem<NR>(st, qa, rows, sb + warp * DT_RUN_BYTES, sb + (DT_CONSUMERS + warp) * DT_RUN_BYTES, j0,
                                     scale_log2, lane);
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty0 + 8 * slot) : "memory");
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
            st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
        }
    }
    __syncthreads();   // every copy has been consumed (or given up): the ring becomes the merge buffer
    // ---- merge the four consumer warps (fragment-wise, through shared memory) ------------------------
    float* smem = reinterpret_cast<float*>(dt_smem);
    constexpr int NACC = NTILES * 2 * NR;
    constexpr int PER_WARP = NACC + 2 * NR;
    if (warp > 0 && warp < DT_CONSUMERS) {
        float* dst = smem + (size_t)(warp - 1) * PER_WARP * 32;
#pragma unroll
        for (int i = 0; i < NTILES; ++i)
#pragma unroll
            for (int c = 0; c < 2 * NR; ++c) dst[(i * 2 * NR + c) * 32 + lane] = st.o[i][c];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            dst[(NACC + r) * 32 + lane] = st.m[r];
            dst[(NACC + NR + r) * 32 + lane] = st.l[r];
        }
    }
    __syncthreads();
    if (warp != 0 && !cluster_merge) return;
    if (warp == 0)
    for (int w = 1; w < DT_CONSUMERS; ++w) {
        const float* src = smem + (size_t)(w - 1) * PER_WARP * 32;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const float mo = src[(NACC + r) * 32 + lane];
            const float lo = src[(NACC + NR + r) * 32 + lane];
            const float m_new = fmaxf(st.m[r], mo);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float ca = exp2f(st.m[r] - m_use), cb = exp2f(mo - m_use);
            st.l[r] = st.l[r] * ca + lo * cb;
            st.m[r] = m_new;
#pragma unroll
            for (int i = 0; i < NTILES; ++i) {
                st.o[i][2 * r] = st.o[i][2 * r] * ca + src[(i * 2 * NR + 2 * r) * 32 + lane] * cb;
                st.o[i][2 * r + 1] = st.o[i][2 * r + 1] * ca + src[(i * 2 * NR + 2 * r + 1) * 32 + lane] * cb;
            }
        }
    }
    if (cluster_merge) {
        // Every CTA of the cluster is past its ring (first barrier; it also says that all of them run), then the
        // splits 1.. store their state into the first CTA's shared memory behind its own merge buffer (second
        // barrier), and its first warp folds them in, in split order.  Every thread of every CTA takes part in
        // both barriers, whatever happened before.
        float* xch = smem + (size_t)(DT_CONSUMERS - 1) * PER_WARP * 32;
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp == 0 && split > 0) {
            const uint32_t local = (uint32_t)__cvta_generic_to_shared(xch + (size_t)(split - 1) * PER_WARP * 32 + lane);
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0u));
#pragma unroll
            for (int i = 0; i < NTILES; ++i)
#pragma unroll
                for (int c = 0; c < 2 * NR; ++c)
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)((i * 2 * NR + c) * 32) * 4u), "f"(st.o[i][c]) : "memory");
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)((NACC + r) * 32) * 4u), "f"(st.m[r]) : "memory");
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)((NACC + NR + r) * 32) * 4u), "f"(st.l[r]) : "memory");
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp != 0 || split != 0) {
            IMP_TL_END()
            return;
        }
        for (int w = 1; w < n_splits; ++w) {
            const float* src = xch + (size_t)(w - 1) * PER_WARP * 32;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const float mo = src[(NACC + r) * 32 + lane];
                const float lo = src[(NACC + NR + r) * 32 + lane];
                const float m_new = fmaxf(st.m[r], mo);
                const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
                const float ca = exp2f(st.m[r] - m_use), cb = exp2f(mo - m_use);
                st.l[r] = st.l[r] * ca + lo * cb;
                st.m[r] = m_new;
#pragma unroll
                for (int i = 0; i < NTILES; ++i) {
                    st.o[i][2 * r] = st.o[i][2 * r] * ca + src[(i * 2 * NR + 2 * r) * 32 + lane] * cb;
                    st.o[i][2 * r + 1] = st.o[i][2 * r + 1] * ca + src[(i * 2 * NR + 2 * r + 1) * 32 + lane] * cb;
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int hr = row0 + g + 8 * r;
        if (hr >= G) continue;
        const int head = hk * G + hr;
        if (n_splits == 1 || cluster_merge) {
            const float inv = st.l[r] > 0.f ? 1.f / st.l[r] : 0.f;
            __nv_bfloat16* o = out + (int64_t)tok * out_stride + (int64_t)head * DH;
#pragma unroll
            for (int i = 0; i < NTILES; ++i) {
                o[dim_of(i, 2 * t4)] = __float2bfloat16_rn(st.o[i][2 * r] * inv);
                o[dim_of(i, 2 * t4 + 1)] = __float2bfloat16_rn(st.o[i][2 * r + 1] * inv);
            }
        } else {
            const int64_t slot = ((int64_t)tok * Hq + head) * n_splits + split;
            float* o = part_o + slot * DH;
#pragma unroll
            for (int i = 0; i < NTILES; ++i) {
                o[dim_of(i, 2 * t4)] = st.o[i][2 * r];
                o[dim_of(i, 2 * t4 + 1)] = st.o[i][2 * r + 1];
            }
            if (t4 == 0) {
                part_ml[slot * 2] = st.m[r];
                part_ml[slot * 2 + 1] = st.l[r];
            }
        }
    }
    IMP_TL_END()
}

// Most key splits that merge inside a cluster.  Measured on the whole decode step (8B shape, context 4096): two
// splits (16 sequences) 4.74 against 4.87 ms with the merge kernel, four (8 sequences) 3.97 against 3.98, eight
// (4 sequences) 3.81 against 3.76: larger clusters wait longer for their slowest member than the kernel saves.
#ifndef IMP_DT_CLUSTER_MAX
#define IMP_DT_CLUSTER_MAX 4
#endif
constexpr int DT_CLUSTER_MAX = IMP_DT_CLUSTER_MAX;

// *merged is set when the key splits merged inside the kernel (a cluster per (token, kv head)): no merge kernel then.
template <int NR>
static int launch_decode_tma(dim3 grid, cudaStream_t s, void* out, int64_t out_stride, const void* q, int64_t q_stride,
                             const void* kc, const void* vc, const int* block_table, int bt_stride, const int* seq_of_token,
                             const int* positions, int n_seqs, int Hq, int Hkv, int P, int num_pages, float scale_log2,
                             int window, int n_splits, float* part_o, float* part_ml, int* status, const DecFused& fz,
                             bool* merged) {
    constexpr int SLOT = (NTILES * 2 * NR + 2 * NR) * 32 * (int)sizeof(float);      // one warp's (or split's) state
    constexpr int MERGE = (DT_CONSUMERS - 1 + DT_CLUSTER_MAX - 1) * SLOT;           // the warps' merge, then the splits'
    constexpr int SMEM = DT_STAGES * DT_STAGE_BYTES > MERGE ? DT_STAGES * DT_STAGE_BYTES : MERGE;
    auto kernel = attn_decode_tma_kernel<NR>;
    static bool attr_set = false;
    if (!attr_set) {   // always: the kernel's static barriers come on top of the ring
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) { imp_set_error("imp_attn_decode: %s", cudaGetErrorString(e)); return (int)e; }
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((DT_CONSUMERS + 1) * 32);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    static int use_cluster = -1;      // IMP_B200_ATTN_CLUSTER=0: partial results through global memory and a merge kernel
    if (use_cluster < 0) { const char* e = getenv("IMP_B200_ATTN_CLUSTER"); use_cluster = e ? atoi(e) : 1; }
    int cluster_merge = 0;
    if (use_cluster && n_splits >= 2 && n_splits <= DT_CLUSTER_MAX) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)n_splits;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        // whether the device can place such a cluster is asked once per size, not found out by a failed launch
        static int placeable[DT_CLUSTER_MAX + 1] = {};       // 0 unknown, 1 yes, -1 no
        if (placeable[n_splits] == 0) {
            int n = 0;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
            if (e != cudaSuccess) (void)cudaGetLastError();
            placeable[n_splits] = (e == cudaSuccess && n > 0) ? 1 : -1;
        }
        if (placeable[n_splits] > 0) { cluster_merge = 1; n_attr = 1; }
    }
    // The call without the fused rotary work (decoding sequences beside prompt portions) is launched as an ordinary
    // dependent of the kernels before it.  With the programmatic attribute, 2 of the first 8 runs of a workload of such
    // steps (8 sequences decoding beside 2,048-token portions, 14B shape) ended with a position error reported by one of
    // the step's kernels; 23 runs without the attribute here, 10 without it anywhere and 12 without this path ran clean,
    // but so did 57 later runs WITH it (a build that tags the reporting check saw nothing to tag), so the attribute is
    // not shown to be the cause.  It stays off here because the start it buys is small beside a prompt portion's work.
    // IMP_B200_ATTN_PLAIN_SERIAL=0 brings it back; -DIMP_TAG_STATUS makes a reported code name its check.
    static int serial_plain = -1;
    if (serial_plain < 0) { const char* e = getenv("IMP_B200_ATTN_PLAIN_SERIAL"); serial_plain = e ? atoi(e) : 1; }
    if (imp_pdl_enabled() && !(serial_plain && fz.qkv == nullptr)) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,
                                       (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, bt_stride, seq_of_token,
                                       positions, n_seqs, Hq, Hkv, P, num_pages, scale_log2, window, n_splits, part_o, part_ml,
                                       status, fz, cluster_merge);
    if (e != cudaSuccess) { imp_set_error("imp_attn_decode: %s", cudaGetErrorString(e)); return (int)e; }
    *merged = cluster_merge != 0;
    return 0;
}

template <int NR>
static int launch_decode(dim3 grid, cudaStream_t s, void* out, int64_t out_stride, const void* q, int64_t q_stride,
                         const void* kc, const void* vc, const int* block_table, int bt_stride, const int* seq_of_token,
                         const int* positions, int n_seqs, int Hq, int Hkv, int P, int num_pages, float scale_log2,
                         int window, int n_splits, float* part_o, float* part_ml, int* status) {
    constexpr int SMEM = (WARPS - 1) * (NTILES * 2 * NR + 2 * NR) * 32 * (int)sizeof(float);   // warp merge buffer
    static bool attr_set = false;
    if (!attr_set && SMEM > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) { imp_set_error("imp_attn_decode: %s", cudaGetErrorString(e)); return (int)e; }
        attr_set = true;
    }
    cudaError_t e = imp_launch(attn_decode_kernel<NR>, grid, dim3(WARPS * 32), (size_t)SMEM, s, (__nv_bfloat16*)out, out_stride,
                               (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                               block_table, bt_stride, seq_of_token, positions, n_seqs, Hq, Hkv, P, num_pages, scale_log2,
                               window, n_splits, part_o, part_ml, status);
    if (e != cudaSuccess) { imp_set_error("imp_attn_decode: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}

static int attn_decode_impl(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* kc,
                            const void* vc, const int* block_table, int bt_stride, const int* seq_of_token,
                            const int* positions, int n_tokens, int n_seqs, int Hq, int Hkv, int P, int num_pages,
                            float scale, int window, int n_splits, float* scratch, int* status, void* stream,
                            const DecFused& fz) {
    if (n_tokens == 0) return 0;
    if (int rc = check_common(out, q, kc, vc, block_table, out_stride, q_stride, Hq, Hkv, P, num_pages)) return rc;
    IMP_CHECK_ARG(seq_of_token && positions, "imp_attn_decode: null pointer");
    IMP_CHECK_ARG(n_splits >= 1 && n_splits <= MERGE_MAX_SPLITS, "imp_attn_decode: %d key splits outside [1, %d]", n_splits,
                  MERGE_MAX_SPLITS);
    IMP_CHECK_ARG(n_splits == 1 || scratch, "imp_attn_decode: splits need scratch memory");
    IMP_CHECK_ARG(n_tokens <= 65535, "imp_attn_decode: more than 65535 tokens");
    cudaStream_t s = (cudaStream_t)stream;
    const int G = Hq / Hkv;
    const int tiles_per_group = (G + 15) / 16;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (int64_t)n_tokens * Hq * n_splits * DH : nullptr;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(n_splits, Hkv * tiles_per_group, n_tokens);
    const bool bulk = P % 16 == 0 && getenv("IMP_B200_ATTN_DIRECT") == nullptr;   // whole 16-key steps per page
    if (fz.qkv && !(bulk && DH % 64 == 0)) return IMP_ERR_UNSUPPORTED;               // only the bulk-copy kernel does that
#define DEC_ARGS grid, s, out, out_stride, q, q_stride, kc, vc, block_table, bt_stride, seq_of_token, positions, n_seqs, Hq, \
                 Hkv, P, num_pages, scale_log2, window, n_splits, part_o, part_ml, status, fz, &merged
    bool merged = false;
    if (bulk) {
        if (int rc = (G <= 8) ? launch_decode_tma<1>(DEC_ARGS) : launch_decode_tma<2>(DEC_ARGS)) return rc;
    } else if (G <= 8) {
        if (int rc = launch_decode<1>(grid, s, out, out_stride, q, q_stride, kc, vc, block_table, bt_stride, seq_of_token,
                                      positions, n_seqs, Hq, Hkv, P, num_pages, scale_log2, window, n_splits, part_o,
                                      part_ml, status))
            return rc;
    } else {
        if (int rc = launch_decode<2>(grid, s, out, out_stride, q, q_stride, kc, vc, block_table, bt_stride, seq_of_token,
                                      positions, n_seqs, Hq, Hkv, P, num_pages, scale_log2, window, n_splits, part_o,
                                      part_ml, status))
            return rc;
    }
#undef DEC_ARGS
    if (n_splits > 1 && !merged) {
        imp_launch(attn_merge_kernel, dim3(n_tokens * Hq), dim3(128), 0, s, (__nv_bfloat16*)out, out_stride,
                   (const float*)part_o, (const float*)part_ml, Hq, n_splits);
    }
    IMP_RETURN_LAUNCH();
}

IMP_API int imp_attn_decode(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* kc,
                            const void* vc, const int* block_table, int bt_stride, const int* seq_of_token,
                            const int* positions, int n_tokens, int n_seqs, int Hq, int Hkv, int P, int num_pages,
                            float scale, int window, int n_splits, float* scratch, int* status, void* stream) {
    return attn_decode_impl(out, out_stride, q, q_stride, kc, vc, block_table, bt_stride, seq_of_token, positions, n_tokens,
                            n_seqs, Hq, Hkv, P, num_pages, scale, window, n_splits, scratch, status, stream, DecFused{});
}

// The decode step from the projection's raw rows: qkv [n_tokens, qkv_stride] holds q heads, k heads, v heads of
// every token as the q,k,v product left them.  q and k are normalised per head (weights [DH] in 32-bit, or null)
// and rotated over the whole head (cos/sin [max_pos, DH/2]) inside the attention kernel, which also writes the new
// key and value into their pages; the rotary kernel is not run for such a step.  IMP_ERR_UNSUPPORTED (and nothing
// done) for head sizes that are no multiple of 64 and page sizes that are no multiple of 16.
IMP_API int imp_attn_decode_fused(void* out, int64_t out_stride, const void* qkv, int64_t qkv_stride, void* kc, void* vc,
                                  const int* block_table, int bt_stride, const int* seq_of_token, const int* positions,
                                  int n_tokens, int n_seqs, int Hq, int Hkv, int P, int num_pages, float scale, int window,
                                  int n_splits, float* scratch, const float* q_norm_w, const float* k_norm_w, float eps,
                                  const float* cos_tab, const float* sin_tab, int max_pos, int* status, void* stream) {
    IMP_CHECK_ARG(qkv && cos_tab && sin_tab && max_pos > 0, "imp_attn_decode_fused: null pointer");
    IMP_CHECK_ARG((q_norm_w == nullptr) == (k_norm_w == nullptr), "imp_attn_decode_fused: q and k norm weights must both be set or both be null");
    IMP_CHECK_ARG(qkv_stride >= (int64_t)(Hq + 2 * Hkv) * DH && qkv_stride % 8 == 0, "imp_attn_decode_fused: bad row stride");
    IMP_CHECK_ARG((uintptr_t)cos_tab % 8 == 0 && (uintptr_t)sin_tab % 8 == 0, "imp_attn_decode_fused: unaligned tables");
    DecFused fz;
    fz.qkv = (const __nv_bfloat16*)qkv; fz.stride = qkv_stride; fz.q_norm_w = q_norm_w; fz.k_norm_w = k_norm_w;
    fz.cos_tab = cos_tab; fz.sin_tab = sin_tab; fz.k_pages = (__nv_bfloat16*)kc; fz.v_pages = (__nv_bfloat16*)vc;
    fz.eps = eps; fz.max_pos = max_pos;
    return attn_decode_impl(out, out_stride, qkv, qkv_stride, kc, vc, block_table, bt_stride, seq_of_token, positions, n_tokens,
                            n_seqs, Hq, Hkv, P, num_pages, scale, window, n_splits, scratch, status, stream, fz);
}

// ================================================================================= prefill
// Tiles of up to 32 consecutive query tokens of one sequence: tile_tok0[i] is the first token's
// index in the batch, tile_rows[i] the number of tokens.  grid (n_tiles, Hkv * ceil(G / HPC));
// a CTA has 2 * HPC warps: warp w owns the 16 tokens of sub-tile w / HPC and query head w % HPC of
// its head group.  Stages of 32 keys go through a three-deep ring shared by all warps.
constexpr int PRE_KEYS = 32;
constexpr int PRE_STAGES = 3;
constexpr int PRE_SMEM_BYTES = PRE_STAGES * StageGeom<PRE_KEYS>::BYTES;

template <int HPC>
__global__ void __launch_bounds__(2 * HPC * 32) attn_prefill_kernel(
    __nv_bfloat16* __restrict__ out, int64_t out_stride, const __nv_bfloat16* __restrict__ q, int64_t q_stride,
    const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
    const int* __restrict__ tile_tok0, const int* __restrict__ tile_rows, int n_seqs, int Hq, int Hkv, int P,
    int num_pages, float scale_log2, int window, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int THREADS = 2 * HPC * 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int G = Hq / Hkv;
    const int groups_per_kv = (G + HPC - 1) / HPC;
    const int tile = blockIdx.x;
    const int hk = blockIdx.y / groups_per_kv;
    const int head_in_group = (blockIdx.y % groups_per_kv) * HPC + warp % HPC;
    const int sub = warp / HPC;                       // which 16 tokens of the tile
    const int tok0 = tile_tok0[tile], n_rows = tile_rows[tile];
    const int seq = seq_of_token[tok0];
    const int pos0 = positions[tok0];
    const int pos_last = pos0 + n_rows - 1;
    if (seq < 0 || seq >= n_seqs || pos0 < 0 || pos_last / P >= bt_stride || n_rows < 1 || n_rows > 32) {
        if (tid == 0) imp_report(status, seq < 0 || seq >= n_seqs ? IMP_TAGGED(IMP_BAD_SEQUENCE, 3) : IMP_TAGGED(IMP_BAD_POSITION, 3));
        return;
    }
    const int* bt = block_table + (int64_t)seq * bt_stride;
    const bool warp_used = head_in_group < G && sub * 16 < n_rows;
    const int head = hk * G + head_in_group;
    RowInfo rows[2];
    const __nv_bfloat16* qrow[2];
    int my_last = -1;                                 // last position any row of this warp may see
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int rr = sub * 16 + g + 8 * r;
        const bool used = warp_used && rr < n_rows;
        const int pos = pos0 + rr;
        rows[r].limit = used ? pos : -1;
        rows[r].first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        qrow[r] = used ? q + (int64_t)(tok0 + rr) * q_stride + (int64_t)head * DH : nullptr;
    }
    if (warp_used) my_last = pos0 + min(n_rows, sub * 16 + 16) - 1;
    const int my_first = (window > 0 && pos0 + sub * 16 - window + 1 > 0) ? pos0 + sub * 16 - window + 1 : 0;
    const int my_lo_limit = pos0 + sub * 16;          // the smallest limit among the warp's rows
    const int my_hi_first = (window > 0 && my_last - window + 1 > 0) ? my_last - window + 1 : 0;   // the largest first

    const int first_tile = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int j_begin = first_tile & ~(PRE_KEYS - 1);
    const int n_stages = (pos_last - j_begin) / PRE_KEYS + 1;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem_raw);
#pragma unroll
    for (int s = 0; s < PRE_STAGES - 1; ++s) {
        if (s < n_stages)
            load_stage<PRE_KEYS, THREADS>(ring + s * StageGeom<PRE_KEYS>::BYTES, kc, vc, bt, P, Hkv, hk, num_pages,
                                          j_begin + PRE_KEYS * s, first_tile, pos_last, tid, status);
        cp_commit();
    }
    uint32_t qa[KSTEPS][4];
    load_q(qa, qrow[0], qrow[1], t4);
    TileState st;
    tile_init(st);
    for (int s = 0; s < n_stages; ++s) {
        cp_wait<PRE_STAGES - 2>();   // stage s has landed (this thread's part)
        __syncthreads();             // ... and everyone's; the slot of stage s-1 is free again
        if (s + PRE_STAGES - 1 < n_stages)
            load_stage<PRE_KEYS, THREADS>(ring + ((s + PRE_STAGES - 1) % PRE_STAGES) * StageGeom<PRE_KEYS>::BYTES, kc, vc, bt,
                                          P, Hkv, hk, num_pages, j_begin + PRE_KEYS * (s + PRE_STAGES - 1), first_tile,
                                          pos_last, tid, status);
        cp_commit();
        const int j0 = j_begin + PRE_KEYS * s;
        const unsigned char* ksm = smem_raw + (s % PRE_STAGES) * StageGeom<PRE_KEYS>::BYTES;
        const unsigned char* vsm = ksm + StageGeom<PRE_KEYS>::K_BYTES;
        if (j0 <= my_last && j0 + PRE_KEYS - 1 >= my_first) {
            // every key of the stage visible to every row of the warp: no mask needed
            const bool need_mask = j0 + PRE_KEYS - 1 > my_lo_limit || j0 < my_hi_first;
            process_stage32(st, qa, rows, ksm, vsm, j0, scale_log2, need_mask, lane);
        }
    }
    cp_wait<0>();
    if (!warp_used) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
        const int rr = sub * 16 + g + 8 * r;
        if (rr >= n_rows) continue;
        const float inv = st.l[r] > 0.f ? 1.f / st.l[r] : 0.f;
        __nv_bfloat16* o = out + (int64_t)(tok0 + rr) * out_stride + (int64_t)head * DH;
#pragma unroll
        for (int i = 0; i < NTILES; ++i) {
            o[dim_of(i, 2 * t4)] = __float2bfloat16_rn(st.o[i][2 * r] * inv);
            o[dim_of(i, 2 * t4 + 1)] = __float2bfloat16_rn(st.o[i][2 * r + 1] * inv);
        }
    }
}

template <int HPC>
static int launch_prefill(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* kc, const void* vc,
                          const int* block_table, int bt_stride, const int* seq_of_token, const int* positions,
                          const int* tile_tok0, const int* tile_rows, int n_tiles, int n_seqs, int Hq, int Hkv, int P,
                          int num_pages, float scale, int window, int* status, cudaStream_t s) {
    static bool attr_set = false;
    if (!attr_set && PRE_SMEM_BYTES > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HPC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             PRE_SMEM_BYTES);
        if (e != cudaSuccess) { imp_set_error("imp_attn_prefill: %s", cudaGetErrorString(e)); return (int)e; }
        attr_set = true;
    }
    const int G = Hq / Hkv;
    dim3 grid(n_tiles, Hkv * ((G + HPC - 1) / HPC));
    imp_launch(attn_prefill_kernel<HPC>, grid, dim3(2 * HPC * 32), (size_t)PRE_SMEM_BYTES, s, (__nv_bfloat16*)out, out_stride,
               (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, bt_stride,
               seq_of_token, positions, tile_tok0, tile_rows, n_seqs, Hq, Hkv, P, num_pages,
               scale * 1.4426950408889634f, window, status);
    IMP_RETURN_LAUNCH();
}

// Query tokens per tile that imp_attn_prefill expects at most.
IMP_API int imp_attn_prefill_tile_tokens(void) { return 32; }

IMP_API int imp_attn_prefill(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* kc,
                             const void* vc, const int* block_table, int bt_stride, const int* seq_of_token,
                             const int* positions, const int* tile_tok0, const int* tile_rows, int n_tiles,
                             int n_seqs, int Hq, int Hkv, int P, int num_pages, float scale, int window, int* status,
                             void* stream) {
    if (n_tiles == 0) return 0;
    if (int rc = check_common(out, q, kc, vc, block_table, out_stride, q_stride, Hq, Hkv, P, num_pages)) return rc;
    IMP_CHECK_ARG(seq_of_token && positions && tile_tok0 && tile_rows, "imp_attn_prefill: null pointer");
    const int G = Hq / Hkv;
    IMP_CHECK_ARG((int64_t)Hkv * ((G + 3) / 4) <= 65535, "imp_attn_prefill: too many head groups");
    cudaStream_t s = (cudaStream_t)stream;
#define ARGS out, out_stride, q, q_stride, kc, vc, block_table, bt_stride, seq_of_token, positions, tile_tok0, tile_rows, \
             n_tiles, n_seqs, Hq, Hkv, P, num_pages, scale, window, status, s
    if (G == 1) return launch_prefill<1>(ARGS);
    if (G == 2) return launch_prefill<2>(ARGS);
    return launch_prefill<4>(ARGS);
#undef ARGS
}

// ================================================================== decode without allocation
// See attention_noalloc.h.  The scratch of the split-key decode kernel lives in the library image.
#include "attention_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[IMP_ATTN_NOALLOC_SCRATCH_FLOATS];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address: the
// address is looked up once per device, with that device current, and kept here.
constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};

IMP_API int imp_attn_decode_noalloc(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* k_cache,
                                    const void* v_cache, const int* block_table, int bt_stride, const int* seq_of_token,
                                    const int* positions, int n_tokens, int n_seqs, int n_q_heads, int n_kv_heads,
                                    int page_size, int num_pages, float scale, int window, int n_splits, int* status,
                                    void* stream) {
    IMP_CHECK_ARG(n_tokens >= 0 && n_q_heads > 0 && n_splits >= 1, "imp_attn_decode_noalloc: bad argument");
    const int64_t need = n_splits > 1 ? (int64_t)n_tokens * n_q_heads * n_splits * (DH + 2) : 0;
    IMP_CHECK_ARG(need <= IMP_ATTN_NOALLOC_SCRATCH_FLOATS,
                  "imp_attn_decode_noalloc: %lld floats of scratch needed (tokens %d x heads %d x splits %d x %d), the "
                  "built-in buffer holds %d; use fewer splits or imp_attn_decode with your own scratch",
                  (long long)need, n_tokens, n_q_heads, n_splits, DH + 2, IMP_ATTN_NOALLOC_SCRATCH_FLOATS);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
        imp_set_error("imp_attn_decode_noalloc: cannot identify the current device (%s)",
                      e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
        return e != cudaSuccess ? (int)e : IMP_ERR_ARG;
    }
    if (g_noalloc_ptr[dev] == nullptr) {   // first call on this device
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            imp_set_error("imp_attn_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : IMP_ERR_ARG;
        }
        g_noalloc_ptr[dev] = p;
    }
    return imp_attn_decode(out, out_stride, q, q_stride, k_cache, v_cache, block_table, bt_stride, seq_of_token,
                           positions, n_tokens, n_seqs, n_q_heads, n_kv_heads, page_size, num_pages, scale, window,
                           n_splits, g_noalloc_ptr[dev], status, stream);
}
