// Per-head RMSNorm on q and k, rotary position encoding, and the write of k and
// v into the paged cache, in one pass over the fused q|k|v projection output.
//
// Reference counterparts: rmsnorm on q/k viewed per head (src/graph/
// executor_forward.cu:537-546), rope_forward_* (src/compute/rope.cu:45-182),
// the fused decode kernel (src/compute/rope.cu:270-413) and
// write_kv_cache_fused_kernel (src/graph/executor_kernels.cu:342-388).
// Pairing is (i, i + rot/2) ("neox"), x_i' = x_i cos a - x_{i+rot/2} sin a,
// x_{i+rot/2}' = x_i sin a + x_{i+rot/2} cos a (src/compute/rope.cu:96-101).
// Differences: cos and sin come from a table built in double precision on the
// host (the reference evaluates __cosf/__sinf of a 32-bit angle), the norm's
// result stays in 32-bit until after the rotation, and any number of tokens of
// any mix of sequences is handled by one launch (the reference's cache write
// assumes token i belongs to sequence i in a batch).
//
// Cache layout of one layer: K and V each [num_pages][kv_heads][page_size][head_dim].
#include "common.cuh"

template <typename TA, typename TW>
__global__ void qk_norm_rope_kv_kernel(
    TA* __restrict__ qkv, int64_t row_stride, int Hq, int Hkv, int Dh,
    const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps, float weight_offset,
    const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int rot_dim, int max_pos,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int bt_stride, int n_seqs,
    TA* __restrict__ k_cache, TA* __restrict__ v_cache, int page_size, int num_pages,
    int n_tokens, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int heads_per_token = Hq + 2 * Hkv;
    if (unit >= n_tokens * heads_per_token) return;
    const int t = unit / heads_per_token;
    const int hh = unit - t * heads_per_token;
    const int pos = positions[t];
    TA* x = qkv + (int64_t)t * row_stride + (int64_t)hh * Dh;

    const bool is_q = hh < Hq;
    const bool is_k = !is_q && hh < Hq + Hkv;
    const int kv_head = is_q ? 0 : (is_k ? hh - Hq : hh - Hq - Hkv);

    // Where this head's row lives in the cache (k and v only).
    TA* dst = nullptr;
    if (!is_q) {
        TA* cache = is_k ? k_cache : v_cache;
        if (cache == nullptr) {
            if (!is_k) return;  // v without a cache: nothing to do
        } else {
            const int seq = seq_of_token[t];
            if (seq < 0 || seq >= n_seqs) {
                if (lane == 0) imp_report(status, IMP_BAD_SEQUENCE);
                return;
            }
            const int slot_page = pos / page_size;
            if (pos < 0 || slot_page >= bt_stride) {
                if (lane == 0) imp_report(status, IMP_TAGGED(IMP_BAD_POSITION, 6));
                return;
            }
            const int page = block_table[(int64_t)seq * bt_stride + slot_page];
            if (page < 0 || page >= num_pages) {
                if (lane == 0) imp_report(status, IMP_BAD_PAGE);
                return;
            }
            dst = cache + (((int64_t)page * Hkv + kv_head) * page_size + (pos - slot_page * page_size)) * Dh;
        }
    }

    if (!is_q && !is_k) {  // v: plain copy into its page
        for (int i = lane; i < Dh; i += 32) dst[i] = x[i];
        return;
    }

    const TW* nw = is_q ? q_norm_w : k_norm_w;
    float inv = 1.f;
    if (nw) {
        float ss = 0.f;
        for (int i = lane; i < Dh; i += 32) {
            const float v = to_float(x[i]);
            ss += v * v;
        }
        ss = warp_sum(ss);
        inv = rsqrtf(ss / (float)Dh + eps);
    }
    const int half = rot_dim >> 1;
    const bool rotate = cos_tab != nullptr && half > 0;
    if (rotate && (pos < 0 || pos >= max_pos)) {
        if (lane == 0) imp_report(status, IMP_TAGGED(IMP_BAD_POSITION, 6));
        return;
    }
    TA* out = is_q ? x : (dst ? dst : x);
    // Rotated part: pairs (i, i + half).
    for (int i = lane; i < half; i += 32) {
        float a = to_float(x[i]) * inv, b = to_float(x[i + half]) * inv;
        if (nw) {
            a *= to_float(nw[i]) + weight_offset;
            b *= to_float(nw[i + half]) + weight_offset;
        }
        float c = 1.f, s = 0.f;
        if (rotate) {
            c = cos_tab[(int64_t)pos * half + i];
            s = sin_tab[(int64_t)pos * half + i];
        }
        out[i] = from_float<TA>(a * c - b * s);
        out[i + half] = from_float<TA>(a * s + b * c);
    }
    // Pass-through part beyond the rotated width (everything when nothing rotates: rot_dim is 0 then).
    for (int i = 2 * half + lane; i < Dh; i += 32) {
        float a = to_float(x[i]) * inv;
        if (nw) a *= to_float(nw[i]) + weight_offset;
        out[i] = from_float<TA>(a);
    }
}

// The same for bfloat16 activations with 4-byte and 8-byte accesses: lane l holds the pairs
// (2l, 2l+1) of both rotary halves (and the next 64 for head sizes above 128), so a warp reads a head's
// row in whole 128-byte lines.  Needs rot_dim % 4 == 0, rot_dim <= 256, Dh % 4 == 0, row_stride % 4 == 0.
template <typename TW>
__global__ void qk_norm_rope_kv_vec_kernel(
    __nv_bfloat16* __restrict__ qkv, int64_t row_stride, int Hq, int Hkv, int Dh,
    const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps, float weight_offset,
    const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int rot_dim, int max_pos,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int bt_stride, int n_seqs,
    __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int page_size, int num_pages,
    int n_tokens, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int heads_per_token = Hq + 2 * Hkv;
    if (unit >= n_tokens * heads_per_token) return;
    const int t = unit / heads_per_token;
    const int hh = unit - t * heads_per_token;
    const int pos = positions[t];
    __nv_bfloat16* x = qkv + (int64_t)t * row_stride + (int64_t)hh * Dh;
    const bool is_q = hh < Hq;
    const bool is_k = !is_q && hh < Hq + Hkv;
    const int kv_head = is_q ? 0 : (is_k ? hh - Hq : hh - Hq - Hkv);

    __nv_bfloat16* dst = nullptr;
    if (!is_q) {
        __nv_bfloat16* cache = is_k ? k_cache : v_cache;
        if (cache == nullptr) {
            if (!is_k) return;
        } else {
            const int seq = seq_of_token[t];
            if (seq < 0 || seq >= n_seqs) {
                if (lane == 0) imp_report(status, IMP_BAD_SEQUENCE);
                return;
            }
            const int slot_page = pos / page_size;
            if (pos < 0 || slot_page >= bt_stride) {
                if (lane == 0) imp_report(status, IMP_TAGGED(IMP_BAD_POSITION, 6));
                return;
            }
            const int page = block_table[(int64_t)seq * bt_stride + slot_page];
            if (page < 0 || page >= num_pages) {
                if (lane == 0) imp_report(status, IMP_BAD_PAGE);
                return;
            }
            dst = cache + (((int64_t)page * Hkv + kv_head) * page_size + (pos - slot_page * page_size)) * Dh;
        }
    }
    if (!is_q && !is_k) {  // v: plain copy into its page, 8 bytes per lane
        for (int i = lane * 4; i < Dh; i += 128) *reinterpret_cast<uint2*>(dst + i) = *reinterpret_cast<const uint2*>(x + i);
        return;
    }
    const TW* nw = is_q ? q_norm_w : k_norm_w;
    const int half = rot_dim >> 1;
    const bool rotate = cos_tab != nullptr && half > 0;
    if (rotate && (pos < 0 || pos >= max_pos)) {
        if (lane == 0) imp_report(status, IMP_TAGGED(IMP_BAD_POSITION, 6));
        return;
    }
    // pairs j = lane, lane + 32 of each half (half <= 128 elements = 64 pairs)
    float2 a[2], b[2];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int j = lane + 32 * r;
        a[r] = b[r] = make_float2(0.f, 0.f);
        if (2 * j < half) {
            a[r] = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x)[j]);
            b[r] = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x + half)[j]);
            ss += a[r].x * a[r].x + a[r].y * a[r].y + b[r].x * b[r].x + b[r].y * b[r].y;
        }
    }
    for (int i = 2 * half + lane; i < Dh; i += 32) {   // the part beyond the rotated width
        const float v = __bfloat162float(x[i]);
        ss += v * v;
    }
    float inv = 1.f;
    if (nw) inv = rsqrtf(warp_sum(ss) / (float)Dh + eps);
    __nv_bfloat16* out = is_q ? x : (dst ? dst : x);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int j = lane + 32 * r;
        if (2 * j >= half) continue;
        float2 av = make_float2(a[r].x * inv, a[r].y * inv), bv = make_float2(b[r].x * inv, b[r].y * inv);
        if (nw) {
            av.x *= to_float(nw[2 * j]) + weight_offset;
            av.y *= to_float(nw[2 * j + 1]) + weight_offset;
            bv.x *= to_float(nw[2 * j + half]) + weight_offset;
            bv.y *= to_float(nw[2 * j + 1 + half]) + weight_offset;
        }
        float2 c = make_float2(1.f, 1.f), sn = make_float2(0.f, 0.f);
        if (rotate) {
            c = *reinterpret_cast<const float2*>(cos_tab + (int64_t)pos * half + 2 * j);
            sn = *reinterpret_cast<const float2*>(sin_tab + (int64_t)pos * half + 2 * j);
        }
        reinterpret_cast<__nv_bfloat162*>(out)[j] = __floats2bfloat162_rn(av.x * c.x - bv.x * sn.x, av.y * c.y - bv.y * sn.y);
        reinterpret_cast<__nv_bfloat162*>(out + half)[j] =
            __floats2bfloat162_rn(av.x * sn.x + bv.x * c.x, av.y * sn.y + bv.y * c.y);
    }
    for (int i = 2 * half + lane; i < Dh; i += 32) {
        float v = __bfloat162float(x[i]) * inv;
        if (nw) v *= to_float(nw[i]) + weight_offset;
        out[i] = __float2bfloat16_rn(v);
    }
}

// qkv: [n_tokens, row_stride] with q heads, then k heads, then v heads, each head_dim wide.
// q is normalised and rotated in place; k (normalised, rotated) and v go to the pages
// (when k_cache/v_cache are null, k is rotated in place and v is left alone).
IMP_API int imp_qk_norm_rope_kv_write(
    void* qkv, int64_t row_stride, int n_tokens, int Hq, int Hkv, int Dh,
    const void* q_norm_w, const void* k_norm_w, float eps, float weight_offset, int w_dtype,
    const float* cos_tab, const float* sin_tab, int rot_dim, int max_pos,
    const int* positions, const int* seq_of_token, const int* block_table, int bt_stride, int n_seqs,
    void* k_cache, void* v_cache, int page_size, int num_pages, int act_dtype, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(qkv && positions && Hq >= 0 && Hkv >= 0 && Dh > 0, "imp_qk_norm_rope_kv_write: bad argument");
    IMP_CHECK_ARG(rot_dim >= 0 && rot_dim <= Dh && rot_dim % 2 == 0,
                  "imp_qk_norm_rope_kv_write: rotary width %d must be even and at most head_dim %d", rot_dim, Dh);
    IMP_CHECK_ARG((k_cache == nullptr) == (v_cache == nullptr), "imp_qk_norm_rope_kv_write: k and v cache must both be set or both be null");
    if (k_cache) IMP_CHECK_ARG(seq_of_token && block_table && page_size > 0 && num_pages > 0,
                               "imp_qk_norm_rope_kv_write: cache write needs the batch's block table");
    IMP_CHECK_ARG((q_norm_w == nullptr) == (k_norm_w == nullptr), "imp_qk_norm_rope_kv_write: q and k norm weights must both be set or both be null");
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    const int64_t units = (int64_t)n_tokens * (Hq + 2 * Hkv);
    const int grid = (int)((units + warps - 1) / warps);
    if (cos_tab == nullptr) rot_dim = 0;
#define LAUNCH(TA, TW)                                                                                      \
    imp_launch(qk_norm_rope_kv_kernel<TA, TW>, dim3(grid), dim3(warps * 32), 0, s,                          \
        (TA*)qkv, row_stride, Hq, Hkv, Dh, (const TW*)q_norm_w, (const TW*)k_norm_w, eps, weight_offset,    \
        cos_tab, sin_tab, rot_dim, max_pos, positions, seq_of_token, block_table, bt_stride, n_seqs,        \
        (TA*)k_cache, (TA*)v_cache, page_size, num_pages, n_tokens, status)
    const bool vec = act_dtype == IMP_BF16 && rot_dim % 4 == 0 && rot_dim <= 256 && Dh % 4 == 0 && row_stride % 4 == 0 &&
                     (uintptr_t)qkv % 8 == 0 && (uintptr_t)k_cache % 8 == 0 && (uintptr_t)v_cache % 8 == 0 &&
                     (uintptr_t)cos_tab % 8 == 0 && (uintptr_t)sin_tab % 8 == 0;
#define LAUNCH_VEC(TW)                                                                                      \
    imp_launch(qk_norm_rope_kv_vec_kernel<TW>, dim3(grid), dim3(warps * 32), 0, s,                          \
        (__nv_bfloat16*)qkv, row_stride, Hq, Hkv, Dh, (const TW*)q_norm_w, (const TW*)k_norm_w, eps, weight_offset, \
        cos_tab, sin_tab, rot_dim, max_pos, positions, seq_of_token, block_table, bt_stride, n_seqs,        \
        (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, page_size, num_pages, n_tokens, status)
    if (vec && w_dtype == IMP_F32) LAUNCH_VEC(float);
    else if (vec) LAUNCH_VEC(__nv_bfloat16);
    else if (act_dtype == IMP_F32 && w_dtype == IMP_F32) LAUNCH(float, float);
    else if (act_dtype == IMP_F32) LAUNCH(float, __nv_bfloat16);
    else if (w_dtype == IMP_F32) LAUNCH(__nv_bfloat16, float);
    else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
#undef LAUNCH_VEC
    IMP_RETURN_LAUNCH();
}
