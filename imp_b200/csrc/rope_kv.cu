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
                if (lane == 0) imp_report(status, IMP_BAD_POSITION);
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
        if (lane == 0) imp_report(status, IMP_BAD_POSITION);
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
    if (act_dtype == IMP_F32 && w_dtype == IMP_F32) LAUNCH(float, float);
    else if (act_dtype == IMP_F32) LAUNCH(float, __nv_bfloat16);
    else if (w_dtype == IMP_F32) LAUNCH(__nv_bfloat16, float);
    else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
    IMP_RETURN_LAUNCH();
}
