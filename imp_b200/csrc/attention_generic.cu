// Paged attention for any batch: every query token attends to the cached keys
// of its own sequence at positions max(0, p-window+1) .. p, p being the token's
// own position (its key and value are already in the pages).
//
// This is the plain kernel of the family: one block per (token, query head),
// 32-bit scores, running max and sum, 32-bit accumulator, IEEE expf.  It is the
// kernel of the float32 path and the yardstick of the faster bfloat16 kernels.
// The order of every reduction depends only on the token's own position, so
// the result is the same whatever else is in the batch and however the prompt
// was cut.
//
// Math as in the reference's flash kernel (src/compute/attention.cu:158-216):
// s_ij = scale * q_i.k_j, masked when j > i or i - j >= window, softmax with a
// running max, o_i = sum_j p_ij v_j; query head h reads kv head h / (Hq/Hkv)
// (src/compute/attention_paged.cu:84-160).  Unlike the reference's prefill
// kernels, which see only the call's own K and V (src/graph/executor_forward.cu:
// 568-604), keys come from the pages, so a later portion of a prompt sees the
// earlier ones.
#include "common.cuh"

constexpr int ATT_BLOCK = 128;
constexpr int ATT_MAX_DH = 256;

template <typename TA>
__global__ void paged_attention_generic_kernel(
    TA* __restrict__ out, int64_t out_stride, const TA* __restrict__ q, int64_t q_stride,
    const TA* __restrict__ k_cache, const TA* __restrict__ v_cache,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ seq_of_token,
    const int* __restrict__ positions, int n_seqs, int Hq, int Hkv, int Dh, int page_size, int num_pages,
    float scale, int window, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float q_s[ATT_MAX_DH];
    __shared__ float p_s[ATT_BLOCK];
    __shared__ int64_t off_s[ATT_BLOCK];
    __shared__ float scratch[33];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int hk = h / (Hq / Hkv);
    const int seq = seq_of_token[t];
    const int pos = positions[t];
    TA* o = out + (int64_t)t * out_stride + (int64_t)h * Dh;
    if (seq < 0 || seq >= n_seqs || pos < 0 || pos / page_size >= bt_stride) {
        if (tid == 0) imp_report(status, seq < 0 || seq >= n_seqs ? IMP_BAD_SEQUENCE : IMP_BAD_POSITION);
        for (int d = tid; d < Dh; d += ATT_BLOCK) o[d] = from_float<TA>(0.f);
        return;
    }
    const TA* qp = q + (int64_t)t * q_stride + (int64_t)h * Dh;
    for (int d = tid; d < Dh; d += ATT_BLOCK) q_s[d] = to_float(qp[d]);
    __syncthreads();

    const int* bt = block_table + (int64_t)seq * bt_stride;
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc0 = 0.f, acc1 = 0.f;  // dims tid and tid + ATT_BLOCK

    for (int j0 = first; j0 <= pos; j0 += ATT_BLOCK) {
        const int j = j0 + tid;
        float s = -INFINITY;
        int64_t off = -1;
        if (j <= pos) {
            const int page = bt[j / page_size];
            if (page < 0 || page >= num_pages) {
                imp_report(status, IMP_BAD_PAGE);
            } else {
                off = (((int64_t)page * Hkv + hk) * page_size + (j % page_size)) * Dh;
                const TA* kp = k_cache + off;
                float dot = 0.f;
                for (int d = 0; d < Dh; ++d) dot = fmaf(q_s[d], to_float(kp[d]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float p = (off >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        p_s[tid] = p;
        off_s[tid] = off;
        const float psum = block_sum(p, scratch);  // contains the barrier that publishes p_s/off_s
        l = l * corr + psum;
        m = m_new;
        const int n_here = min(ATT_BLOCK, pos - j0 + 1);
        if (tid < Dh) {
            float a = acc0 * corr;
            for (int i = 0; i < n_here; ++i)
                if (off_s[i] >= 0) a = fmaf(p_s[i], to_float(v_cache[off_s[i] + tid]), a);
            acc0 = a;
        }
        if (tid + ATT_BLOCK < Dh) {
            float a = acc1 * corr;
            for (int i = 0; i < n_here; ++i)
                if (off_s[i] >= 0) a = fmaf(p_s[i], to_float(v_cache[off_s[i] + tid + ATT_BLOCK]), a);
            acc1 = a;
        }
        __syncthreads();  // p_s/off_s are rewritten by the next chunk
    }
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    if (tid < Dh) o[tid] = from_float<TA>(acc0 * inv_l);
    if (tid + ATT_BLOCK < Dh) o[tid + ATT_BLOCK] = from_float<TA>(acc1 * inv_l);
}

// out: [n_tokens, out_stride] (head h at column h*Dh); q likewise with q_stride.
// k_cache, v_cache: [num_pages, Hkv, page_size, Dh] of one layer.
IMP_API int imp_paged_attention_generic(
    void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
    const int* block_table, int bt_stride, const int* seq_of_token, const int* positions, int n_tokens,
    int n_seqs, int Hq, int Hkv, int Dh, int page_size, int num_pages, float scale, int window, int dtype,
    int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(out && q && k_cache && v_cache && block_table && seq_of_token && positions,
                  "imp_paged_attention_generic: null pointer");
    IMP_CHECK_ARG(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "imp_paged_attention_generic: %d query heads are not a multiple of %d kv heads", Hq, Hkv);
    IMP_CHECK_ARG(Dh > 0 && Dh <= ATT_MAX_DH, "imp_paged_attention_generic: head_dim %d outside (0, %d]", Dh, ATT_MAX_DH);
    IMP_CHECK_ARG(page_size > 0 && num_pages > 0 && window >= 0, "imp_paged_attention_generic: bad cache geometry");
    IMP_CHECK_ARG(Hq <= 65535, "imp_paged_attention_generic: more than 65535 query heads");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, Hq);
    if (dtype == IMP_F32)
        paged_attention_generic_kernel<float><<<grid, ATT_BLOCK, 0, s>>>(
            (float*)out, out_stride, (const float*)q, q_stride, (const float*)k_cache, (const float*)v_cache,
            block_table, bt_stride, seq_of_token, positions, n_seqs, Hq, Hkv, Dh, page_size, num_pages, scale,
            window, status);
    else
        paged_attention_generic_kernel<__nv_bfloat16><<<grid, ATT_BLOCK, 0, s>>>(
            (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache,
            (const __nv_bfloat16*)v_cache, block_table, bt_stride, seq_of_token, positions, n_seqs, Hq, Hkv, Dh,
            page_size, num_pages, scale, window, status);
    IMP_RETURN_LAUNCH();
}
