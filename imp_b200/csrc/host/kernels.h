// Declarations of the kernel launchers of this library (defined in the .cu files beside this
// folder) for the host code.  Every launcher returns 0, a negative argument error (-2: the kernel
// does not take this shape), or a cudaError_t; imp_last_error() has the text.
#pragma once

#include <stdint.h>

extern "C" {

const char* imp_last_error(void);
const char* imp_status_string(int code);
int imp_device_arch(void);
int imp_device_sm_count(void);

int imp_embedding(float* out, const void* table, const int* ids, int n_tokens, int d, int vocab, int table_dtype,
                  float scale, int* status, void* stream);
int imp_swiglu(void* out, const void* gate_up, int n_tokens, int F, int block, int dtype, void* stream);
int imp_cast(void* dst, int dst_dtype, const void* src, int src_dtype, int64_t n, void* stream);
int imp_random_fill(void* out, int dtype, int64_t n, uint64_t tensor_seed, int mode, float std, float norm_std,
                    int round_bf16, void* stream);
int imp_tensor_stats(const void* x, int dtype, int64_t n, float* out5, void* stream);

int imp_add_rmsnorm(float* h, const void* branch, const void* w, void* out, const int* rows, int n_out_rows, int d,
                    float eps, float weight_offset, int act_dtype, int w_dtype, int write_h, void* stream);
int imp_add_rmsnorm_split(float* h, const float* part, int64_t split_stride, int n_splits, const void* w, void* out,
                          const int* rows, int n_out_rows, int d, float eps, float weight_offset, int act_dtype,
                          int w_dtype, int write_h, void* stream);
int imp_rmsnorm_rows(const void* x, int64_t x_stride, const void* w, void* out, int64_t out_stride, int n_rows, int d,
                     float eps, float weight_offset, int act_dtype, int w_dtype, void* stream);

int imp_qk_norm_rope_kv_write(void* qkv, int64_t row_stride, int n_tokens, int Hq, int Hkv, int Dh, const void* q_norm_w,
                              const void* k_norm_w, float eps, float weight_offset, int w_dtype, const float* cos_tab,
                              const float* sin_tab, int rot_dim, int max_pos, const int* positions,
                              const int* seq_of_token, const int* block_table, int bt_stride, int n_seqs, void* k_cache,
                              void* v_cache, int page_size, int num_pages, int act_dtype, int* status, void* stream);

int imp_paged_attention_generic(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* k_cache,
                                const void* v_cache, const int* block_table, int bt_stride, const int* seq_of_token,
                                const int* positions, int n_tokens, int n_seqs, int Hq, int Hkv, int Dh, int page_size,
                                int num_pages, float scale, int window, int dtype, int* status, void* stream);

int imp_gemm_f32(float* C, int64_t ldc, const float* A, int64_t lda, const float* W, int64_t ldw, int M, int N, int K,
                 void* stream);
int imp_gemm_bf16_plain(void* C, int64_t ldc, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, int M,
                        int N, int K, void* stream);
int imp_gemm_bf16_small_m(void* C, int64_t ldc, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw,
                          int M, int N, int K, void* stream);
int imp_gemm_bf16_stream(void* C, int64_t ldc, int out_dtype, const void* A, int64_t lda, const void* W, int64_t ldw, int M,
                         int N, int K, void* stream);
int imp_gemm_bf16_stream_swiglu(void* C, int64_t ldc, const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N,
                                int K, void* stream);
int imp_gemm_bf16_tc_splits(int M, int N, int K);
int imp_gemm_bf16_tc_partials(float* scratch, const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N, int K, int* status,
                              void* stream);
int imp_gemm_bf16_tc(void* C, int64_t ldc, int epilogue, const void* A, int64_t lda, const void* W, int64_t ldw, int M,
                     int N, int K, int* status, void* stream);
int64_t imp_gemm_bf16_tc_swap_scratch_floats(int M, int N, int K, int epilogue);
int imp_gemm_bf16_tc_swap(void* C, int64_t ldc, int epilogue, const void* A, int64_t lda, const void* W, int64_t ldw, int M,
                          int N, int K, float* scratch, int* status, void* stream);
int imp_gemm_bf16_tc_swap_splits(int M, int N, int K);
int imp_gemm_bf16_tc_swap_partials(float* scratch, const void* A, int64_t lda, const void* W, int64_t ldw, int M, int N,
                                   int K, int* status, void* stream);
int imp_gemm_bf16_tc_swap_sum(void* C, int64_t ldc, int epilogue, const float* scratch, int M, int N, int splits,
                              void* stream);
int imp_gemm_bf16_tc_qkv_rope(const void* A, int64_t lda, const void* W, int64_t ldw, int M, int K, int Hq, int Hkv, int Dh,
                              const float* q_norm_w, const float* k_norm_w, float eps, const float* cos_tab,
                              const float* sin_tab, int max_pos, const int* positions, const int* seq_of_token,
                              const int* block_table, int bt_stride, int n_seqs, void* q_out, int64_t q_stride,
                              void* k_cache, void* v_cache, int page_size, int num_pages, int* status, void* stream);

int imp_argmax_scratch_words(int n_rows);
int imp_argmax(const float* logits, int64_t ld, int n_rows, int V, int* out, void* scratch, void* stream);
int imp_apply_penalties(float* logits, int64_t ld, int n_rows, int V, const int* history, const int* hist_start,
                        int max_hist, const float* rep, const float* freq, const float* pres, int* counts_scratch,
                        void* stream);
int imp_sample(const float* logits, int64_t ld, int n_rows, int V, const float* temperature, const int* top_k,
               const float* top_p, const float* min_p, const float* uniform, int* out, void* stream);
int imp_sparse_subtract(float* logits, int64_t ld, int n_rows, int V, const int* rows, const int* tokens,
                        const float* values, int n, void* stream);
int imp_typical_filter(float* logits, int64_t ld, int n_rows, int V, const float* typical_p, const float* min_p,
                       void* stream);
int imp_sample_mirostat(const float* logits, int64_t ld, int n_rows, int V, const int* active, const float* temperature,
                        const float* mu, const float* uniform, int* out, float* surprise, void* stream);
}

// Epilogues of the tcgen05 products.
enum { TC_OUT_BF16 = 0, TC_OUT_F32 = 1, TC_OUT_SWIGLU = 2 };
