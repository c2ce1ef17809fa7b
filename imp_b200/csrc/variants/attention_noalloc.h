// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in kekzl/imp: it exists for users of this library.
//
// Who needs it: code that runs where cudaMalloc is forbidden or harmful -- a latency-critical
// serving thread that has promised not to touch the allocator after start-up (cudaMalloc and
// cudaFree may synchronise the whole device), a plug-in hosted by a process that owns all device
// memory and hands out none, a callback that runs while another part of the program holds the
// allocator's lock.  The regular entry point, imp_attn_decode, splits long contexts over several
// CTAs and needs scratch memory for the partial results, which its caller has to allocate.  This
// variant brings its own: a fixed buffer of IMP_ATTN_NOALLOC_SCRATCH_FLOATS floats (4 MiB) that
// is part of the library image, so every GPU that loads the library holds it until the process
// exits.  The caller still passes inputs and outputs; the function itself calls no cudaMalloc,
// cudaFree or allocating library routine.
//
// Limits and rules:
//   * n_tokens * Hq * n_splits * (head size + 2) must not exceed IMP_ATTN_NOALLOC_SCRATCH_FLOATS
//     (n_splits == 1 needs none); larger requests are refused with an error text, nothing runs.
//   * The first call on a device looks the buffer's device address up (cudaGetSymbolAddress) and
//     sets a kernel attribute.  Make that first call outside any stream capture.
//   * All calls share the one buffer.  Two calls that overlap on the GPU (different streams, or
//     the same call replayed concurrently) race on it; calls on one stream are safe, because the
//     merge of one call finishes before the next call's partial results are written.  Nothing in
//     the buffer has to start at zero: every slot that is read was written earlier in the same
//     call, so the leftovers of the previous call do no harm.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IMP_ATTN_NOALLOC_SCRATCH_FLOATS (1 << 20)

// Same arguments and result as imp_attn_decode, without the scratch pointer.
// Returns 0 on success; a negative value for refused arguments (imp_last_error() has the text),
// a positive cudaError_t if CUDA reported one.
int imp_attn_decode_noalloc(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* k_cache,
                            const void* v_cache, const int* block_table, int bt_stride, const int* seq_of_token,
                            const int* positions, int n_tokens, int n_seqs, int n_q_heads, int n_kv_heads,
                            int page_size, int num_pages, float scale, int window, int n_splits, int* status,
                            void* stream);

#ifdef __cplusplus
}
#endif
