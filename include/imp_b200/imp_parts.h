/* imp_b200 — extension interface: part kinds and architectures registered from outside the library.
 *
 * A model is a plan (JSON): parts by kind, their parameters, the checkpoint names of their
 * tensors, the layers, and the order in which layers run.  An architecture is a function from
 * config.json to such a plan.  A part kind is a table of functions.  Both can be registered at
 * run time, from C or through the Python package, without touching the library's files.
 *
 * The reference has neither: its forward pass is one function that switches on tensor presence
 * (src/graph/executor_forward.cu:2701-3140, src/graph/executor_workspace.cu:2314-2330).
 *
 * Plan JSON:
 *   {"architecture": str, "hidden_size": int, "vocab_size": int, "max_positions": int,
 *    "embedding": PART, "final_norm": PART, "head": PART,
 *    "layers": [{"block": kind, "block_params": {...}, "parts": {slot: PART, ...}, "cache_from": int|null}],
 *    "order": [layer index, ...] | null,
 *    "ignored_tensors": [checkpoint names that may be present and are not read]}
 *   PART = {"kind": str, "params": {...}, "tensors": {local name: checkpoint name}}
 * Tensor specs JSON (what a part expects of its tensors):
 *   {local name: {"shape": [..], "role": "matrix"|"norm"|"vector"|"int_table",
 *                 "init": "normal"|"one_plus_normal"|"zeros"|"arange_mod", "optional": bool}}
 * Cache spec JSON (what a mixer asks of the cache):
 *   null | {"kind": "paged", "num_kv_heads": int, "head_dim": int, "window": int}
 *        | {"kind": "state", "tensors": [{"name": str, "shape": [..], "dtype": "float32"|"bfloat16"|"int32"}]}
 * Block slots JSON: [{"name": slot, "category": "mixer"|"feed_forward"|"norm"}, ...] (at most one mixer).
 */
#ifndef IMP_B200_IMP_PARTS_H
#define IMP_B200_IMP_PARTS_H

#include "imp.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { IMP_ELEM_F32 = 0, IMP_ELEM_BF16 = 1, IMP_ELEM_I32 = 2 };

/* A view of device memory: up to 4 dimensions, dense but for the stride of the first one. */
typedef struct {
    void* data;
    int32_t dtype;                 /* IMP_ELEM_* */
    int32_t ndim;
    int64_t shape[4];
    int64_t stride0;               /* elements between consecutive indices of dimension 0 */
} ImpTensor;

/* What a part sees of the step's batch.  Device arrays are int32. */
typedef struct {
    int32_t n_tokens, n_seqs, n_rows;
    int32_t decode_only;           /* every sequence brings exactly one token */
    int32_t max_q_len, max_kv_len;
    const int32_t* token_ids;      /* [n_tokens] */
    const int32_t* positions;      /* [n_tokens] absolute position of each token in its sequence */
    const int32_t* seq_of_token;   /* [n_tokens] index of the token's sequence in the batch */
    const int32_t* logit_rows;     /* [n_rows] tokens whose logits are wanted */
    const int32_t* q_start;        /* [n_seqs + 1] first token of each sequence in the batch */
    const int32_t* kv_len;         /* [n_seqs] length of each sequence after this step */
    const int32_t* state_slots;    /* [n_seqs] fixed-size state slot of each sequence */
    /* the same on the host, for parts with per-sequence host logic */
    const int32_t* host_q_lens;    /* [n_seqs] */
    const int32_t* host_starts;    /* [n_seqs] length of each sequence before this step */
    const int32_t* host_slots;     /* [n_seqs] */
    void* stream;                  /* cudaStream_t every launch of this step goes to */
    int32_t* status;               /* device status word (0 = ok) */
    int32_t compute_dtype;         /* IMP_ELEM_F32 or IMP_ELEM_BF16: activations and cache */
    void* step;                    /* opaque; for imp_step_alloc */
} ImpBatchView;

/* What a mixer gets of the cache for one run position. */
typedef struct {
    int32_t kind;                  /* 0 none, 1 paged, 2 state */
    int32_t writes;                /* 0: this layer reads another layer's cache */
    /* paged: keys and values [pages, kv_heads, page_size, head_dim] each */
    void* k_pages;
    void* v_pages;
    int32_t num_pages, kv_heads, page_size, head_dim, window;
    const int32_t* block_table;    /* [n_seqs, bt_stride] rows in batch order, -1 = no page */
    int32_t bt_stride;
    /* state: tensors [slots, ...] in the order of the cache spec */
    int32_t n_states;
    ImpTensor states[4];
} ImpCacheView;

typedef struct ImpPart_T* ImpPart;

/* One call of a part.  Which fields are used depends on the part's category:
 *   norm          h [T, d] f32 stream (branch, if given, is added into it first), rows/n_rows
 *                 (optional: produce only those rows and leave h untouched) -> out [n, d]
 *   mixer         x [T, d], batch, cache -> out [T, d]
 *   feed_forward  x [T, d], batch -> out [T, d]
 *   block         h, branch (the pending sum of the block before, data == NULL: none), batch,
 *                 cache -> out [T, d]: the sum this block leaves pending (has_out = 0: none)
 *   embedding     batch -> h [T, d] f32
 *   head          x [R, d] -> out [R, vocab] f32
 *   position      q [T, Hq, Dh], k [T, Hkv, Dh] rewritten in place, batch
 */
typedef struct {
    const ImpBatchView* batch;
    const ImpCacheView* cache;
    ImpTensor h;
    ImpTensor branch;
    ImpTensor x;
    ImpTensor q, k;
    ImpTensor out;
    const int32_t* rows;
    int32_t n_rows;
    int32_t has_out;
} ImpCall;

/* A part kind implemented outside the library.  Strings returned by the first three functions
 * must stay valid until the next call of the same function.  Functions that do not apply to the
 * category may be NULL.  `forward` returns 0, or non-zero after imp_part_set_error(). */
typedef struct {
    void* user;
    const char* (*tensor_specs)(void* user, const char* params_json);
    const char* (*cache_spec)(void* user, const char* params_json);       /* mixers */
    const char* (*part_slots)(void* user, const char* params_json);       /* blocks */
    /* tensors: this part's weights on the device, by local name; parts: a block's built parts by slot */
    void* (*create)(void* user, const char* params_json, int n_tensors, const char* const* tensor_names,
                    const ImpTensor* tensors, int n_parts, const char* const* part_names, const ImpPart* parts,
                    int compute_dtype, int device_id);
    int (*forward)(void* self, ImpCall* call);
    void (*destroy)(void* self);
} ImpPartVTable;

/* category: "mixer", "feed_forward", "norm", "position", "block", "embedding", "head". */
IMP_EXPORT ImpError imp_register_part(const char* category, const char* kind, const ImpPartVTable* vtable);
IMP_EXPORT ImpError imp_unregister_part(const char* category, const char* kind);
IMP_EXPORT const char* imp_known_parts(const char* category);   /* JSON list */
IMP_EXPORT void imp_part_set_error(const char* message);

/* Run a built part (one of the library's or a registered one): what a block does with its parts. */
IMP_EXPORT ImpError imp_part_forward(ImpPart part, ImpCall* call);
/* Device memory that lives until the end of the current layer of the step in `batch->step`. */
IMP_EXPORT void* imp_step_alloc(void* step, size_t bytes);

/* Architectures.  `plan` returns the plan JSON for a config.json text (valid until its next call),
 * or NULL after imp_part_set_error(). */
typedef const char* (*ImpPlanFn)(void* user, const char* config_json);
IMP_EXPORT ImpError imp_register_architecture(const char* name, ImpPlanFn plan, void* user);
IMP_EXPORT ImpError imp_unregister_architecture(const char* name);
IMP_EXPORT const char* imp_known_architectures(void);           /* JSON list */
/* The validated, typed configuration of a config.json text, and the plan its architecture gives. */
IMP_EXPORT ImpError imp_config_parse(const char* config_json, const char* where, const char** out_json);
IMP_EXPORT ImpError imp_plan_for_config(const char* config_json, const char** out_json);
/* Checkpoint tensor name -> spec JSON, over all parts of a plan. */
IMP_EXPORT ImpError imp_plan_expected_tensors(const char* plan_json, const char** out_json);

/* ----------------------------------------------------- single parts and a bare step function */

/* A device context without a model: a stream, a status word, a workspace, a cache manager built
 * from `cache_specs_json` (a list of cache specs, one per run position), and the batch builder of
 * the step function.  For driving single parts and for tests. */
typedef struct ImpBench_T* ImpBench;
IMP_EXPORT ImpError imp_bench_create(int device_id, ImpComputeDType dtype, const char* cache_specs_json, int page_size,
                                     int num_pages, int slots, int max_tokens, int max_seq_len, ImpBench* out);
IMP_EXPORT void imp_bench_free(ImpBench b);
/* Build a part: tensors are device views by local name (copied, converted to the compute type
 * where the loader would, and owned by the part). */
IMP_EXPORT ImpError imp_bench_build_part(ImpBench b, const char* category, const char* spec_json, int n_tensors,
                                         const char* const* names, const ImpTensor* tensors, ImpPart* out);
/* Build a block of kind `kind` over parts this bench built, by slot name. */
IMP_EXPORT ImpError imp_bench_build_block(ImpBench b, const char* kind, const char* params_json, int n_parts,
                                          const char* const* slot_names, const ImpPart* parts, ImpPart* out);
IMP_EXPORT void imp_bench_free_part(ImpBench b, ImpPart part);
/* Reserve cache for the entries and upload the batch arrays (tokens may be NULL: zeros). */
IMP_EXPORT ImpError imp_bench_prepare(ImpBench b, const ImpStepEntry* entries, int n_entries, const ImpBatchView** out);
/* The cache view of a run position for the prepared batch. */
IMP_EXPORT ImpError imp_bench_cache_view(ImpBench b, int position, int writes, const ImpCacheView** out);
/* Record the prepared batch's new lengths (what the step function does after the model ran). */
IMP_EXPORT ImpError imp_bench_commit(ImpBench b);
IMP_EXPORT ImpError imp_bench_end(ImpBench b, int64_t id);
/* Wait for the stream; IMP_ERROR_CUDA with the device's message if the status word is set. */
IMP_EXPORT ImpError imp_bench_sync(ImpBench b);
IMP_EXPORT void* imp_bench_stream(ImpBench b);                  /* the cudaStream_t its work goes to */
IMP_EXPORT const char* imp_bench_cache_info_json(ImpBench b);

/* The batched sampler on logits [n_rows, vocab] (float32, device, row stride `ld`; modified in place):
 * one token per row into `out_tokens` (host).  `history`/`hist_start` ([n_rows + 1] offsets; may be NULL)
 * are each row's tokens so far, for penalties and DRY; `mu_inout` ([n_rows], may be NULL) carries
 * Mirostat's mu (NaN = not started). */
IMP_EXPORT ImpError imp_bench_sample(ImpBench b, void* logits, int64_t ld, int n_rows, int vocab,
                                     const ImpGenerateParams* params, const int64_t* seeds, const int64_t* steps,
                                     const int32_t* history, const int32_t* hist_start, float* mu_inout,
                                     int32_t* out_tokens);
/* The uniform number of draw `step` of a request seeded with `seed`; the DRY penalties of a token
 * history (returns how many tokens are penalised; writes up to `max_out` of them). */
IMP_EXPORT float imp_uniform_for(uint64_t seed, int64_t step);
IMP_EXPORT int imp_dry_penalties(const int32_t* tokens, int n, float multiplier, float base, int allowed_length, int last_n,
                                 int32_t* out_tokens, float* out_values, int max_out);

/* Where the attention libraries (one per head size, built from csrc/variants/) are found: `fn`
 * returns the path of the library built from `source` for a head size, or NULL.  Without a resolver
 * (or when it returns NULL) the folder this library was loaded from is searched. */
IMP_EXPORT void imp_set_variant_resolver(const char* (*fn)(const char* source, int head_dim));

/* ------------------------------------------------------------ host components, without a device */

typedef struct ImpCache_T* ImpCache;
IMP_EXPORT ImpError imp_cache_create(const char* cache_specs_json, int page_size, int num_pages, int slots,
                                     int max_pages_per_seq, ImpCache* out);
IMP_EXPORT void imp_cache_free(ImpCache c);
IMP_EXPORT ImpError imp_cache_add_request(ImpCache c, int64_t id, int* out_slot);
IMP_EXPORT ImpError imp_cache_reserve(ImpCache c, int64_t id, int new_len);
IMP_EXPORT ImpError imp_cache_commit(ImpCache c, int64_t id, int new_len, int* n_freed);
IMP_EXPORT ImpError imp_cache_release(ImpCache c, int64_t id);
IMP_EXPORT ImpError imp_cache_check(ImpCache c);                /* invariants: no page lost or held twice */
IMP_EXPORT const char* imp_cache_info_json(ImpCache c);        /* groups, free pages, tables per request */

typedef struct ImpScheduler_T* ImpScheduler;
IMP_EXPORT ImpError imp_scheduler_create(ImpCache c, int max_batch_size, int max_batch_tokens, int prefill_chunk_size,
                                         int max_seq_len, ImpScheduler* out);
IMP_EXPORT void imp_scheduler_free(ImpScheduler s);
IMP_EXPORT ImpError imp_scheduler_add(ImpScheduler s, int64_t id, const int32_t* prompt, int n_prompt,
                                      const ImpGenerateParams* params, const int32_t* eos_ids, int n_eos, int* out_status);
IMP_EXPORT ImpError imp_scheduler_cancel(ImpScheduler s, int64_t id);
/* Decide the next step (the caller reserves and commits the cache as the step function would).  JSON:
 * {"entries": [{"id", "start", "n_tokens", "samples"}], "preempted": [ids], "failed": [ids]} */
IMP_EXPORT ImpError imp_scheduler_schedule(ImpScheduler s, const char** out_json);
/* Record the scheduled step with one sampled token per sampling entry, in entry order.
 * JSON list of the ids that finished. */
IMP_EXPORT ImpError imp_scheduler_complete(ImpScheduler s, const int32_t* tokens, int n_tokens, const char** out_json);
IMP_EXPORT const char* imp_scheduler_info_json(ImpScheduler s);   /* waiting, running, requests */

#ifdef __cplusplus
}
#endif
#endif
