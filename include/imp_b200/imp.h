/* imp_b200 — C API of the engine (one B200 GPU, the Qwen3 dense decoder).
 *
 * In the manner of the reference's include/imp/imp.h:34-143: an opaque model handle, an opaque
 * context with the engine's settings, whole-request generation, and token-level stepping.  This
 * engine has no tokenizer: prompts and outputs are token ids.  New beside the reference's calls:
 * imp_submit / imp_step (continuous batching from the caller's loop) and imp_step_tokens (run
 * given tokens as one batch and return 32-bit logits; nothing is sampled).
 *
 * Threading: a model handle is read-only after creation and may be shared; a context is used
 * from one thread at a time.
 *
 * Errors: every call returns an ImpError; imp_error_message() gives the detail of the last failed
 * call on the calling thread.
 */
#ifndef IMP_B200_IMP_H
#define IMP_B200_IMP_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define IMP_EXPORT __attribute__((visibility("default")))
#else
#define IMP_EXPORT
#endif

/* Codes and meanings of the reference's include/imp/error.h:7-17. */
typedef enum {
    IMP_SUCCESS = 0,
    IMP_ERROR_INVALID_ARG = -1,
    IMP_ERROR_OUT_OF_MEMORY = -2,   /* device memory, or cache pages for a request */
    IMP_ERROR_CUDA = -3,
    IMP_ERROR_FILE_NOT_FOUND = -4,
    IMP_ERROR_INVALID_MODEL = -5,   /* config.json or the checkpoint does not describe a model this engine runs */
    IMP_ERROR_UNSUPPORTED = -6,
    IMP_ERROR_INTERNAL = -7,
    IMP_ERROR_CANCELLED = -8
} ImpError;

IMP_EXPORT const char* imp_error_string(ImpError err);
IMP_EXPORT const char* imp_error_message(void);
IMP_EXPORT const char* imp_version(void);

typedef enum { IMP_COMPUTE_FP32 = 0, IMP_COMPUTE_BF16 = 1 } ImpComputeDType;

typedef struct ImpModel_T* ImpModel;
typedef struct ImpContext_T* ImpContext;

/* ---------------------------------------------------------------------------------- model */

/* `path`: a folder with config.json and model.safetensors (or model.safetensors.index.json and
 * its shards), or the path of config.json itself.  The architecture named by config.json's
 * `architectures[0]` selects the model class.  Names, shapes and element types of every tensor
 * are checked here; one error lists everything that is missing, unexpected or of the wrong
 * shape or type.  Weights reach the device when a context is created. */
IMP_EXPORT ImpError imp_model_load(const char* path, ImpModel* out_model);

/* A model whose tensors are random: matrices N(0, std), norm weights 1 + N(0, norm_std), each
 * tensor a function of (seed, its name).  `config` is a path as above or the JSON text itself. */
IMP_EXPORT ImpError imp_model_random(const char* config, int64_t seed, float std, float norm_std, ImpModel* out_model);

/* Write config.json and model.safetensors with such random tensors into `folder`.
 * `store_dtype`: "bfloat16", "float32", or NULL for the configuration's torch_dtype. */
IMP_EXPORT ImpError imp_model_write_random(const char* config, const char* folder, int64_t seed, float std,
                                           float norm_std, const char* store_dtype);

IMP_EXPORT void imp_model_free(ImpModel model);

IMP_EXPORT const char* imp_model_arch(ImpModel model);     /* e.g. "Qwen3ForCausalLM" */
IMP_EXPORT int imp_model_n_layers(ImpModel model);
IMP_EXPORT int imp_model_d_model(ImpModel model);
IMP_EXPORT int imp_model_vocab_size(ImpModel model);
IMP_EXPORT int imp_model_max_seq_len(ImpModel model);
IMP_EXPORT const char* imp_model_config_json(ImpModel model);  /* the typed configuration, as JSON */
IMP_EXPORT const char* imp_model_plan_json(ImpModel model);    /* parts, sizes, tensor names, run order */
/* checkpoint tensor name -> {"stored", "device", "shape", "role"}: the element type each tensor is
 * stored in and the one it gets on the device under `dtype`. */
IMP_EXPORT const char* imp_model_tensor_info_json(ImpModel model, ImpComputeDType dtype);

/* -------------------------------------------------------------------------------- context */

/* Field names of the reference's ImpConfig (include/imp/config.h:11-81) where it has them;
 * kv_block_size from src/runtime/engine.h:59.  kv_cache_tokens, max_batch_tokens, state_slots,
 * gpu_memory_fraction and lookahead are this engine's. */
typedef struct {
    int device_id;
    size_t kv_cache_max_blocks;    /* pages per cache group; 0 = from kv_cache_tokens, else from memory */
    size_t kv_cache_tokens;        /* pool size in tokens when kv_cache_max_blocks == 0 */
    int kv_block_size;             /* tokens per page */
    int max_batch_size;            /* requests decoded together */
    int max_seq_len;               /* longest context of one request */
    int max_batch_tokens;          /* token budget of one step: decode tokens plus prompt portions */
    int prefill_chunk_size;        /* longest portion of one prompt in a step; 0 = no cut */
    ImpComputeDType compute_dtype;
    int enable_cuda_graphs;        /* capture decode-only steps */
    float gpu_memory_fraction;     /* of free memory to the cache when nothing else sizes it */
    int state_slots;               /* fixed-size state slots; 0 = max_batch_size */
    int lookahead;                 /* queue the next decode step before the last one's tokens are read */
} ImpConfig;

IMP_EXPORT ImpConfig imp_config_default(void);

IMP_EXPORT ImpError imp_context_create(ImpModel model, const ImpConfig* config, ImpContext* out_ctx);
IMP_EXPORT void imp_context_free(ImpContext ctx);

/* Drop every request and give all pages and state slots back. */
IMP_EXPORT ImpError imp_context_reset(ImpContext ctx);

/* The end-of-sequence token ids of requests submitted from now on (default: config.json's eos_token_id). */
IMP_EXPORT ImpError imp_context_set_eos(ImpContext ctx, const int32_t* ids, int n);
/* The cache manager's invariants (no page lost or held twice): IMP_ERROR_INTERNAL names a broken one. */
IMP_EXPORT ImpError imp_context_check(ImpContext ctx);

/* Device time, for measurement: CUDA events on the context's stream.  Work queued between the two calls
 * lies between the two events; imp_context_timer_stop waits for it and gives the milliseconds. */
IMP_EXPORT ImpError imp_context_timer_start(ImpContext ctx);
IMP_EXPORT ImpError imp_context_timer_stop(ImpContext ctx, float* out_ms);

/* State of the context as JSON (cache groups, free pages, run positions, counters, ...). */
IMP_EXPORT const char* imp_context_info_json(ImpContext ctx);

/* ----------------------------------------------------------------------------- generation */

/* Fields and defaults of the reference's ImpGenerateParams (include/imp/imp.h:61-85,
 * src/api/imp_api.cpp:76-102) that apply to an engine without tokenizer, templates or JSON mode. */
typedef struct {
    float temperature;             /* <= 0: greedy */
    float top_p;
    int top_k;
    int max_tokens;
    int64_t seed;                  /* -1 = random */
    float min_p;
    float typical_p;
    float repetition_penalty;
    float frequency_penalty;
    float presence_penalty;
    int repeat_last_n;
    float dry_multiplier;
    float dry_base;
    int dry_allowed_length;
    int dry_penalty_last_n;
    int mirostat;                  /* 0 = off, 2 = Mirostat v2 */
    float mirostat_tau;
    float mirostat_eta;
    int ignore_eos;
} ImpGenerateParams;

IMP_EXPORT ImpGenerateParams imp_generate_params_default(void);

typedef enum {
    IMP_REQUEST_WAITING = 0,
    IMP_REQUEST_RUNNING = 1,
    IMP_REQUEST_FINISHED = 2,
    IMP_REQUEST_CANCELLED = 3,
    IMP_REQUEST_OUT_OF_MEMORY = 4
} ImpRequestStatus;

typedef enum { IMP_FINISH_NONE = 0, IMP_FINISH_EOS = 1, IMP_FINISH_LENGTH = 2, IMP_FINISH_CONTEXT = 3 } ImpFinishReason;

typedef struct {
    int64_t id;
    int32_t token;                 /* -1: the request ended without a token in this step */
    int32_t finished;
    int32_t status;                /* ImpRequestStatus */
    int32_t finish_reason;         /* ImpFinishReason */
} ImpStepOutput;

typedef struct {
    int32_t status;
    int32_t finish_reason;
    int32_t n_prompt;
    int32_t n_output;
    int32_t n_computed;
    int32_t n_preempted;
} ImpRequestInfo;

/* Queue one request.  `*out_id` is its id in this context.  IMP_ERROR_OUT_OF_MEMORY: the prompt
 * plus max_tokens needs more pages than the whole pool holds (the request is not queued). */
IMP_EXPORT ImpError imp_submit(ImpContext ctx, const int32_t* tokens, int n_tokens, const ImpGenerateParams* params,
                               int64_t* out_id);
IMP_EXPORT ImpError imp_cancel(ImpContext ctx, int64_t id);

/* One engine step: admit, run one mixed batch (decode tokens beside prompt portions), sample,
 * finish.  Writes up to `max_out` outputs (at most max_batch_size exist) and their count. */
IMP_EXPORT ImpError imp_step(ImpContext ctx, ImpStepOutput* out, int max_out, int* n_out);
/* Finish a step that was queued ahead, if there is one. */
IMP_EXPORT ImpError imp_drain(ImpContext ctx, ImpStepOutput* out, int max_out, int* n_out);
IMP_EXPORT int imp_has_work(ImpContext ctx);

IMP_EXPORT ImpError imp_request_info(ImpContext ctx, int64_t id, ImpRequestInfo* out);
/* The tokens generated so far (all of them once the request is finished). */
IMP_EXPORT ImpError imp_request_output(ImpContext ctx, int64_t id, int32_t* out_tokens, int max_tokens, int* n_tokens);
/* Forget a finished request's record. */
IMP_EXPORT ImpError imp_request_release(ImpContext ctx, int64_t id);

/* Whole-request generation for one prompt (continuous batching inside, should other requests be
 * queued).  Writes at most `max_out` tokens. */
IMP_EXPORT ImpError imp_generate(ImpContext ctx, const int32_t* prompt, int n_prompt, const ImpGenerateParams* params,
                                 int32_t* out_tokens, int max_out, int* n_out);

/* The reference's token-level pair for one request at a time (include/imp/imp.h:129-143):
 * imp_prefill drops what the context held, runs the prompt and samples the first token with the
 * parameters given; imp_decode_step returns the next token (the first call returns the token the
 * prefill sampled).  IMP_ERROR_CANCELLED once the request has ended. */
IMP_EXPORT ImpError imp_prefill(ImpContext ctx, const int32_t* tokens, int n_tokens, const ImpGenerateParams* params);
IMP_EXPORT ImpError imp_decode_step(ImpContext ctx, int32_t* out_token);

/* ------------------------------------------------------------------------------ replaying */

typedef struct {
    int64_t id;                    /* the caller's request id; a new id starts a request */
    const int32_t* tokens;         /* its next tokens: a portion of a prompt, or one decoded token */
    int n_tokens;
    const int32_t* want;           /* indices into `tokens` whose logits are asked for */
    int n_want;
} ImpStepEntry;

/* Run the entries as ONE batch through the step function (no scheduling, no sampling).  The
 * 32-bit logits of the wanted rows, in the order of the entries and of each `want`, are copied to
 * `logits_out` [sum of n_want, vocab] on the host (`capacity` counts floats).  The requests keep
 * their cache until imp_end. */
IMP_EXPORT ImpError imp_step_tokens(ImpContext ctx, const ImpStepEntry* entries, int n_entries, float* logits_out,
                                    size_t capacity);
IMP_EXPORT ImpError imp_end(ImpContext ctx, int64_t id);

#ifdef __cplusplus
}
#endif
#endif
