// The C API: handle lifetime, argument checks, and the translation of exceptions into error codes
// (the reference's src/api/imp_api.cpp:128-169, 224-294, 573-753 does the same over its engine).
#include <cstring>
#include <mutex>

#include "engine.hpp"
#include "ops.hpp"

using namespace imp;

namespace imp {
void register_foreign_part(const std::string& category, const std::string& kind, const ImpPartVTable& vt);
void set_part_error(const char* m);
}  // namespace imp

struct ImpModel_T {
    std::unique_ptr<HostModel> m;
    std::string text;
};
struct ImpContext_T {
    std::unique_ptr<Engine> e;
    std::string text;
};
struct ImpCache_T {
    std::unique_ptr<CacheManager> c;
    std::string text;
};
struct ImpScheduler_T {
    std::unique_ptr<Scheduler> s;
    CacheManager* cache = nullptr;
    StepPlan plan;
    std::string text;
};
struct ImpBench_T {
    std::unique_ptr<DeviceContext> dev;
    std::unique_ptr<Sampler> sampler;
    int64_t sampler_vocab = 0;
    int sampler_rows = 0;
    std::unique_ptr<CacheManager> cache;
    std::unique_ptr<Stepper> stepper;
    std::unique_ptr<WeightStore> store;
    std::unique_ptr<PartFactory> factory;
    std::vector<TilingSpec> tilings;
    ImpCacheView view{};
    bool prepared = false;
};

namespace {
thread_local std::string g_message;
thread_local std::string g_text;   // strings handed out by functions without a handle

ImpError report(const std::exception* e, ImpError code) {
    g_message = e ? e->what() : "unknown error";
    return code;
}

#define IMP_TRY try {
#define IMP_CATCH                                         \
    g_message.clear();                                    \
    return IMP_SUCCESS;                                   \
    }                                                     \
    catch (const imp::Error& e) {                         \
        return report(&e, e.code);                        \
    }                                                     \
    catch (const std::bad_alloc& e) {                     \
        return report(&e, IMP_ERROR_OUT_OF_MEMORY);       \
    }                                                     \
    catch (const std::exception& e) {                     \
        return report(&e, IMP_ERROR_INTERNAL);            \
    }                                                     \
    catch (...) {                                         \
        return report(nullptr, IMP_ERROR_INTERNAL);       \
    }

void need_arg(bool cond, const char* what) {
    if (!cond) fail(IMP_ERROR_INVALID_ARG, what);
}

int write_outputs(const std::vector<ImpStepOutput>& outs, ImpStepOutput* out, int max_out) {
    const int n = (int)std::min<size_t>(outs.size(), (size_t)std::max(max_out, 0));
    for (int i = 0; i < n; ++i) out[i] = outs[(size_t)i];
    return n;
}

std::vector<CacheSpec> parse_cache_specs(const char* json) {
    need_arg(json != nullptr, "cache specs must be given as a JSON list");
    std::vector<CacheSpec> specs;
    const Json list = Json::parse(json, "cache specs");
    for (const auto& j : list.items()) specs.push_back(CacheSpec::from_json(j));
    return specs;
}
}  // namespace

extern "C" {

// --------------------------------------------------------------------------------------- basics
IMP_EXPORT const char* imp_error_string(ImpError err) {
    switch (err) {
        case IMP_SUCCESS: return "success";
        case IMP_ERROR_INVALID_ARG: return "invalid argument";
        case IMP_ERROR_OUT_OF_MEMORY: return "out of memory";
        case IMP_ERROR_CUDA: return "CUDA error";
        case IMP_ERROR_FILE_NOT_FOUND: return "file not found";
        case IMP_ERROR_INVALID_MODEL: return "invalid model";
        case IMP_ERROR_UNSUPPORTED: return "unsupported";
        case IMP_ERROR_INTERNAL: return "internal error";
        case IMP_ERROR_CANCELLED: return "cancelled";
    }
    return "unknown error";
}
IMP_EXPORT const char* imp_error_message(void) { return g_message.c_str(); }
IMP_EXPORT const char* imp_version(void) { return "0.2.0"; }

IMP_EXPORT ImpConfig imp_config_default(void) {
    // defaults of the reference where it has the field (src/api/imp_api.cpp:35-72)
    ImpConfig c{};
    c.device_id = 0;
    c.kv_cache_max_blocks = 0;
    c.kv_cache_tokens = 0;
    c.kv_block_size = 16;
    c.max_batch_size = 32;
    c.max_seq_len = 4096;
    c.max_batch_tokens = 2048;
    c.prefill_chunk_size = 0;
    c.compute_dtype = IMP_COMPUTE_BF16;
    c.enable_cuda_graphs = 1;
    c.gpu_memory_fraction = 0.8f;
    c.state_slots = 0;
    c.lookahead = 1;
    return c;
}

IMP_EXPORT ImpGenerateParams imp_generate_params_default(void) {
    // src/api/imp_api.cpp:76-102
    ImpGenerateParams p{};
    p.temperature = 0.7f;
    p.top_p = 0.9f;
    p.top_k = 40;
    p.max_tokens = 256;
    p.seed = -1;
    p.min_p = 0.f;
    p.typical_p = 1.f;
    p.repetition_penalty = 1.f;
    p.frequency_penalty = 0.f;
    p.presence_penalty = 0.f;
    p.repeat_last_n = 0;
    p.dry_multiplier = 0.f;
    p.dry_base = 1.75f;
    p.dry_allowed_length = 2;
    p.dry_penalty_last_n = 0;
    p.mirostat = 0;
    p.mirostat_tau = 5.f;
    p.mirostat_eta = 0.1f;
    p.ignore_eos = 0;
    return p;
}

// ---------------------------------------------------------------------------------------- model
IMP_EXPORT ImpError imp_model_load(const char* path, ImpModel* out_model) {
    IMP_TRY
    need_arg(path && out_model, "imp_model_load: path and out_model must not be null");
    *out_model = nullptr;
    auto h = std::make_unique<ImpModel_T>();
    h->m = HostModel::load(path);
    *out_model = h.release();
    IMP_CATCH
}

IMP_EXPORT ImpError imp_model_random(const char* config, int64_t seed, float std, float norm_std, ImpModel* out_model) {
    IMP_TRY
    need_arg(config && out_model, "imp_model_random: config and out_model must not be null");
    *out_model = nullptr;
    need_arg(std >= 0 && norm_std >= 0, "imp_model_random: standard deviations must not be negative");
    auto h = std::make_unique<ImpModel_T>();
    h->m = HostModel::make_random(config, seed, std, norm_std);
    *out_model = h.release();
    IMP_CATCH
}

IMP_EXPORT ImpError imp_model_write_random(const char* config, const char* folder, int64_t seed, float std, float norm_std,
                                           const char* store_dtype) {
    IMP_TRY
    need_arg(config && folder, "imp_model_write_random: config and folder must not be null");
    auto m = HostModel::make_random(config, seed, std, norm_std);
    write_random_model(m->config->to_json(), m->plan, folder, seed, std, norm_std, store_dtype ? store_dtype : m->config->torch_dtype);
    IMP_CATCH
}

IMP_EXPORT void imp_model_free(ImpModel model) { delete model; }
IMP_EXPORT const char* imp_model_arch(ImpModel m) { return m ? m->m->arch_text.c_str() : ""; }
IMP_EXPORT int imp_model_n_layers(ImpModel m) { return m ? (int)m->m->config->num_hidden_layers : 0; }
IMP_EXPORT int imp_model_d_model(ImpModel m) { return m ? (int)m->m->config->hidden_size : 0; }
IMP_EXPORT int imp_model_vocab_size(ImpModel m) { return m ? (int)m->m->config->vocab_size : 0; }
IMP_EXPORT int imp_model_max_seq_len(ImpModel m) { return m ? (int)m->m->config->max_position_embeddings : 0; }
IMP_EXPORT const char* imp_model_config_json(ImpModel m) { return m ? m->m->config_text.c_str() : ""; }
IMP_EXPORT const char* imp_model_plan_json(ImpModel m) { return m ? m->m->plan_text.c_str() : ""; }
IMP_EXPORT const char* imp_model_tensor_info_json(ImpModel m, ImpComputeDType dtype) {
    if (!m) return "";
    m->text = m->m->tensor_info(dtype == IMP_COMPUTE_FP32 ? F32 : BF16).dump();
    return m->text.c_str();
}

// -------------------------------------------------------------------------------------- context
IMP_EXPORT ImpError imp_context_create(ImpModel model, const ImpConfig* config, ImpContext* out_ctx) {
    IMP_TRY
    need_arg(model && config && out_ctx, "imp_context_create: model, config and out_ctx must not be null");
    *out_ctx = nullptr;
    auto h = std::make_unique<ImpContext_T>();
    h->e = std::make_unique<Engine>(*model->m, *config);
    *out_ctx = h.release();
    IMP_CATCH
}

IMP_EXPORT void imp_context_free(ImpContext ctx) {
    if (ctx && ctx->e) {
        try {
            ctx->e->make_current();
        } catch (...) {
        }
    }
    delete ctx;
}

IMP_EXPORT ImpError imp_context_reset(ImpContext ctx) {
    IMP_TRY
    need_arg(ctx != nullptr, "imp_context_reset: ctx must not be null");
    ctx->e->make_current();
    ctx->e->reset();
    IMP_CATCH
}

IMP_EXPORT ImpError imp_context_set_eos(ImpContext ctx, const int32_t* ids, int n) {
    IMP_TRY
    need_arg(ctx && (ids || n == 0) && n >= 0, "imp_context_set_eos: null argument");
    ctx->e->set_eos(std::vector<int>(ids, ids + n));
    IMP_CATCH
}

IMP_EXPORT ImpError imp_context_check(ImpContext ctx) {
    IMP_TRY
    need_arg(ctx != nullptr, "imp_context_check: ctx must not be null");
    ctx->e->check_invariants();
    IMP_CATCH
}

IMP_EXPORT ImpError imp_context_timer_start(ImpContext ctx) {
    IMP_TRY
    need_arg(ctx != nullptr, "imp_context_timer_start: ctx must not be null");
    ctx->e->make_current();
    ctx->e->timer_start();
    IMP_CATCH
}

IMP_EXPORT ImpError imp_context_timer_stop(ImpContext ctx, float* out_ms) {
    IMP_TRY
    need_arg(ctx && out_ms, "imp_context_timer_stop: ctx and out_ms must not be null");
    ctx->e->make_current();
    *out_ms = ctx->e->timer_stop();
    IMP_CATCH
}

IMP_EXPORT const char* imp_context_info_json(ImpContext ctx) {
    if (!ctx) return "";
    try {
        ctx->text = ctx->e->info_json().dump();
    } catch (const std::exception& e) {
        ctx->text = std::string("{\"error\": \"") + e.what() + "\"}";
    }
    return ctx->text.c_str();
}

// ----------------------------------------------------------------------------------- generation
IMP_EXPORT ImpError imp_submit(ImpContext ctx, const int32_t* tokens, int n_tokens, const ImpGenerateParams* params, int64_t* out_id) {
    IMP_TRY
    need_arg(ctx && tokens && out_id, "imp_submit: ctx, tokens and out_id must not be null");
    const ImpGenerateParams p = params ? *params : imp_generate_params_default();
    ImpRequestStatus status = IMP_REQUEST_WAITING;
    *out_id = ctx->e->submit(tokens, n_tokens, p, &status);
    if (status == IMP_REQUEST_OUT_OF_MEMORY)
        fail(IMP_ERROR_OUT_OF_MEMORY, "request " + std::to_string(*out_id) + ": prompt plus max_tokens needs more cache pages than the pool holds");
    IMP_CATCH
}

IMP_EXPORT ImpError imp_cancel(ImpContext ctx, int64_t id) {
    IMP_TRY
    need_arg(ctx != nullptr, "imp_cancel: ctx must not be null");
    need_arg(ctx->e->request(id) != nullptr, "imp_cancel: unknown request");
    ctx->e->cancel(id);
    IMP_CATCH
}

IMP_EXPORT ImpError imp_step(ImpContext ctx, ImpStepOutput* out, int max_out, int* n_out) {
    IMP_TRY
    need_arg(ctx && n_out && (out || max_out == 0), "imp_step: ctx, out and n_out must not be null");
    *n_out = 0;
    ctx->e->make_current();
    *n_out = write_outputs(ctx->e->step(), out, max_out);
    IMP_CATCH
}

IMP_EXPORT ImpError imp_drain(ImpContext ctx, ImpStepOutput* out, int max_out, int* n_out) {
    IMP_TRY
    need_arg(ctx && n_out && (out || max_out == 0), "imp_drain: ctx, out and n_out must not be null");
    *n_out = 0;
    ctx->e->make_current();
    *n_out = write_outputs(ctx->e->drain(), out, max_out);
    IMP_CATCH
}

IMP_EXPORT int imp_has_work(ImpContext ctx) { return ctx && ctx->e->has_work() ? 1 : 0; }

IMP_EXPORT ImpError imp_request_info(ImpContext ctx, int64_t id, ImpRequestInfo* out) {
    IMP_TRY
    need_arg(ctx && out, "imp_request_info: ctx and out must not be null");
    const Request* r = ctx->e->request(id);
    need_arg(r != nullptr, "imp_request_info: unknown request");
    out->status = r->status;
    out->finish_reason = r->finish_reason;
    out->n_prompt = (int)r->prompt.size();
    out->n_output = (int)r->output.size();
    out->n_computed = r->n_computed;
    out->n_preempted = r->n_preempted;
    IMP_CATCH
}

IMP_EXPORT ImpError imp_request_output(ImpContext ctx, int64_t id, int32_t* out_tokens, int max_tokens, int* n_tokens) {
    IMP_TRY
    need_arg(ctx && n_tokens && (out_tokens || max_tokens == 0), "imp_request_output: ctx, out_tokens and n_tokens must not be null");
    const Request* r = ctx->e->request(id);
    need_arg(r != nullptr, "imp_request_output: unknown request");
    const int n = std::min((int)r->output.size(), std::max(max_tokens, 0));
    for (int i = 0; i < n; ++i) out_tokens[i] = r->output[(size_t)i];
    *n_tokens = (int)r->output.size();
    IMP_CATCH
}

IMP_EXPORT ImpError imp_request_release(ImpContext ctx, int64_t id) {
    IMP_TRY
    need_arg(ctx != nullptr, "imp_request_release: ctx must not be null");
    ctx->e->forget(id);
    IMP_CATCH
}

IMP_EXPORT ImpError imp_generate(ImpContext ctx, const int32_t* prompt, int n_prompt, const ImpGenerateParams* params,
                                 int32_t* out_tokens, int max_out, int* n_out) {
    IMP_TRY
    need_arg(ctx && prompt && out_tokens && n_out, "imp_generate: ctx, prompt, out_tokens and n_out must not be null");
    *n_out = 0;
    ctx->e->make_current();
    const ImpGenerateParams p = params ? *params : imp_generate_params_default();
    ImpRequestStatus status = IMP_REQUEST_WAITING;
    const int64_t id = ctx->e->submit(prompt, n_prompt, p, &status);
    if (status == IMP_REQUEST_OUT_OF_MEMORY) {
        ctx->e->forget(id);
        fail(IMP_ERROR_OUT_OF_MEMORY, "the prompt plus max_tokens needs more cache pages than the pool holds");
    }
    const Request* r = ctx->e->request(id);
    while (!r->done()) ctx->e->step();
    if (!ctx->e->has_work() || true) ctx->e->drain();
    const bool ok = r->status == IMP_REQUEST_FINISHED;
    const int n = std::min((int)r->output.size(), std::max(max_out, 0));
    for (int i = 0; i < n; ++i) out_tokens[i] = r->output[(size_t)i];
    *n_out = n;
    ctx->e->forget(id);
    if (!ok) fail(IMP_ERROR_OUT_OF_MEMORY, "the request ran out of cache pages");
    IMP_CATCH
}

IMP_EXPORT ImpError imp_prefill(ImpContext ctx, const int32_t* tokens, int n_tokens, const ImpGenerateParams* params) {
    IMP_TRY
    need_arg(ctx && tokens, "imp_prefill: ctx and tokens must not be null");
    Engine& e = *ctx->e;
    e.make_current();
    e.reset();   // as the reference: a new prefill drops what the context held (src/api/imp_api.cpp:585-590)
    ImpGenerateParams p = params ? *params : imp_generate_params_default();
    ImpRequestStatus status = IMP_REQUEST_WAITING;
    const int64_t id = e.submit(tokens, n_tokens, p, &status);
    if (status == IMP_REQUEST_OUT_OF_MEMORY) fail(IMP_ERROR_OUT_OF_MEMORY, "the prompt needs more cache pages than the pool holds");
    e.single_rid = id;
    e.single_read = 0;
    const Request* r = e.request(id);
    while (r->output.empty() && !r->done()) e.step();
    if (r->output.empty()) fail(IMP_ERROR_OUT_OF_MEMORY, "the prompt ran out of cache pages");
    IMP_CATCH
}

IMP_EXPORT ImpError imp_decode_step(ImpContext ctx, int32_t* out_token) {
    IMP_TRY
    need_arg(ctx && out_token, "imp_decode_step: ctx and out_token must not be null");
    Engine& e = *ctx->e;
    e.make_current();
    const Request* r = e.single_rid >= 0 ? e.request(e.single_rid) : nullptr;
    need_arg(r != nullptr, "imp_decode_step: no request is under way (call imp_prefill first)");
    while (r->output.size() <= e.single_read && !r->done()) e.step();
    if (r->output.size() <= e.single_read) fail(IMP_ERROR_CANCELLED, "the request has ended");
    *out_token = r->output[e.single_read++];
    IMP_CATCH
}

IMP_EXPORT ImpError imp_step_tokens(ImpContext ctx, const ImpStepEntry* entries, int n_entries, float* logits_out, size_t capacity) {
    IMP_TRY
    need_arg(ctx != nullptr, "imp_step_tokens: ctx must not be null");
    ctx->e->make_current();
    ctx->e->step_tokens(entries, n_entries, logits_out, capacity);
    IMP_CATCH
}

IMP_EXPORT ImpError imp_end(ImpContext ctx, int64_t id) {
    IMP_TRY
    need_arg(ctx != nullptr, "imp_end: ctx must not be null");
    ctx->e->end(id);
    IMP_CATCH
}

// ---------------------------------------------------------------------- parts and architectures
IMP_EXPORT ImpError imp_register_part(const char* category, const char* kind, const ImpPartVTable* vtable) {
    IMP_TRY
    need_arg(category && kind && vtable, "imp_register_part: category, kind and vtable must not be null");
    ensure_builtin_parts();
    register_foreign_part(category, kind, *vtable);
    IMP_CATCH
}

IMP_EXPORT ImpError imp_unregister_part(const char* category, const char* kind) {
    IMP_TRY
    need_arg(category && kind, "imp_unregister_part: category and kind must not be null");
    unregister_part_class(category, kind);
    IMP_CATCH
}

IMP_EXPORT const char* imp_known_parts(const char* category) {
    try {
        g_text = Json::array_of(known_parts(category ? category : "")).dump();
    } catch (const std::exception&) {
        g_text = "[]";
    }
    return g_text.c_str();
}

IMP_EXPORT void imp_part_set_error(const char* message) { set_part_error(message); }

IMP_EXPORT ImpError imp_part_forward(ImpPart part, ImpCall* call) {
    IMP_TRY
    need_arg(part && call && call->batch && call->batch->step, "imp_part_forward: part, call and call->batch must not be null");
    Step& st = *(Step*)call->batch->step;
    ((Part*)part)->call(st, *call);
    IMP_CATCH
}

IMP_EXPORT void* imp_step_alloc(void* step, size_t bytes) {
    if (!step) return nullptr;
    try {
        return ((Step*)step)->rt->arena->alloc(bytes);
    } catch (const std::exception& e) {
        g_message = e.what();
        return nullptr;
    }
}

IMP_EXPORT ImpError imp_register_architecture(const char* name, ImpPlanFn plan, void* user) {
    IMP_TRY
    need_arg(name && plan, "imp_register_architecture: name and plan must not be null");
    Architecture a;
    a.name = name;
    const std::string arch_name = name;
    a.parse_config = [](const Json& d, const std::string& where) -> std::shared_ptr<ModelConfig> {
        auto c = std::make_shared<ModelConfig>();
        ModelConfig::read_base(*c, d, where);
        return c;
    };
    a.plan = [plan, user, arch_name](const Json& d) {
        set_part_error("");
        const std::string text = d.dump();
        const char* p = plan(user, text.c_str());
        if (!p) fail(IMP_ERROR_INVALID_MODEL, "the plan function of architecture '" + arch_name + "' failed: " + imp_error_message());
        return ModelPlan::from_json(Json::parse(p, "plan of " + arch_name));
    };
    register_architecture(a, false);
    IMP_CATCH
}

IMP_EXPORT ImpError imp_unregister_architecture(const char* name) {
    IMP_TRY
    need_arg(name != nullptr, "imp_unregister_architecture: name must not be null");
    unregister_architecture(name);
    IMP_CATCH
}

IMP_EXPORT const char* imp_known_architectures(void) {
    g_text = Json::array_of(known_architectures()).dump();
    return g_text.c_str();
}

IMP_EXPORT ImpError imp_config_parse(const char* config_json, const char* where, const char** out_json) {
    IMP_TRY
    need_arg(config_json && out_json, "imp_config_parse: config_json and out_json must not be null");
    std::string w = where ? where : "config.json", folder;
    Json d = read_config_json(config_json, where ? nullptr : &w, &folder);
    g_text = architecture_of(d, w).parse_config(d, w)->to_json().dump();
    *out_json = g_text.c_str();
    IMP_CATCH
}

IMP_EXPORT ImpError imp_plan_for_config(const char* config_json, const char** out_json) {
    IMP_TRY
    need_arg(config_json && out_json, "imp_plan_for_config: config_json and out_json must not be null");
    std::string w, folder;
    Json d = read_config_json(config_json, &w, &folder);
    const Architecture& a = architecture_of(d, w);
    a.parse_config(d, w);
    ModelPlan p = a.plan(d);
    p.expected_tensors();   // the plan must name known parts and every tensor they need
    g_text = p.to_json().dump();
    *out_json = g_text.c_str();
    IMP_CATCH
}

IMP_EXPORT ImpError imp_plan_expected_tensors(const char* plan_json, const char** out_json) {
    IMP_TRY
    need_arg(plan_json && out_json, "imp_plan_expected_tensors: plan_json and out_json must not be null");
    ModelPlan p = ModelPlan::from_json(Json::parse(plan_json, "plan"));
    Json j = Json::object();
    for (const auto& e : p.expected_tensors()) j[e.first] = e.second.to_json();
    g_text = j.dump();
    *out_json = g_text.c_str();
    IMP_CATCH
}

IMP_EXPORT void imp_set_variant_resolver(const char* (*fn)(const char*, int)) { set_variant_resolver(fn); }

// --------------------------------------------------------- single parts and a bare step function
IMP_EXPORT ImpError imp_bench_create(int device_id, ImpComputeDType dtype, const char* cache_specs_json, int page_size, int num_pages,
                                     int slots, int max_tokens, int max_seq_len, ImpBench* out) {
    IMP_TRY
    need_arg(out != nullptr, "imp_bench_create: out must not be null");
    *out = nullptr;
    need_arg(page_size > 0 && num_pages > 0 && slots > 0 && max_tokens > 0 && max_seq_len > 0, "imp_bench_create: sizes must be positive");
    auto b = std::make_unique<ImpBench_T>();
    const int dt = dtype == IMP_COMPUTE_FP32 ? F32 : BF16;
    b->dev = std::make_unique<DeviceContext>(device_id, dt, (size_t)1 << 22, (size_t)1 << 22);
    b->cache = std::make_unique<CacheManager>(parse_cache_specs(cache_specs_json ? cache_specs_json : "[]"), page_size, num_pages, slots);
    b->cache->allocate_storage(dt);
    b->tilings = attention_tilings();
    b->stepper = std::make_unique<Stepper>(nullptr, b->cache.get(), &b->dev->rt, max_tokens, slots, max_seq_len, false, (int64_t)1 << 30, b->tilings);
    b->store = std::make_unique<WeightStore>();
    b->factory = std::make_unique<PartFactory>(&b->dev->rt, b->store.get());
    *out = b.release();
    IMP_CATCH
}

IMP_EXPORT void imp_bench_free(ImpBench b) {
    if (b && b->dev) {
        try {
            b->dev->make_current();
            cudaStreamSynchronize(b->dev->rt.stream);
        } catch (...) {
        }
        b->factory.reset();   // parts before the memory they point into
    }
    delete b;
}

IMP_EXPORT ImpError imp_bench_build_part(ImpBench b, const char* category, const char* spec_json, int n_tensors,
                                         const char* const* names, const ImpTensor* tensors, ImpPart* out) {
    IMP_TRY
    need_arg(b && category && spec_json && out && (n_tensors == 0 || (names && tensors)), "imp_bench_build_part: null argument");
    *out = nullptr;
    b->dev->make_current();
    PartSpec spec = PartSpec::from_json(Json::parse(spec_json, "part spec"), category);
    const PartClass& cls = part_class(category, spec.kind);
    TensorSpecs specs;
    if (cls.tensor_specs) specs = cls.tensor_specs(spec.params);
    std::vector<std::pair<std::string, Tensor>> placed;
    for (int i = 0; i < n_tensors; ++i) {
        std::string role = "matrix";
        bool known = false;
        for (const auto& s : specs)
            if (s.first == names[i]) {
                role = s.second.role;
                known = true;
                std::vector<int64_t> shape(tensors[i].shape, tensors[i].shape + tensors[i].ndim);
                if (shape != s.second.shape)
                    fail(IMP_ERROR_INVALID_ARG, std::string("tensor '") + names[i] + "' has shape " + shape_string(tensors[i]) + ", not what the part expects");
            }
        if (!known) fail(IMP_ERROR_INVALID_ARG, std::string(category) + " '" + spec.kind + "' has no tensor '" + names[i] + "'");
        placed.emplace_back(names[i], place_device_tensor(tensors[i], role, b->dev->rt.dtype, *b->store, b->dev->rt.stream));
    }
    for (const auto& s : specs) {
        bool have = false;
        for (const auto& p : placed) have = have || p.first == s.first;
        if (!have && !s.second.optional) fail(IMP_ERROR_INVALID_ARG, std::string(category) + " '" + spec.kind + "' needs its tensor '" + s.first + "'");
    }
    IMP_CUDA(cudaStreamSynchronize(b->dev->rt.stream));
    // parts without tensors are shared between equal specs, as in a model
    Part* p = (placed.empty() && specs.empty()) ? b->factory->shared(category, spec.to_json()) : b->factory->build(category, spec, placed);
    if (Mixer* m = dynamic_cast<Mixer*>(p)) {
        m->tiling_ids.clear();
        for (const TilingSpec& t : m->tilings()) {
            auto it = std::find(b->tilings.begin(), b->tilings.end(), t);
            if (it == b->tilings.end()) fail(IMP_ERROR_UNSUPPORTED, "this mixer wants a tiling the bare step function does not fill");
            m->tiling_ids.push_back((int)(it - b->tilings.begin()));
        }
    }
    *out = (ImpPart)p;
    IMP_CATCH
}

IMP_EXPORT ImpError imp_bench_build_block(ImpBench b, const char* kind, const char* params_json, int n_parts,
                                          const char* const* slot_names, const ImpPart* parts, ImpPart* out) {
    IMP_TRY
    need_arg(b && kind && out && (n_parts == 0 || (slot_names && parts)), "imp_bench_build_block: null argument");
    *out = nullptr;
    b->dev->make_current();
    PartSpec spec;
    spec.kind = kind;
    if (params_json && *params_json) spec.params = Json::parse(params_json, "block params");
    const PartClass& cls = part_class("block", spec.kind);
    std::vector<std::pair<std::string, Part*>> given;
    for (int i = 0; i < n_parts; ++i) given.emplace_back(slot_names[i], (Part*)parts[i]);
    if (cls.part_slots)
        for (const auto& slot : cls.part_slots(spec.params)) {
            bool have = false;
            for (const auto& g : given) have = have || g.first == slot.name;
            if (!have) fail(IMP_ERROR_INVALID_ARG, std::string("block '") + kind + "' needs a part in its slot '" + slot.name + "'");
        }
    *out = (ImpPart)b->factory->build("block", spec, {}, given);
    IMP_CATCH
}

IMP_EXPORT void imp_bench_free_part(ImpBench, ImpPart) { /* parts live as long as the bench that built them */ }

IMP_EXPORT ImpError imp_bench_prepare(ImpBench b, const ImpStepEntry* entries, int n_entries, const ImpBatchView** out) {
    IMP_TRY
    need_arg(b && entries && out, "imp_bench_prepare: null argument");
    b->dev->make_current();
    std::vector<StepEntryView> views;
    for (int i = 0; i < n_entries; ++i)
        views.push_back(StepEntryView{entries[i].id, entries[i].tokens, entries[i].n_tokens, entries[i].want, entries[i].n_want});
    b->dev->arena->begin_step(b->dev->rt.stream);
    b->dev->arena->next_layer();
    Step& st = b->stepper->prepare(views.data(), n_entries);
    b->prepared = true;
    *out = &st.view;
    IMP_CATCH
}

IMP_EXPORT ImpError imp_bench_cache_view(ImpBench b, int position, int writes, const ImpCacheView** out) {
    IMP_TRY
    need_arg(b && out && b->prepared, "imp_bench_cache_view: prepare a batch first");
    need_arg(position >= 0 && position < (int)b->cache->layer_ref().size(), "imp_bench_cache_view: no such run position");
    b->view = b->cache->layer_view(position, b->dev->rt.dtype);
    b->view.writes = writes ? 1 : 0;
    if (b->view.kind == 1) {
        Step& st = b->stepper->current();
        b->view.block_table = st.block_tables.at((size_t)b->cache->layer_ref()[(size_t)position].group);
        b->view.bt_stride = st.bt_stride;
    }
    *out = &b->view;
    IMP_CATCH
}

IMP_EXPORT ImpError imp_bench_commit(ImpBench b) {
    IMP_TRY
    need_arg(b && b->prepared, "imp_bench_commit: prepare a batch first");
    b->stepper->commit(b->stepper->current());
    b->prepared = false;
    IMP_CATCH
}

IMP_EXPORT ImpError imp_bench_end(ImpBench b, int64_t id) {
    IMP_TRY
    need_arg(b != nullptr, "imp_bench_end: null argument");
    b->cache->release(id);
    IMP_CATCH
}

IMP_EXPORT ImpError imp_bench_sync(ImpBench b) {
    IMP_TRY
    need_arg(b != nullptr, "imp_bench_sync: null argument");
    b->dev->make_current();
    b->stepper->check_device_status("part");
    IMP_CATCH
}

IMP_EXPORT void* imp_bench_stream(ImpBench b) { return b ? (void*)b->dev->rt.stream : nullptr; }
IMP_EXPORT const char* imp_bench_cache_info_json(ImpBench b) {
    if (!b) return "";
    g_text = b->cache->info_json().dump();
    return g_text.c_str();
}

IMP_EXPORT float imp_uniform_for(uint64_t seed, int64_t step) { return uniform_for(seed, step); }

IMP_EXPORT int imp_dry_penalties(const int32_t* tokens, int n, float multiplier, float base, int allowed_length, int last_n,
                                 int32_t* out_tokens, float* out_values, int max_out) {
    if (!tokens || n <= 0) return 0;
    int k = 0;
    for (const auto& kv : dry_penalties(std::vector<int32_t>(tokens, tokens + n), multiplier, base, allowed_length, last_n)) {
        if (k < max_out && out_tokens && out_values) {
            out_tokens[k] = kv.first;
            out_values[k] = kv.second;
        }
        ++k;
    }
    return k;
}

IMP_EXPORT ImpError imp_bench_sample(ImpBench b, void* logits, int64_t ld, int n_rows, int vocab, const ImpGenerateParams* params,
                                     const int64_t* seeds, const int64_t* steps, const int32_t* history, const int32_t* hist_start,
                                     float* mu_inout, int32_t* out_tokens) {
    IMP_TRY
    need_arg(b && logits && params && seeds && steps && out_tokens && n_rows > 0 && vocab > 0, "imp_bench_sample: null argument");
    b->dev->make_current();
    if (!b->sampler || b->sampler_vocab != vocab || b->sampler_rows < n_rows) {
        b->sampler = std::make_unique<Sampler>(vocab, std::max(n_rows, 8), &b->dev->rt);
        b->sampler_vocab = vocab;
        b->sampler_rows = std::max(n_rows, 8);
    }
    b->dev->arena->begin_step(b->dev->rt.stream);
    std::vector<std::unique_ptr<Request>> reqs;
    std::vector<Request*> rows_;
    std::vector<int64_t> st(steps, steps + n_rows);
    for (int r = 0; r < n_rows; ++r) {
        auto q = std::make_unique<Request>();
        q->rid = r;
        q->params = SamplingParams::from(params[r]);
        q->params.validate();
        q->seed = (uint64_t)seeds[r];
        if (history && hist_start) q->prompt.assign(history + hist_start[r], history + hist_start[r + 1]);
        if (mu_inout && mu_inout[r] == mu_inout[r]) {   // NaN: not started yet
            q->has_mu = true;
            q->mirostat_mu = mu_inout[r];
        }
        rows_.push_back(q.get());
        reqs.push_back(std::move(q));
    }
    Tensor lg = tensor2d(logits, F32, n_rows, vocab, ld);
    const int32_t* dev_tokens = b->sampler->sample_device(lg, rows_, st);
    IMP_CUDA(cudaMemcpyAsync(out_tokens, dev_tokens, (size_t)n_rows * 4, cudaMemcpyDeviceToHost, b->dev->rt.stream));
    IMP_CUDA(cudaStreamSynchronize(b->dev->rt.stream));
    if (mu_inout)
        for (int r = 0; r < n_rows; ++r)
            if (rows_[(size_t)r]->has_mu) mu_inout[r] = rows_[(size_t)r]->mirostat_mu;
    IMP_CATCH
}

// ------------------------------------------------------------- host components, without a device
IMP_EXPORT ImpError imp_cache_create(const char* cache_specs_json, int page_size, int num_pages, int slots, int max_pages_per_seq,
                                     ImpCache* out) {
    IMP_TRY
    need_arg(out != nullptr, "imp_cache_create: out must not be null");
    *out = nullptr;
    auto h = std::make_unique<ImpCache_T>();
    h->c = std::make_unique<CacheManager>(parse_cache_specs(cache_specs_json), page_size, num_pages, slots, max_pages_per_seq);
    *out = h.release();
    IMP_CATCH
}
IMP_EXPORT void imp_cache_free(ImpCache c) { delete c; }
IMP_EXPORT ImpError imp_cache_add_request(ImpCache c, int64_t id, int* out_slot) {
    IMP_TRY
    need_arg(c != nullptr, "imp_cache_add_request: null argument");
    const int slot = c->c->add_request(id);
    if (out_slot) *out_slot = slot;
    IMP_CATCH
}
IMP_EXPORT ImpError imp_cache_reserve(ImpCache c, int64_t id, int new_len) {
    IMP_TRY
    need_arg(c != nullptr, "imp_cache_reserve: null argument");
    c->c->reserve(id, new_len);
    IMP_CATCH
}
IMP_EXPORT ImpError imp_cache_commit(ImpCache c, int64_t id, int new_len, int* n_freed) {
    IMP_TRY
    need_arg(c != nullptr, "imp_cache_commit: null argument");
    const int n = c->c->commit(id, new_len);
    if (n_freed) *n_freed = n;
    IMP_CATCH
}
IMP_EXPORT ImpError imp_cache_release(ImpCache c, int64_t id) {
    IMP_TRY
    need_arg(c != nullptr, "imp_cache_release: null argument");
    c->c->release(id);
    IMP_CATCH
}
IMP_EXPORT ImpError imp_cache_check(ImpCache c) {
    IMP_TRY
    need_arg(c != nullptr, "imp_cache_check: null argument");
    c->c->check_invariants();
    IMP_CATCH
}
IMP_EXPORT const char* imp_cache_info_json(ImpCache c) {
    if (!c) return "";
    c->text = c->c->info_json().dump();
    return c->text.c_str();
}

IMP_EXPORT ImpError imp_scheduler_create(ImpCache c, int max_batch_size, int max_batch_tokens, int prefill_chunk_size, int max_seq_len,
                                         ImpScheduler* out) {
    IMP_TRY
    need_arg(c && out, "imp_scheduler_create: null argument");
    auto h = std::make_unique<ImpScheduler_T>();
    h->cache = c->c.get();
    h->s = std::make_unique<Scheduler>(h->cache, max_batch_size, max_batch_tokens, prefill_chunk_size, max_seq_len);
    *out = h.release();
    IMP_CATCH
}
IMP_EXPORT void imp_scheduler_free(ImpScheduler s) { delete s; }

IMP_EXPORT ImpError imp_scheduler_add(ImpScheduler s, int64_t id, const int32_t* prompt, int n_prompt, const ImpGenerateParams* params,
                                      const int32_t* eos_ids, int n_eos, int* out_status) {
    IMP_TRY
    need_arg(s && (prompt || n_prompt == 0), "imp_scheduler_add: null argument");
    const ImpGenerateParams p = params ? *params : imp_generate_params_default();
    auto req = std::make_unique<Request>();
    req->rid = id;
    if (n_prompt > 0) req->prompt.assign(prompt, prompt + n_prompt);
    req->max_tokens = p.max_tokens;
    req->params = SamplingParams::from(p);
    req->ignore_eos = p.ignore_eos != 0;
    for (int i = 0; i < n_eos; ++i) req->eos_token_ids.push_back(eos_ids[i]);
    Request* r = s->s->add(std::move(req));
    if (out_status) *out_status = r->status;
    IMP_CATCH
}

IMP_EXPORT ImpError imp_scheduler_cancel(ImpScheduler s, int64_t id) {
    IMP_TRY
    need_arg(s != nullptr, "imp_scheduler_cancel: null argument");
    s->s->cancel(id);
    IMP_CATCH
}

IMP_EXPORT ImpError imp_scheduler_schedule(ImpScheduler s, const char** out_json) {
    IMP_TRY
    need_arg(s && out_json, "imp_scheduler_schedule: null argument");
    s->plan = s->s->schedule();
    Json j = Json::object(), es = Json::array(), pre = Json::array(), failed = Json::array();
    for (const auto& e : s->plan.entries) {
        Json o = Json::object();
        o["id"] = e.request->rid;
        o["start"] = e.start;
        o["n_tokens"] = e.n_tokens;
        o["samples"] = e.samples;
        es.push(o);
    }
    for (const Request* r : s->plan.preempted) pre.push(Json(r->rid));
    for (const Request* r : s->plan.failed) failed.push(Json(r->rid));
    j["entries"] = es;
    j["preempted"] = pre;
    j["failed"] = failed;
    j["pages"] = s->plan.pages;
    s->text = j.dump();
    *out_json = s->text.c_str();
    IMP_CATCH
}

IMP_EXPORT ImpError imp_scheduler_complete(ImpScheduler s, const int32_t* tokens, int n_tokens, const char** out_json) {
    IMP_TRY
    need_arg(s && (tokens || n_tokens == 0), "imp_scheduler_complete: null argument");
    std::vector<int32_t> sampled(tokens, tokens + n_tokens);
    Json fin = Json::array();
    for (const Request* r : s->s->complete_step(s->plan, sampled)) fin.push(Json(r->rid));
    s->plan = StepPlan();
    s->text = fin.dump();
    if (out_json) *out_json = s->text.c_str();
    IMP_CATCH
}

IMP_EXPORT const char* imp_scheduler_info_json(ImpScheduler s) {
    if (!s) return "";
    s->text = s->s->info_json().dump();
    return s->text.c_str();
}

}  // extern "C"
