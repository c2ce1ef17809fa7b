#include "engine.hpp"

#include <algorithm>
#include <cstring>

#include "diagnostics.hpp"
#include "kernels.h"

namespace imp {

// ------------------------------------------------------------------------------ device context
DeviceContext::DeviceContext(int device_id, int dtype, size_t step_bytes, size_t layer_bytes) {
    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess || n_dev == 0) {
        (void)cudaGetLastError();
        fail(IMP_ERROR_CUDA, "no CUDA device: this engine runs only on a B200-class GPU (no CPU path exists)");
    }
    if (device_id < 0 || device_id >= n_dev)
        fail(IMP_ERROR_INVALID_ARG, "device " + std::to_string(device_id) + " does not exist (" + std::to_string(n_dev) + " devices)");
    IMP_CUDA(cudaSetDevice(device_id));
    const int arch = imp_device_arch();
    if (arch < 0) fail(IMP_ERROR_CUDA, std::string("cannot query the device: ") + imp_last_error());
    if (arch / 10 != 10) fail(IMP_ERROR_UNSUPPORTED, "the kernels are built for sm_100a only; this device is sm_" + std::to_string(arch));
    rt.dtype = dtype;
    rt.device = device_id;
    IMP_CUDA(cudaStreamCreateWithFlags(&rt.stream, cudaStreamNonBlocking));
    status = DeviceBuffer(4, true);
    rt.status = (int32_t*)status.data();
    arena = std::make_unique<Arena>(step_bytes, layer_bytes);
    rt.arena = arena.get();
    rt.sm_count = imp_device_sm_count();
    rt.time_without = env_string("IMP_B200_TIME_WITHOUT", "");
    if (!rt.time_without.empty())
        log_line(LOG_WARN, "IMP_B200_TIME_WITHOUT=%s: these operations are not launched, every result of this context is meaningless",
                 rt.time_without.c_str());
}

DeviceContext::~DeviceContext() {
    if (rt.stream) {
        cudaStreamSynchronize(rt.stream);
        cudaStreamDestroy(rt.stream);
    }
}

void DeviceContext::make_current() const { IMP_CUDA(cudaSetDevice(rt.device)); }

// -------------------------------------------------------------------------------------- engine
Engine::Engine(const HostModel& host, const ImpConfig& cfg) : cfg_(cfg) {
    validate_engine_config(cfg);
    const int dtype = cfg.compute_dtype == IMP_COMPUTE_FP32 ? F32 : BF16;
    const size_t T = (size_t)cfg.max_batch_tokens, d = (size_t)host.plan.hidden_size, V = (size_t)host.plan.vocab_size;
    // A first estimate of the workspace from the token budget; a step that needs more makes it grow once.
    dev_ = std::make_unique<DeviceContext>(cfg.device_id, dtype, T * d * 4 + (size_t)cfg.max_batch_size * (V * 4 + d * 4), T * d * 2 * 12);
    model_ = std::make_unique<DeviceModel>(host, &dev_->rt);
    max_seq_len_ = (int)std::min<int64_t>(cfg.max_seq_len, host.plan.max_positions);
    const int pages = decide_pages(host);
    const int slots = cfg.state_slots > 0 ? cfg.state_slots : cfg.max_batch_size;
    cache_ = std::make_unique<CacheManager>(model_->cache_specs(), cfg.kv_block_size, pages, slots);
    cache_->allocate_storage(dtype);
    stepper_ = std::make_unique<Stepper>(model_.get(), cache_.get(), &dev_->rt, cfg.max_batch_tokens, cfg.max_batch_size, max_seq_len_,
                                         cfg.enable_cuda_graphs != 0, model_->vocab_size(), model_->tilings());
    sched_ = std::make_unique<Scheduler>(cache_.get(), cfg.max_batch_size, cfg.max_batch_tokens, cfg.prefill_chunk_size, max_seq_len_);
    sampler_ = std::make_unique<Sampler>(model_->vocab_size(), cfg.max_batch_size, &dev_->rt);
    for (auto& l : landing_) l = PinnedBuffer(((size_t)cfg.max_batch_size + 1) * 4);
    for (auto& e : events_) IMP_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    eos_ = host.config->eos_token_ids;
    IMP_CUDA(cudaStreamSynchronize(dev_->rt.stream));
}

Engine::~Engine() {
    if (dev_) cudaStreamSynchronize(dev_->rt.stream);
    for (auto e : events_)
        if (e) cudaEventDestroy(e);
    for (auto e : timer_)
        if (e) cudaEventDestroy(e);
}

void Engine::timer_start() {
    for (auto& e : timer_)
        if (!e) IMP_CUDA(cudaEventCreate(&e));
    IMP_CUDA(cudaEventRecord(timer_[0], dev_->rt.stream));
}

float Engine::timer_stop() {
    if (!timer_[0]) fail(IMP_ERROR_INVALID_ARG, "the timer was not started");
    IMP_CUDA(cudaEventRecord(timer_[1], dev_->rt.stream));
    IMP_CUDA(cudaEventSynchronize(timer_[1]));
    float ms = 0.f;
    IMP_CUDA(cudaEventElapsedTime(&ms, timer_[0], timer_[1]));
    return ms;
}

// Pages per cache group: explicit, or from a token count, or from free memory (the reference gives 80% of
// free memory, clamped to 1-2x the configured worst case: src/runtime/engine.cpp:226-243; an explicit block
// count wins, :531-535).
int Engine::decide_pages(const HostModel&) const {
    const int P = cfg_.kv_block_size;
    if (cfg_.kv_cache_max_blocks > 0) return (int)cfg_.kv_cache_max_blocks;
    if (cfg_.kv_cache_tokens > 0) return (int)((cfg_.kv_cache_tokens + (size_t)P - 1) / (size_t)P);
    const int64_t worst = (int64_t)((max_seq_len_ + P - 1) / P) * cfg_.max_batch_size;
    CacheManager probe(model_->cache_specs(), P, 1, 1);
    const size_t per_page = std::max<size_t>(1, probe.storage_bytes((int)elem_size(dev_->rt.dtype)));
    size_t free_b = 0, total_b = 0;
    IMP_CUDA(cudaMemGetInfo(&free_b, &total_b));
    const int64_t by_memory = (int64_t)((double)free_b * cfg_.gpu_memory_fraction / (double)per_page);
    return (int)std::max<int64_t>(1, std::min(worst, by_memory));
}

int64_t Engine::submit(const int32_t* tokens, int n, const ImpGenerateParams& params, ImpRequestStatus* status) {
    if (!tokens || n <= 0) fail(IMP_ERROR_INVALID_ARG, "a request needs at least one prompt token");
    const int64_t V = model_->vocab_size();
    for (int i = 0; i < n; ++i)
        if (tokens[i] < 0 || tokens[i] >= V)
            fail(IMP_ERROR_INVALID_ARG, "token id " + std::to_string(tokens[i]) + " outside the vocabulary of " + std::to_string(V));
    auto req = std::make_unique<Request>();
    req->rid = next_id_++;
    req->prompt.assign(tokens, tokens + n);
    req->max_tokens = params.max_tokens;
    req->params = SamplingParams::from(params);
    req->eos_token_ids = eos_;
    req->ignore_eos = params.ignore_eos != 0;
    Request* r = sched_->add(std::move(req));
    if (status) *status = r->status;
    return r->rid;
}

std::unique_ptr<Engine::InFlight> Engine::launch(StepPlan plan, const int32_t* device_tokens, std::vector<ImpStepOutput> early) {
    auto fl = std::make_unique<InFlight>();
    std::vector<StepEntryView> entries;
    std::vector<int32_t> want_last;
    int total = 0;
    for (const auto& e : plan.entries) total += e.n_tokens;
    scratch_tokens_.assign((size_t)total, 0);
    want_last.reserve(plan.entries.size());
    int t0 = 0;
    for (const auto& e : plan.entries) {
        StepEntryView v{};
        v.rid = e.request->rid;
        v.n_tokens = e.n_tokens;
        if (!device_tokens) {
            e.request->tokens_slice(e.start, e.n_tokens, scratch_tokens_.data() + t0);
            v.tokens = scratch_tokens_.data() + t0;
        }
        want_last.push_back(e.n_tokens - 1);
        v.want = e.samples ? &want_last.back() : nullptr;
        v.n_want = e.samples ? 1 : 0;
        entries.push_back(v);
        if (e.samples) fl->rows.push_back(e.request);
        t0 += e.n_tokens;
    }
    Runtime& rt = dev_->rt;
    Tensor logits = stepper_->step(entries.data(), (int)entries.size(), device_tokens);
    fl->landing = landing_turn_;
    landing_turn_ ^= 1;
    int32_t* land = (int32_t*)landing_[fl->landing].data();
    if (!fl->rows.empty()) {
        // a token launched ahead of the last one's arrival counts as one more output
        const int ahead = device_tokens ? 1 : 0;
        std::vector<int64_t> steps;
        for (Request* r : fl->rows) steps.push_back((int64_t)r->output.size() + ahead);
        fl->tokens_dev = sampler_->sample_device(logits, fl->rows, steps);
        IMP_CUDA(cudaMemcpyAsync(land, fl->tokens_dev, fl->rows.size() * 4, cudaMemcpyDeviceToHost, rt.stream));
    }
    IMP_CUDA(cudaMemcpyAsync(land + cfg_.max_batch_size, rt.status, 4, cudaMemcpyDeviceToHost, rt.stream));
    fl->event = events_[fl->landing];
    IMP_CUDA(cudaEventRecord(fl->event, rt.stream));
    fl->plan = std::move(plan);
    fl->early = std::move(early);
    ++steps_;
    return fl;
}

std::vector<ImpStepOutput> Engine::finish(std::unique_ptr<InFlight> fl) {
    IMP_CUDA(cudaEventSynchronize(fl->event));
    const int32_t* land = (const int32_t*)landing_[fl->landing].data();
    if (land[cfg_.max_batch_size] != 0) stepper_->check_device_status("step");   // throws with the device's message and clears the word
    std::vector<ImpStepOutput> outs = std::move(fl->early);
    std::vector<int32_t> sampled(land, land + fl->rows.size());
    std::vector<bool> live;
    for (Request* r : fl->rows) live.push_back(!r->done());   // a request may have finished while this step was under way
    const std::vector<Request*> finished = sched_->complete_step(fl->plan, sampled);
    for (size_t i = 0; i < fl->rows.size(); ++i) {
        if (!live[i]) continue;
        Request* r = fl->rows[i];
        const bool fin = std::find(finished.begin(), finished.end(), r) != finished.end();
        outs.push_back(ImpStepOutput{r->rid, sampled[i], fin ? 1 : 0, (int32_t)r->status, (int32_t)r->finish_reason});
    }
    return outs;
}

// The step after `fl` if it can be decided before `fl`'s tokens are known: every running request gets a
// token from `fl`, none of them ends with it for a reason known in advance (length, context), none needs its
// token on the host to sample the next one, nothing waits for admission, and the pages are there.
bool Engine::plan_ahead(const InFlight& fl, StepPlan* out) {
    if (!cfg_.lookahead || fl.rows.empty() || !sched_->waiting.empty() || fl.rows.size() != sched_->running.size()) return false;
    if (fl.plan.entries.size() != fl.rows.size() || !fl.plan.preempted.empty() || !fl.plan.failed.empty()) return false;
    StepPlan plan;
    std::vector<StepEntryView> probe;
    for (const auto& e : fl.plan.entries) {
        Request* r = e.request;
        if (r->done() || r->params.needs_history() || r->params.mirostat) return false;
        const int start = e.start + e.n_tokens;
        if ((int)r->output.size() + 1 >= r->max_tokens || start + 1 >= max_seq_len_) return false;
        plan.entries.push_back(ScheduledEntry{r, start, 1, true});
        probe.push_back(StepEntryView{r->rid, nullptr, 1, nullptr, 0});
    }
    if (stepper_->pages_short(probe.data(), (int)probe.size()) > 0) return false;
    *out = std::move(plan);
    return true;
}

std::vector<ImpStepOutput> Engine::step() {
    std::unique_ptr<InFlight> fl = std::move(inflight_);
    if (!fl) {
        StepPlan plan = sched_->schedule();
        std::vector<ImpStepOutput> early;
        for (Request* r : plan.failed) early.push_back(ImpStepOutput{r->rid, -1, 1, (int32_t)r->status, (int32_t)r->finish_reason});
        if (plan.entries.empty()) return early;
        fl = launch(std::move(plan), nullptr, std::move(early));
    }
    StepPlan ahead;
    if (plan_ahead(*fl, &ahead)) inflight_ = launch(std::move(ahead), fl->tokens_dev, {});
    return finish(std::move(fl));
}

std::vector<ImpStepOutput> Engine::drain() {
    std::unique_ptr<InFlight> fl = std::move(inflight_);
    if (!fl) return {};
    return finish(std::move(fl));
}

void Engine::reset() {
    if (inflight_) {
        cudaEventSynchronize(inflight_->event);
        inflight_.reset();
    }
    IMP_CUDA(cudaStreamSynchronize(dev_->rt.stream));
    sched_->reset();
    cache_->release_all();
    single_rid = -1;
    single_read = 0;
}

void Engine::step_tokens(const ImpStepEntry* entries, int n, float* logits_out, size_t capacity) {
    if (!entries || n <= 0) fail(IMP_ERROR_INVALID_ARG, "a step needs at least one entry");
    std::vector<StepEntryView> views;
    size_t want = 0;
    for (int i = 0; i < n; ++i) {
        const ImpStepEntry& e = entries[i];
        if (!e.tokens || (e.n_want > 0 && !e.want)) fail(IMP_ERROR_INVALID_ARG, "an entry lacks its tokens or its wanted rows");
        views.push_back(StepEntryView{e.id, e.tokens, e.n_tokens, e.want, e.n_want});
        want += (size_t)std::max(e.n_want, 0);
    }
    const size_t V = (size_t)model_->vocab_size();
    if (want * V > capacity) fail(IMP_ERROR_INVALID_ARG, "the logits buffer is too small for the wanted rows");
    if (want && !logits_out) fail(IMP_ERROR_INVALID_ARG, "rows are wanted but there is no logits buffer");
    Tensor logits = stepper_->step(views.data(), n);
    if (want) IMP_CUDA(cudaMemcpyAsync(logits_out, logits.data, want * V * 4, cudaMemcpyDeviceToHost, dev_->rt.stream));
    stepper_->check_device_status("step");
}

void Engine::end(int64_t rid) {
    if (!cache_->has(rid)) fail(IMP_ERROR_INVALID_ARG, "request " + std::to_string(rid) + " holds nothing (ended twice?)");
    stepper_->finish(rid);
}

Json Engine::info_json() const {
    Json j = Json::object();
    j["cache"] = cache_->info_json();
    j["model"] = model_->info_json();
    j["scheduler"] = sched_->info_json();
    j["max_seq_len"] = max_seq_len_;
    j["steps"] = steps_;
    j["inflight"] = inflight_ != nullptr;
    j["eos_token_ids"] = Json::array_of(eos_);
    j["launches"] = dev_->rt.launches;
    j["fallback_calls"] = dev_->rt.fallback_calls;
    j["split_norm_calls"] = dev_->rt.split_norm_calls;
    j["h2d_bytes_last_step"] = stepper_->h2d_bytes_last_step;
    j["graph_replays"] = stepper_->graph_replays;
    j["graph_captures"] = stepper_->graph_captures;
    j["eager_steps"] = stepper_->eager_steps;
    j["workspace_bytes"] = dev_->arena->capacity_bytes();
    j["workspace_high_water"] = dev_->arena->high_water_bytes();
    j["sm_count"] = dev_->rt.sm_count;
    j["compute_dtype"] = dtype_name(dev_->rt.dtype);
    return j;
}

}  // namespace imp
