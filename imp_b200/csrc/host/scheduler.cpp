#include "scheduler.hpp"

#include <algorithm>
#include <random>

namespace imp {

// ------------------------------------------------------------------------------------- params
SamplingParams SamplingParams::from(const ImpGenerateParams& p) {
    SamplingParams s;
    s.temperature = p.temperature;
    s.top_p = p.top_p;
    s.top_k = p.top_k;
    s.min_p = p.min_p;
    s.repetition_penalty = p.repetition_penalty;
    s.frequency_penalty = p.frequency_penalty;
    s.presence_penalty = p.presence_penalty;
    s.repeat_last_n = p.repeat_last_n;
    s.typical_p = p.typical_p;
    s.dry_multiplier = p.dry_multiplier;
    s.dry_base = p.dry_base;
    s.dry_allowed_length = p.dry_allowed_length;
    s.dry_penalty_last_n = p.dry_penalty_last_n;
    s.mirostat = p.mirostat;
    s.mirostat_tau = p.mirostat_tau;
    s.mirostat_eta = p.mirostat_eta;
    s.seed = p.seed;
    return s;
}

void SamplingParams::validate() const {
    auto arg = [](const char* m) { fail(IMP_ERROR_INVALID_ARG, m); };
    if (top_k < 0) arg("top_k must be >= 0");
    if (min_p < 0 || min_p > 1) arg("min_p must be in [0, 1]");
    if (repetition_penalty <= 0) arg("repetition_penalty must be positive");
    if (repeat_last_n < 0) arg("repeat_last_n must be >= 0");
    if (mirostat != 0 && mirostat != 2) arg("mirostat must be 0 (off) or 2 (Mirostat v2)");
    if (dry_multiplier < 0 || dry_base <= 0 || dry_allowed_length < 0 || dry_penalty_last_n < 0)
        arg("DRY parameters must not be negative (base positive)");
}

uint64_t resolve_seed(int64_t seed) {
    if (seed >= 0) return (uint64_t)seed;
    std::random_device rd;
    return (((uint64_t)rd() << 32) | rd()) >> 1;
}

float uniform_for(uint64_t seed, int64_t step) {
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + (uint64_t)(step + 1) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) / 16777216.0f;
}

// ------------------------------------------------------------------------------------ request
void Request::tokens_slice(int start, int n, int32_t* out) const {
    for (int i = 0; i < n; ++i) out[i] = token_at(start + i);
}

std::vector<int32_t> Request::all_tokens() const {
    std::vector<int32_t> t(prompt);
    t.insert(t.end(), output.begin(), output.end());
    return t;
}

int StepPlan::n_tokens() const {
    int n = 0;
    for (const auto& e : entries) n += e.n_tokens;
    return n;
}

// ---------------------------------------------------------------------------------- scheduler
Scheduler::Scheduler(CacheManager* cache, int mbs, int mbt, int chunk, int msl)
    : max_batch_size(mbs), max_batch_tokens(mbt), prefill_chunk_size(chunk), max_seq_len(msl), cache_(cache) {}

Request* Scheduler::find(int64_t rid) const {
    auto it = by_id_.find(rid);
    return it == by_id_.end() ? nullptr : it->second.get();
}

bool Scheduler::is_running(const Request* r) const { return std::find(running.begin(), running.end(), r) != running.end(); }

Request* Scheduler::add(std::unique_ptr<Request> req) {
    Request* old = find(req->rid);
    if (old && !old->done()) fail(IMP_ERROR_INVALID_ARG, "request id " + std::to_string(req->rid) + " is already in use");
    if (req->prompt.empty()) fail(IMP_ERROR_INVALID_ARG, "a request needs at least one prompt token");
    if (req->max_tokens <= 0) fail(IMP_ERROR_INVALID_ARG, "max_tokens must be positive");
    if ((int)req->prompt.size() >= max_seq_len)
        fail(IMP_ERROR_INVALID_ARG, "prompt of " + std::to_string(req->prompt.size()) + " tokens leaves no room under max_seq_len " +
                                        std::to_string(max_seq_len));
    req->params.validate();
    req->seed = resolve_seed(req->params.seed);
    Request* r = req.get();
    by_id_[r->rid] = std::move(req);
    const int most = std::min((int)r->prompt.size() + r->max_tokens, max_seq_len);
    if (pages_for_whole(most) > cache_->num_pages()) {
        r->status = IMP_REQUEST_OUT_OF_MEMORY;
        return r;
    }
    r->status = IMP_REQUEST_WAITING;
    waiting.push_back(r);
    return r;
}

int Scheduler::pages_for_whole(int n_tokens) const {
    const int P = cache_->page_size();
    int need = 0;
    for (const auto& g : cache_->paged()) {
        if (g.spec.window > 0) {
            // live span is at most window + one portion; count the window plus one page of slack
            const int span = std::min(n_tokens, g.spec.window + std::max(prefill_chunk_size, 1) + P);
            need = std::max(need, (span + P - 1) / P);
        } else {
            need = std::max(need, (n_tokens + P - 1) / P);
        }
    }
    return need;
}

void Scheduler::cancel(int64_t rid) {
    Request* r = find(rid);
    if (!r || r->done()) return;
    auto it = std::find(running.begin(), running.end(), r);
    if (it != running.end()) {
        running.erase(it);
        release(r);
    } else {
        auto w = std::find(waiting.begin(), waiting.end(), r);
        if (w != waiting.end()) waiting.erase(w);
    }
    r->status = IMP_REQUEST_CANCELLED;
}

void Scheduler::forget(int64_t rid) {
    Request* r = find(rid);
    if (r && r->done()) by_id_.erase(rid);
}

void Scheduler::reset() {
    for (Request* r : running) release(r);
    running.clear();
    waiting.clear();
    by_id_.clear();
}

void Scheduler::release(Request* r) {
    if (cache_->has(r->rid)) cache_->release(r->rid);
    r->n_computed = 0;
}

int Scheduler::pages_needed(const Request* r, int new_len) const {
    return cache_->has(r->rid) ? cache_->pages_needed(r->rid, new_len) : cache_->pages_for_new(new_len);
}

void Scheduler::preempt(Request* victim, StepPlan& plan) {
    running.erase(std::find(running.begin(), running.end(), victim));
    plan.entries.erase(std::remove_if(plan.entries.begin(), plan.entries.end(),
                                      [&](const ScheduledEntry& e) { return e.request == victim; }),
                       plan.entries.end());
    release(victim);
    plan.pages = 0;
    for (const auto& e : plan.entries) plan.pages += pages_needed(e.request, e.start + e.n_tokens);
    victim->status = IMP_REQUEST_WAITING;
    victim->n_preempted += 1;
    ++preemptions;
    waiting.push_front(victim);
    plan.preempted.push_back(victim);
}

int Scheduler::largest_fit(const Request* r, int n, int free) const {
    const int P = cache_->page_size();
    const int room_in_last_page = cache_->has(r->rid) ? ((P - r->n_computed % P) % P) : 0;
    int fit = std::min(n, std::max(free, 0) * P + room_in_last_page);
    while (fit >= 1 && pages_needed(r, r->n_computed + fit) > free) --fit;   // windowed groups can need a page more
    return std::max(fit, 0);
}

// A portion that does not end its prompt is cut so that the step's rows so far plus the portion are a multiple of 256:
// the products of 129 rows and more work in tiles of 256 rows, and a last tile that holds the 64 rows of the decoding
// sequences beside a 512-token portion costs as much as a full one (576 rows: three tiles; 512: two).  Only portions
// of 256 tokens and more, never below half of what was asked.  IMP_B200_SCHED_ALIGN=0 keeps portions as asked.
static int aligned_portion(int n, int remaining, int rows_so_far) {
    static const bool on = env_flag("IMP_B200_SCHED_ALIGN", true);
    constexpr int TILE_ROWS = 256;
    if (!on || n >= remaining || n < TILE_ROWS) return n;
    const int whole = (rows_so_far + n) / TILE_ROWS * TILE_ROWS - rows_so_far;
    return (whole >= n / 2 && whole > 0) ? whole : n;
}

int Scheduler::serve_running(Request* r, StepPlan& plan, int budget, int chunk) {
    const int remaining = r->n_total() - r->n_computed;
    const bool decoding = remaining == 1;
    int n = decoding ? 1 : std::min({remaining, chunk, budget});
    if (!decoding) n = aligned_portion(n, remaining, max_batch_tokens - budget);
    while (true) {
        const int free = free_after(plan);
        if (pages_needed(r, r->n_computed + n) <= free) break;
        if (!decoding) {
            const int fit = largest_fit(r, n, free);
            if (fit >= 1) {
                n = fit;
                break;
            }
            if (r != running.front()) return 0;   // a younger prompt waits for pages; the oldest request always goes on
        }
        Request* victim = running.back();
        if (victim == r) {
            if (running.size() == 1) {
                // alone with the whole pool and still short of pages: it cannot go on
                running.clear();
                release(r);
                r->status = IMP_REQUEST_OUT_OF_MEMORY;
                plan.failed.push_back(r);
            } else {
                preempt(r, plan);
            }
            return 0;
        }
        preempt(victim, plan);
    }
    plan.pages += pages_needed(r, r->n_computed + n);
    plan.entries.push_back(ScheduledEntry{r, r->n_computed, n, r->n_computed + n == r->n_total()});
    return n;
}

StepPlan Scheduler::schedule() {
    StepPlan plan;
    int budget = max_batch_tokens;
    const int chunk = prefill_chunk_size > 0 ? prefill_chunk_size : max_batch_tokens;
    for (int pass = 0; pass < 2; ++pass) {
        const bool decoding = pass == 0;
        const std::vector<Request*> snapshot(running);
        for (Request* r : snapshot) {
            if (!is_running(r) || budget <= 0) continue;
            if (((r->n_total() - r->n_computed) == 1) != decoding) continue;
            budget -= serve_running(r, plan, budget, chunk);
        }
    }
    const int P = cache_->page_size();
    while (!waiting.empty() && budget > 0 && (int)running.size() < max_batch_size) {
        Request* r = waiting.front();
        if (std::find(plan.preempted.begin(), plan.preempted.end(), r) != plan.preempted.end())
            break;   // just preempted for lack of pages: not again in the same step
        int new_in_plan = 0;
        for (const auto& e : plan.entries)
            if (!cache_->has(e.request->rid)) ++new_in_plan;
        if (cache_->slots().n_free() - new_in_plan <= 0) break;
        int n = std::min({r->n_total(), chunk, budget});
        n = aligned_portion(n, r->n_total(), max_batch_tokens - budget);
        const int free = free_after(plan);
        // Keep one page in hand per running request so that decoding can go on.
        const int usable = running.empty() ? free : free - (int)running.size();
        if (pages_needed(r, n) > usable) {
            n = std::min(n, std::max(usable, 0) * P);
            if (n < 1) break;
        }
        waiting.pop_front();
        r->status = IMP_REQUEST_RUNNING;
        r->n_computed = 0;
        running.push_back(r);
        plan.pages += pages_needed(r, n);
        plan.entries.push_back(ScheduledEntry{r, 0, n, n == r->n_total()});
        budget -= n;
    }
    return plan;
}

std::vector<Request*> Scheduler::complete_step(const StepPlan& plan, const std::vector<int32_t>& sampled) {
    std::vector<Request*> finished;
    size_t si = 0;
    for (const auto& e : plan.entries) {
        Request* r = e.request;
        const bool has_token = e.samples;
        const int32_t tok = has_token && si < sampled.size() ? sampled[si] : -1;
        if (has_token) ++si;
        if (r->done()) continue;   // finished or cancelled while this step was already under way
        r->n_computed = e.start + e.n_tokens;
        if (!has_token) continue;
        r->output.push_back(tok);
        ImpFinishReason reason = IMP_FINISH_NONE;
        if (!r->ignore_eos && std::find(r->eos_token_ids.begin(), r->eos_token_ids.end(), (int)tok) != r->eos_token_ids.end())
            reason = IMP_FINISH_EOS;
        else if ((int)r->output.size() >= r->max_tokens)
            reason = IMP_FINISH_LENGTH;
        else if (r->n_total() >= max_seq_len)
            reason = IMP_FINISH_CONTEXT;
        if (reason != IMP_FINISH_NONE) {
            r->status = IMP_REQUEST_FINISHED;
            r->finish_reason = reason;
            running.erase(std::find(running.begin(), running.end(), r));
            release(r);
            finished.push_back(r);
        }
    }
    return finished;
}

Json Scheduler::info_json() const {
    Json j = Json::object();
    Json w = Json::array(), r = Json::array();
    for (const Request* q : waiting) w.push(Json(q->rid));
    for (const Request* q : running) r.push(Json(q->rid));
    j["waiting"] = w;
    j["running"] = r;
    j["preemptions"] = preemptions;
    Json reqs = Json::object();
    for (const auto& kv : by_id_) {
        const Request& q = *kv.second;
        Json o = Json::object();
        o["status"] = (int)q.status;
        o["finish_reason"] = (int)q.finish_reason;
        o["n_prompt"] = (int)q.prompt.size();
        o["n_computed"] = q.n_computed;
        o["n_preempted"] = q.n_preempted;
        o["output"] = Json::array_of(std::vector<int>(q.output.begin(), q.output.end()));
        reqs[std::to_string(kv.first)] = o;
    }
    j["requests"] = reqs;
    return j;
}

}  // namespace imp
