// Continuous batching: admission, prompt portions under a token budget, decode, finish.
//
// Compared with the reference (src/runtime/scheduler.cpp:16-112, src/runtime/engine.cpp:1074-1515,
// 1528-2050):
//   * admission is first come first served (the reference sorts the queue by prompt length,
//     scheduler.cpp:32-38), so the same arrivals always give the same batches;
//   * one step holds decode tokens and prompt portions together, under `max_batch_tokens` (the
//     reference runs every prefilling request in a forward pass of its own and has no per-step token
//     budget, engine.cpp:1101-1120);
//   * pages are reserved portion by portion, not for the whole prompt up front (scheduler.cpp:48-80);
//   * when pages run out, nothing is evicted silently (the reference frees the least recently used
//     sequence's pages without telling its request, which is then cancelled at its next step:
//     engine.cpp:1541-1553, kv_cache_manager.cpp:158-170).  Instead the scheduler *preempts* the
//     request that was admitted last: its pages and slot are returned, and it goes back to the head of
//     the waiting queue to be recomputed later from its prompt plus the tokens it has generated so
//     far.  A request that could not fit even with the whole pool to itself is refused when it is added
//     (status OUT_OF_MEMORY).
// The scheduler only decides; it talks to the cache manager for page counts and to nothing else, so it
// runs without a GPU.
#pragma once

#include <deque>
#include <map>
#include <memory>
#include <vector>

#include "cache.hpp"

namespace imp {

// Per-request sampling settings: the fields of ImpGenerateParams that steer the sampler.
struct SamplingParams {
    float temperature = 0.7f, top_p = 0.9f;
    int top_k = 40;
    float min_p = 0.f, repetition_penalty = 1.f, frequency_penalty = 0.f, presence_penalty = 0.f;
    int repeat_last_n = 0;
    float typical_p = 1.f, dry_multiplier = 0.f, dry_base = 1.75f;
    int dry_allowed_length = 2, dry_penalty_last_n = 0, mirostat = 0;
    float mirostat_tau = 5.f, mirostat_eta = 0.1f;
    int64_t seed = -1;

    static SamplingParams from(const ImpGenerateParams& p);
    bool is_greedy() const { return mirostat != 2 && (temperature <= 0.f || top_k == 1); }
    bool has_penalties() const { return repetition_penalty != 1.f || frequency_penalty != 0.f || presence_penalty != 0.f; }
    bool has_dry() const { return dry_multiplier > 0.f; }
    bool has_typical() const { return mirostat != 2 && typical_p > 0.f && typical_p < 1.f; }
    bool needs_history() const { return has_penalties() || has_dry(); }
    void validate() const;   // throws Error(IMP_ERROR_INVALID_ARG)
};

// One generation request (the reference's Request: src/runtime/request.h:32-74).
struct Request {
    int64_t rid = 0;
    std::vector<int32_t> prompt, output;
    int max_tokens = 256;
    SamplingParams params;
    std::vector<int> eos_token_ids;
    bool ignore_eos = false;
    ImpRequestStatus status = IMP_REQUEST_WAITING;
    ImpFinishReason finish_reason = IMP_FINISH_NONE;
    int n_computed = 0;        // tokens of prompt + output whose keys/state are in the cache
    uint64_t seed = 0;         // resolved sampling seed
    int n_preempted = 0;
    bool has_mu = false;       // Mirostat's mu carried from token to token (starts at 2 * tau)
    float mirostat_mu = 0.f;

    int n_total() const { return (int)(prompt.size() + output.size()); }
    bool done() const { return status == IMP_REQUEST_FINISHED || status == IMP_REQUEST_CANCELLED || status == IMP_REQUEST_OUT_OF_MEMORY; }
    int32_t token_at(int i) const { return i < (int)prompt.size() ? prompt[(size_t)i] : output[(size_t)i - prompt.size()]; }
    void tokens_slice(int start, int n, int32_t* out) const;   // tokens [start, start + n) of prompt then output
    std::vector<int32_t> all_tokens() const;
};

struct ScheduledEntry {
    Request* request;
    int start;        // index into prompt + output of the first token of this portion
    int n_tokens;
    bool samples;     // the portion ends at the last known token: its last row is sampled
};

struct StepPlan {
    std::vector<ScheduledEntry> entries;
    std::vector<Request*> preempted, failed;
    int pages = 0;    // pages the entries so far will take from the pool
    int n_tokens() const;
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, int max_batch_size, int max_batch_tokens, int prefill_chunk_size, int max_seq_len);

    // Takes the request; returns it (status WAITING, or OUT_OF_MEMORY when it can never fit).
    Request* add(std::unique_ptr<Request> req);
    void cancel(int64_t rid);
    bool has_work() const { return !waiting.empty() || !running.empty(); }
    Request* find(int64_t rid) const;
    void forget(int64_t rid);        // drop a finished request's record
    void reset();                    // drop every request, release their cache

    // Decide the next step's batch: decode tokens first, then portions of running prompts, then new
    // requests.  Touches the cache only to release what it preempts.
    StepPlan schedule();
    // Record a finished step: advance lengths, append sampled tokens (one per sampling entry, in entry
    // order), finish requests.  Returns the requests that finished (their cache has been released).
    std::vector<Request*> complete_step(const StepPlan& plan, const std::vector<int32_t>& sampled);

    std::deque<Request*> waiting;
    std::vector<Request*> running;   // in admission order
    int max_batch_size, max_batch_tokens, prefill_chunk_size, max_seq_len;
    int64_t preemptions = 0;         // requests sent back to the queue for lack of pages, in all
    Json info_json() const;

private:
    int pages_for_whole(int n_tokens) const;
    void release(Request* r);
    void preempt(Request* victim, StepPlan& plan);
    int pages_needed(const Request* r, int new_len) const;
    int free_after(const StepPlan& plan) const { return cache_->free_pages() - plan.pages; }
    int largest_fit(const Request* r, int n, int free) const;
    int serve_running(Request* r, StepPlan& plan, int budget, int chunk);
    bool is_running(const Request* r) const;
    CacheManager* cache_;
    std::map<int64_t, std::unique_ptr<Request>> by_id_;
};

// A concrete 63-bit seed: `seed` itself, or fresh randomness for a negative one.
uint64_t resolve_seed(int64_t seed);
// The uniform number in [0, 1) of draw `step` of a request seeded with `seed` (splitmix64).  It is a
// function of (seed, step) alone, so a request's tokens do not depend on the batch it was sampled in;
// the reference re-seeds its generator with the same seed at every call
// (src/compute/sampling.cu:541-543) and so repeats one draw.
float uniform_for(uint64_t seed, int64_t step);

}  // namespace imp
