// The engine: model + cache + step function + scheduler + sampler on one GPU, behind one handle.
//
// step() wraps the step function with scheduling and sampling.  With `lookahead` it queues the next
// decode step on the device before it has read the last step's tokens: the sampled ids stay on the
// device and feed the next step's embedding, the host reads them (pinned memory, an event) while that
// step runs, and schedules meanwhile.  The step ahead is launched only when its batch is known in
// advance: every running request got a token, none ends with it by length or context, none needs its
// tokens on the host to sample (penalties, DRY, Mirostat), nothing waits for admission, pages are
// there.  A request that ends on its end-of-sequence token rides along for one step; its result is
// dropped.  Each call still returns exactly one step's tokens.
//
// The reference's engine (src/runtime/engine.cpp:993-2059) runs each prefilling request in a forward
// pass of its own, then one batched decode, and waits for the sampled token inside the sampler
// (src/compute/sampling.cu:210-213).
#pragma once

#include <memory>
#include <vector>

#include "sampler.hpp"
#include "step.hpp"

namespace imp {

// The device side every context (and every bench of single parts) owns: stream, status word, workspace.
struct DeviceContext {
    Runtime rt;
    std::unique_ptr<Arena> arena;
    DeviceBuffer status;
    DeviceContext(int device_id, int dtype, size_t step_bytes, size_t layer_bytes);
    ~DeviceContext();
    void make_current() const;
};

class Engine {
public:
    Engine(const HostModel& host, const ImpConfig& cfg);
    ~Engine();

    int64_t submit(const int32_t* tokens, int n, const ImpGenerateParams& params, ImpRequestStatus* status);
    void cancel(int64_t rid) { sched_->cancel(rid); }
    bool has_work() const { return sched_->has_work() || inflight_ != nullptr; }
    std::vector<ImpStepOutput> step();
    std::vector<ImpStepOutput> drain();
    void reset();
    Request* request(int64_t rid) const { return sched_->find(rid); }
    void forget(int64_t rid) { sched_->forget(rid); }

    // Run given tokens as one batch (no scheduling, no sampling); logits of the wanted rows on the host.
    void step_tokens(const ImpStepEntry* entries, int n, float* logits_out, size_t capacity);
    void end(int64_t rid);

    Json info_json() const;
    const ImpConfig& config() const { return cfg_; }
    int max_seq_len() const { return max_seq_len_; }
    int64_t vocab_size() const { return model_->vocab_size(); }
    void make_current() const { dev_->make_current(); }
    void set_eos(const std::vector<int>& ids) { eos_ = ids; }      // for requests submitted from now on
    void check_invariants() const { cache_->check_invariants(); }
    // Device time between two points of the context's stream (CUDA events): for measurement.
    void timer_start();
    float timer_stop();   // waits for the stream; milliseconds since timer_start
    // the reference's token-level pair (one request at a time)
    int64_t single_rid = -1;
    size_t single_read = 0;

private:
    struct InFlight {
        StepPlan plan;
        std::vector<Request*> rows;          // the requests that get a token, in the order of the sampled tokens
        const int32_t* tokens_dev = nullptr; // int32 [rows] on the device
        int landing = 0;                     // which pinned landing place holds (tokens, status)
        cudaEvent_t event = nullptr;
        std::vector<ImpStepOutput> early;    // outputs known at launch (requests the scheduler gave up on)
    };
    int decide_pages(const HostModel& host) const;
    std::unique_ptr<InFlight> launch(StepPlan plan, const int32_t* device_tokens, std::vector<ImpStepOutput> early);
    std::vector<ImpStepOutput> finish(std::unique_ptr<InFlight> fl);
    bool plan_ahead(const InFlight& fl, StepPlan* out);

    ImpConfig cfg_;
    int max_seq_len_ = 0;
    std::unique_ptr<DeviceContext> dev_;
    std::unique_ptr<DeviceModel> model_;
    std::unique_ptr<CacheManager> cache_;
    std::unique_ptr<Stepper> stepper_;
    std::unique_ptr<Scheduler> sched_;
    std::unique_ptr<Sampler> sampler_;
    std::unique_ptr<InFlight> inflight_;
    PinnedBuffer landing_[2];     // int32 [max_batch_size + 1]: tokens, then the status word
    cudaEvent_t events_[2] = {nullptr, nullptr};
    int landing_turn_ = 0;
    int64_t next_id_ = 0;
    std::vector<int> eos_;
    std::vector<int32_t> scratch_tokens_;
    int64_t steps_ = 0;
    cudaEvent_t timer_[2] = {nullptr, nullptr};
};

}  // namespace imp
