// The two debugging switches of the forward pass, in the reference's manner.
//   IMP_B200_PROFILE=1        CUDA-event timers between named stages (embedding, each layer's mixer
//                             and feed-forward, final norm, head), averaged and printed every 32 steps;
//                             CUDA graphs are off while it is set
//                             (src/graph/executor_forward.cu:2729-2772, 3093-3139).
//   IMP_B200_DEBUG_FORWARD=1  per-stage min / max / mean / L2 / count of non-finite values and the ten
//                             largest logits, with a stream synchronisation at every stage
//                             (src/graph/executor_forward.cu:168-246).
#pragma once

#include <string>
#include <vector>

#include "parts.hpp"

namespace imp {

struct Diagnostics {
    Diagnostics();
    ~Diagnostics();
    const bool profile, debug;
    void begin(Step& st);
    void stage(Step& st, const std::string& name, const Tensor& t);
    void end(Step& st, const Tensor& logits);
    Json profile_json() const;
    void print_profile() const;
    Json last_stats = Json::array(), last_top = Json::array();
    float last_step_ms = 0.f;

private:
    void stamp(Step& st, const std::string& name);
    std::vector<cudaEvent_t> events_;
    std::vector<std::string> names_, sum_names_;
    std::vector<double> sums_;
    int n_stamps_ = 0, steps_ = 0;
    double total_ms_ = 0;
    DeviceBuffer stats_;
};

}  // namespace imp
