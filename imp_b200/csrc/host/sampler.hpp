// The batched sampler over 32-bit logits.
//
// Parameter names and defaults follow the reference's ImpGenerateParams (include/imp/imp.h:61-85;
// defaults src/api/imp_api.cpp:76-102, src/runtime/request.h:40-57).  Order of application as in the
// reference (src/graph/executor.cu:43-115): penalties, DRY, then either Mirostat v2 (which takes the
// temperature and ignores the other filters) or min-p, typical-p and greedy if temperature <= 0 or
// top_k == 1, else top-k/top-p at the given temperature.  The uniform number of a draw is a function
// of (seed, step index of the request) alone.
#pragma once

#include <map>
#include <vector>

#include "scheduler.hpp"

namespace imp {

// The DRY penalty per token id, from the request's tokens so far.  For every position `pos` in the
// window, the length of the match between the tokens before `pos` and the end of the sequence says how
// long a repetition would become if tokens[pos] came next; longer than `allowed_length` costs
// multiplier * base ** (length - allowed_length), the longest match per token counting
// (src/compute/sampling.cu:826-880).
std::map<int32_t, float> dry_penalties(const std::vector<int32_t>& tokens, float multiplier, float base, int allowed_length,
                                       int last_n);

class Sampler {
public:
    Sampler(int64_t vocab_size, int max_rows, Runtime* rt);
    // logits [R, V] float32 on the device (modified in place by penalties and filters); one token per row,
    // left on the device (int32 [R], valid until the call after next).  rows[r] is the request of row r,
    // steps[r] the index of this draw in its request.  Without Mirostat rows nothing here waits for the
    // device, so the caller can queue more work before it reads the tokens.
    const int32_t* sample_device(Tensor logits, const std::vector<Request*>& rows, const std::vector<int64_t>& steps);

private:
    template <typename T> T* upload(const std::vector<T>& host);
    void penalties(Tensor logits, const std::vector<Request*>& rows);
    void dry(Tensor logits, const std::vector<Request*>& rows);
    int64_t V_;
    int max_rows_;
    Runtime* rt_;
    DeviceBuffer out_[2], counts_, argmax_scratch_;
    int turn_ = 0;
};

}  // namespace imp
