// The step function: one batch of (request, its next tokens) through the model.
//
// A batch holds, for each request in it, the tokens that come next for that request: a portion of
// its prompt of any length, or a single decoded token.  Everything is one flat list of tokens with,
// per token, its position and the index of its sequence in the batch; per sequence, its row of each
// cache group's block table, its state slot and its length after the step.  The step reserves pages,
// uploads these arrays with one copy from pinned memory, runs the model once and returns the logits
// of the wanted rows.
//
// The reference builds two kinds of batches, never mixed: one prompt portion with a flat block
// table, or B decode tokens with token i belonging to sequence i (src/runtime/batch.cpp:86-135,
// src/runtime/engine.cpp:1203-1258, 1655-1713); its `seq_offsets` array is uploaded but never read by
// a kernel (src/graph/executor.h:122).
#pragma once

#include <map>
#include <memory>
#include <vector>

#include "model.hpp"

namespace imp {

// The next tokens of one request, and which of them should yield logits.
struct StepEntryView {
    int64_t rid;
    const int32_t* tokens;   // may be null: placeholders (the ids come from the device)
    int n_tokens;
    const int32_t* want;     // indices into `tokens`
    int n_want;
};

// Persistent device arrays of a batch at fixed addresses, with pinned staging.  Layout in int32 words,
// by capacity (so a view's address does not depend on the batch): tokens | positions | seq_of_token |
// logit_rows | per declared tiling (first token, rows) | q_start | kv_len | slots | one block table
// [max_seqs, max_pages] per paged cache group.
class BatchBuffers {
public:
    BatchBuffers(int max_tokens, int max_seqs, int max_pages, int n_groups, int n_tilings);
    ~BatchBuffers();
    int max_tokens, max_seqs, max_pages, n_groups, n_tilings;
    size_t off_tok, off_pos, off_seq, off_rows, off_q_start, off_kv_len, off_slots, small_words, words;
    std::vector<size_t> off_tile0, off_tilen, off_bt;
    int32_t* dev() const { return (int32_t*)dev_.data(); }
    // The next staging buffer, once the copy that last used it has finished.
    int32_t* staging(int* which);
    // Small arrays in one copy, then the used rows of each block table.
    void upload(int which, int n_seqs, cudaStream_t stream);

private:
    DeviceBuffer dev_;
    PinnedBuffer host_[2];
    cudaEvent_t events_[2] = {nullptr, nullptr};
    bool used_[2] = {false, false};
    int turn_ = 0;
};

// Owns the batch buffers and runs steps of a model against a cache manager.  `model` may be null:
// then only the batch arrays are built (single parts are driven that way).
class Stepper {
public:
    Stepper(DeviceModel* model, CacheManager* cache, Runtime* rt, int max_tokens, int max_seqs, int max_seq_len,
            bool use_cuda_graphs, int64_t vocab_size, const std::vector<TilingSpec>& tilings);
    ~Stepper();

    // How many pages the scarcest group lacks for this batch (0 = it fits).
    int pages_short(const StepEntryView* entries, int n) const;
    // Check the batch on the host, reserve cache, fill and upload the batch arrays.
    Step& prepare(const StepEntryView* entries, int n);
    // Record the new lengths; pages behind a window return to their pool.
    void commit(const Step& st);
    // Run one batch.  Returns float32 logits [wanted rows, vocab] on the device, in the order of the entries
    // and of each entry's `want`.  `device_tokens` (int32, one per token of the batch, on the device) replaces
    // the entries' token ids: the ids of a step whose tokens were sampled on the device and have not come back
    // to the host yet.  The logits live until the next step.
    Tensor step(const StepEntryView* entries, int n, const int32_t* device_tokens = nullptr);
    void finish(int64_t rid) { cache_->release(rid); }
    // Read the status word (waits for the stream) and throw if a kernel reported a bad index or a wait ran out.
    void check_device_status(const std::string& what);
    Step& current() { return step_; }
    int64_t graph_replays = 0, graph_captures = 0, eager_steps = 0;
    int64_t h2d_bytes_last_step = 0;   // batch arrays copied from pinned memory by the last prepare()

private:
    Tensor forward_decode_graph(Step& st);
    void drop_graphs();
    DeviceModel* model_;
    CacheManager* cache_;
    Runtime* rt_;
    int max_tokens_, max_seqs_, max_seq_len_, max_pages_;
    bool use_graphs_;
    int64_t vocab_;
    std::vector<TilingSpec> tilings_;
    BatchBuffers buf_;
    Step step_;
    struct Graph {
        cudaGraphExec_t exec = nullptr;
        Tensor logits{};
        int64_t launches = 0;
        Arena::Mark mark;    // the workspace's cursors when the capture ended
    };
    std::map<int, Graph> graphs_;
    std::map<int, int> graph_uses_;
    uint64_t arena_generation_ = 0;
};

}  // namespace imp
