#include "step.hpp"

#include <algorithm>
#include <cstring>
#include <set>

#include "diagnostics.hpp"
#include "kernels.h"

namespace imp {

// ------------------------------------------------------------------------------ batch buffers
BatchBuffers::BatchBuffers(int mt, int ms, int mp, int ng, int nt)
    : max_tokens(mt), max_seqs(ms), max_pages(mp), n_groups(ng), n_tilings(nt) {
    size_t o = 0;
    auto take = [&](size_t n) {
        const size_t at = o;
        o += n;
        return at;
    };
    off_tok = take((size_t)mt);
    off_pos = take((size_t)mt);
    off_seq = take((size_t)mt);
    off_rows = take((size_t)mt);
    for (int i = 0; i < nt; ++i) {
        off_tile0.push_back(take((size_t)mt));
        off_tilen.push_back(take((size_t)mt));
    }
    off_q_start = take((size_t)ms + 1);
    off_kv_len = take((size_t)ms);
    off_slots = take((size_t)ms);
    small_words = o;
    for (int g = 0; g < ng; ++g) off_bt.push_back(take((size_t)ms * (size_t)mp));
    words = o;
    dev_ = DeviceBuffer(words * 4, true);
    for (auto& h : host_) h = PinnedBuffer(words * 4);
    for (auto& e : events_) IMP_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
}

BatchBuffers::~BatchBuffers() {
    for (auto e : events_)
        if (e) cudaEventDestroy(e);
}

int32_t* BatchBuffers::staging(int* which) {
    const int i = turn_;
    turn_ ^= 1;
    if (used_[i]) IMP_CUDA(cudaEventSynchronize(events_[i]));
    *which = i;
    return (int32_t*)host_[i].data();
}

void BatchBuffers::upload(int i, int n_seqs, cudaStream_t stream) {
    const int32_t* h = (const int32_t*)host_[i].data();
    IMP_CUDA(cudaMemcpyAsync(dev(), h, small_words * 4, cudaMemcpyHostToDevice, stream));
    for (size_t off : off_bt)
        IMP_CUDA(cudaMemcpyAsync(dev() + off, h + off, (size_t)n_seqs * (size_t)max_pages * 4, cudaMemcpyHostToDevice, stream));
    IMP_CUDA(cudaEventRecord(events_[i], stream));
    used_[i] = true;
}

// ------------------------------------------------------------------------------------ stepper
Stepper::Stepper(DeviceModel* model, CacheManager* cache, Runtime* rt, int max_tokens, int max_seqs, int max_seq_len,
                 bool use_cuda_graphs, int64_t vocab_size, const std::vector<TilingSpec>& tilings)
    : model_(model), cache_(cache), rt_(rt), max_tokens_(max_tokens), max_seqs_(max_seqs), max_seq_len_(max_seq_len),
      max_pages_((max_seq_len + cache->page_size() - 1) / cache->page_size()), use_graphs_(use_cuda_graphs), vocab_(vocab_size),
      tilings_(tilings), buf_(max_tokens, max_seqs, max_pages_, (int)cache->paged().size(), (int)tilings.size()) {
    if (model_) {
        model_->attach_cache(cache);
        if (!model_->graph_safe() || model_->diagnostics()) use_graphs_ = false;
    }
    step_.rt = rt;
}

Stepper::~Stepper() { drop_graphs(); }

void Stepper::drop_graphs() {
    for (auto& kv : graphs_)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    graphs_.clear();
    graph_uses_.clear();
}

int Stepper::pages_short(const StepEntryView* entries, int n) const {
    int short_by = 0;
    for (const auto& g : cache_->paged()) {
        int need = 0;
        for (int i = 0; i < n; ++i) {
            const auto& e = entries[i];
            if (cache_->has(e.rid)) {
                const int cur = cache_->length(e.rid);
                need += g.pages_needed_n(g.n_entries[(size_t)cache_->slot_of(e.rid)], cur, cur + e.n_tokens);
            } else {
                need += g.pages_needed_n(0, 0, e.n_tokens);
            }
        }
        short_by = std::max(short_by, need - g.pool.n_free());
    }
    return short_by;
}

Step& Stepper::prepare(const StepEntryView* entries, int B) {
    auto arg = [](const std::string& m) { fail(IMP_ERROR_INVALID_ARG, m); };
    if (B <= 0) arg("a step needs at least one entry");
    if (B > max_seqs_) arg(std::to_string(B) + " requests in one step; the engine was made for " + std::to_string(max_seqs_));
    {
        std::set<int64_t> ids;
        for (int i = 0; i < B; ++i)
            if (!ids.insert(entries[i].rid).second) arg("a request appears twice in one step");
    }
    int T = 0, R = 0;
    for (int i = 0; i < B; ++i) {
        if (entries[i].n_tokens <= 0) arg("an entry needs at least one token");
        T += entries[i].n_tokens;
        R += entries[i].n_want;
    }
    if (T > max_tokens_) arg(std::to_string(T) + " tokens in one step; the engine was made for " + std::to_string(max_tokens_));
    Step& st = step_;
    st.q_lens.assign((size_t)B, 0);
    st.starts.assign((size_t)B, 0);
    st.slots.assign((size_t)B, 0);
    st.rids.assign((size_t)B, 0);
    int64_t total_len = 0;
    for (int i = 0; i < B; ++i) {
        const auto& e = entries[i];
        st.rids[(size_t)i] = e.rid;
        st.q_lens[(size_t)i] = e.n_tokens;
        st.starts[(size_t)i] = cache_->has(e.rid) ? cache_->length(e.rid) : 0;
        total_len += st.starts[(size_t)i] + e.n_tokens;
        if (e.tokens)
            for (int t = 0; t < e.n_tokens; ++t)
                if (e.tokens[t] < 0 || e.tokens[t] >= vocab_)
                    arg("token id " + std::to_string(e.tokens[t]) + " outside the vocabulary of " + std::to_string(vocab_));
        if (st.starts[(size_t)i] + e.n_tokens > max_seq_len_)
            arg("request " + std::to_string(e.rid) + ": " + std::to_string(st.starts[(size_t)i] + e.n_tokens) +
                " tokens exceed the maximum sequence length " + std::to_string(max_seq_len_));
        for (int w = 0; w < e.n_want; ++w)
            if (e.want[w] < 0 || e.want[w] >= e.n_tokens)
                arg("request " + std::to_string(e.rid) + ": wanted row " + std::to_string(e.want[w]) + " outside its " +
                    std::to_string(e.n_tokens) + " tokens");
    }
    const int lacking = pages_short(entries, B);
    if (lacking > 0) throw OutOfPages("the batch needs " + std::to_string(lacking) + " more pages than are free");
    int new_slots = 0;
    for (int i = 0; i < B; ++i) new_slots += cache_->has(entries[i].rid) ? 0 : 1;
    if (new_slots > cache_->slots().n_free())
        throw OutOfPages(std::to_string(new_slots) + " new requests but only " + std::to_string(cache_->slots().n_free()) + " free state slots");

    {   // the mean length, rounded to the nearest power of two (in the logarithm)
        const double mean = (double)total_len / B;
        int c = 1;
        while ((double)c * 1.41421356 < mean && c < (1 << 30)) c <<= 1;
        st.context = c;
    }
    for (int i = 0; i < B; ++i) {
        const int64_t rid = entries[i].rid;
        if (!cache_->has(rid)) cache_->zero_state(cache_->add_request(rid), rt_->stream);
        cache_->reserve(rid, st.starts[(size_t)i] + entries[i].n_tokens);
        st.slots[(size_t)i] = cache_->slot_of(rid);
    }

    int which = 0;
    int32_t* host = buf_.staging(&which);
    const bool decode_only = T == B;
    int t0 = 0, r = 0, max_q = 0, max_kv = 0;
    int32_t* q_start = host + buf_.off_q_start;
    for (int s = 0; s < B; ++s) {
        const auto& e = entries[s];
        const int n = e.n_tokens, start = st.starts[(size_t)s];
        for (int t = 0; t < n; ++t) {
            host[buf_.off_tok + (size_t)(t0 + t)] = e.tokens ? e.tokens[t] : 0;
            host[buf_.off_pos + (size_t)(t0 + t)] = start + t;
            host[buf_.off_seq + (size_t)(t0 + t)] = s;
        }
        for (int w = 0; w < e.n_want; ++w) host[buf_.off_rows + (size_t)r++] = t0 + e.want[w];
        q_start[s] = t0;
        host[buf_.off_kv_len + (size_t)s] = start + n;
        host[buf_.off_slots + (size_t)s] = st.slots[(size_t)s];
        max_q = std::max(max_q, n);
        max_kv = std::max(max_kv, start + n);
        t0 += n;
    }
    q_start[B] = T;
    for (size_t g = 0; g < cache_->paged().size(); ++g) {
        const PagedGroup& grp = cache_->paged()[g];
        int32_t* view = host + buf_.off_bt[g];
        const int width = std::min(grp.width, buf_.max_pages);
        for (int s = 0; s < B; ++s) {
            int32_t* row = view + (size_t)s * buf_.max_pages;
            std::copy(grp.row(st.slots[(size_t)s]), grp.row(st.slots[(size_t)s]) + width, row);
            std::fill(row + width, row + buf_.max_pages, -1);
        }
    }
    std::vector<int> tile_counts(tilings_.size(), 0);
    if (!decode_only) {
        // Each declared tiling: runs of up to `tile` consecutive tokens of every sequence whose portion length
        // lies in [min_len, max_len).
        for (size_t k = 0; k < tilings_.size(); ++k) {
            const TilingSpec& ts = tilings_[k];
            int32_t* tok0 = host + buf_.off_tile0[k];
            int32_t* tn = host + buf_.off_tilen[k];
            int c = 0;
            for (int s = 0; s < B; ++s) {
                const int n = st.q_lens[(size_t)s];
                if (n < ts.min_len || (ts.max_len > 0 && n >= ts.max_len)) continue;
                for (int a = 0; a < n; a += ts.tile) {
                    tok0[c] = q_start[s] + a;
                    tn[c] = std::min(ts.tile, n - a);
                    ++c;
                }
            }
            tile_counts[k] = c;
        }
    }
    buf_.upload(which, B, rt_->stream);
    h2d_bytes_last_step = (int64_t)(buf_.small_words + buf_.off_bt.size() * (size_t)B * (size_t)buf_.max_pages) * 4;

    int32_t* d = buf_.dev();
    ImpBatchView& v = st.view;
    v = ImpBatchView{};
    v.n_tokens = T;
    v.n_seqs = B;
    v.n_rows = R;
    v.decode_only = decode_only ? 1 : 0;
    v.max_q_len = max_q;
    v.max_kv_len = max_kv;
    v.token_ids = d + buf_.off_tok;
    v.positions = d + buf_.off_pos;
    v.seq_of_token = d + buf_.off_seq;
    v.logit_rows = d + buf_.off_rows;
    v.q_start = d + buf_.off_q_start;
    v.kv_len = d + buf_.off_kv_len;
    v.state_slots = d + buf_.off_slots;
    v.host_q_lens = st.q_lens.data();
    v.host_starts = st.starts.data();
    v.host_slots = st.slots.data();
    v.stream = rt_->stream;
    v.status = rt_->status;
    v.compute_dtype = rt_->dtype;
    v.step = &st;
    st.block_tables.clear();
    for (size_t g = 0; g < buf_.off_bt.size(); ++g) st.block_tables.push_back(d + buf_.off_bt[g]);
    st.bt_stride = buf_.max_pages;
    st.tiles.assign(tilings_.size(), Tiles());
    for (size_t k = 0; k < tilings_.size(); ++k)
        st.tiles[k] = Tiles{d + buf_.off_tile0[k], d + buf_.off_tilen[k], tile_counts[k]};
    return st;
}

void Stepper::commit(const Step& st) {
    for (size_t i = 0; i < st.rids.size(); ++i) cache_->commit(st.rids[i], st.starts[i] + st.q_lens[i]);
}

Tensor Stepper::step(const StepEntryView* entries, int n, const int32_t* device_tokens) {
    if (!model_) fail(IMP_ERROR_INTERNAL, "this step function has no model");
    rt_->arena->begin_step(rt_->stream);
    if (rt_->arena->generation() != arena_generation_) {
        drop_graphs();   // the workspace moved: addresses baked into captured graphs are stale
        arena_generation_ = rt_->arena->generation();
    }
    Step& st = prepare(entries, n);
    if (device_tokens)
        IMP_CUDA(cudaMemcpyAsync((void*)st.view.token_ids, device_tokens, (size_t)st.T() * 4, cudaMemcpyDeviceToDevice, rt_->stream));
    Tensor logits;
    if (use_graphs_ && st.decode_only() && st.R() == st.B()) {
        logits = forward_decode_graph(st);
    } else {
        ++eager_steps;
        logits = model_->forward(st);
    }
    commit(st);
    return logits;
}

// Decode-only batches of a given size replay one captured CUDA graph.  The batch arrays live at fixed
// addresses and the workspace hands out the same addresses for the same sequence of requests, so a graph
// captured for B sequences serves every later step of B sequences; only the arrays' contents change.  The
// first step of a size runs eagerly (it sizes the workspace and sets kernel attributes), the second is
// captured.  The returned logits are the graph's own: read them before the next step.
Tensor Stepper::forward_decode_graph(Step& st) {
    // one graph per batch size and context class: the decode attention's key splits depend on both
    int ctx_class = 0;
    while ((1 << ctx_class) < st.context && ctx_class < 30) ++ctx_class;
    const int B = st.B(), key = B * 32 + ctx_class;
    auto hit = graphs_.find(key);
    if (hit == graphs_.end()) {
        const int uses = graph_uses_[key]++;
        if (uses == 0) {
            ++eager_steps;
            return model_->forward(st);
        }
        const uint64_t gen = rt_->arena->generation();
        const int64_t launches_before = rt_->launches;
        cudaGraph_t graph = nullptr;
        Tensor logits{};
        IMP_CUDA(cudaStreamSynchronize(rt_->stream));
        IMP_CUDA(cudaStreamBeginCapture(rt_->stream, cudaStreamCaptureModeThreadLocal));
        rt_->arena->freeze(true);
        try {
            logits = model_->forward(st);
        } catch (...) {
            rt_->arena->freeze(false);
            cudaStreamEndCapture(rt_->stream, &graph);
            if (graph) cudaGraphDestroy(graph);
            (void)cudaGetLastError();
            graph_uses_[key] = 0;        // try again after an eager step has sized the workspace
            rt_->arena->begin_step(rt_->stream);
            ++eager_steps;
            return model_->forward(st);
        }
        rt_->arena->freeze(false);
        IMP_CUDA(cudaStreamEndCapture(rt_->stream, &graph));
        Graph g;
        g.logits = logits;
        g.mark = rt_->arena->mark();
        g.launches = rt_->launches - launches_before;   // launcher calls the graph stands for
        rt_->launches = launches_before;
        cudaError_t e = cudaGraphInstantiate(&g.exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) fail(IMP_ERROR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
        if (gen != rt_->arena->generation()) fail(IMP_ERROR_INTERNAL, "the workspace moved during graph capture");
        ++graph_captures;
        hit = graphs_.emplace(key, g).first;
    }
    rt_->arena->restore(hit->second.mark);
    IMP_CUDA(cudaGraphLaunch(hit->second.exec, rt_->stream));
    rt_->launches += hit->second.launches;
    ++graph_replays;
    return hit->second.logits;
}

void Stepper::check_device_status(const std::string& what) {
    int32_t code = 0;
    IMP_CUDA(cudaMemcpyAsync(&code, rt_->status, 4, cudaMemcpyDeviceToHost, rt_->stream));
    IMP_CUDA(cudaStreamSynchronize(rt_->stream));
    if (code != 0) {
        IMP_CUDA(cudaMemsetAsync(rt_->status, 0, 4, rt_->stream));
        fail(IMP_ERROR_CUDA, what + ": device reported '" + imp_status_string(code) + "' (code " + std::to_string(code) + ")");
    }
}

}  // namespace imp
