#include "model.hpp"

#include <algorithm>
#include <cmath>

#include "diagnostics.hpp"
#include "kernels.h"
#include "ops.hpp"

namespace imp {

// ---------------------------------------------------------------------------------- host model
static void describe(HostModel& m, const Json& config, const std::string& where) {
    const Architecture& arch = architecture_of(config, where);
    m.config_json = config;
    m.config = arch.parse_config(config, where);
    m.plan = arch.plan(config);
    if (m.plan.architecture.empty()) m.plan.architecture = m.config->architecture;
    m.expected = m.plan.expected_tensors();
    m.config_text = m.config->to_json().dump();
    m.plan_text = m.plan.to_json().dump();
    m.arch_text = m.config->architecture;
}

std::unique_ptr<HostModel> HostModel::load(const std::string& path) {
    auto m = std::make_unique<HostModel>();
    std::string where;
    const Json config = read_config_json(path, &where, &m->folder);
    if (m->folder.empty()) fail(IMP_ERROR_INVALID_ARG, "imp_model_load takes a folder or a config.json path, not JSON text");
    describe(*m, config, where);
    m->files = open_model_files(m->folder);
    std::map<std::string, FoundTensor> found;
    for (const auto& f : m->files)
        for (const auto& kv : f->tensors()) {
            m->stored[kv.first] = kv.second;
            found[kv.first] = FoundTensor{kv.second.shape, kv.second.dtype};
        }
    check_checkpoint(m->expected, found, m->plan.ignored_tensors, m->folder);
    return m;
}

std::unique_ptr<HostModel> HostModel::make_random(const std::string& config_path_or_text, int64_t seed, float std, float norm_std) {
    auto m = std::make_unique<HostModel>();
    std::string where;
    const Json config = read_config_json(config_path_or_text, &where, &m->folder);
    describe(*m, config, where);
    m->random = true;
    m->seed = seed;
    m->std = std;
    m->norm_std = norm_std;
    return m;
}

Json HostModel::tensor_info(int compute_dtype) const {
    Json j = Json::object();
    for (const auto& e : expected) {
        Json o = Json::object();
        std::string stored = config->torch_dtype == "float32" ? "F32" : "BF16";
        if (e.second.role == "int_table") stored = "I32";
        auto it = this->stored.find(e.first);
        if (!random) {
            if (it == this->stored.end()) continue;
            stored = it->second.dtype;
        }
        o["stored"] = stored;
        o["device"] = dtype_name(device_dtype(stored, e.second.role, compute_dtype));
        o["shape"] = Json::array_of(e.second.shape);
        o["role"] = e.second.role;
        j[e.first] = o;
    }
    return j;
}

// ---------------------------------------------------------------------------------- diagnostics
Diagnostics::Diagnostics() : profile(env_flag("IMP_B200_PROFILE", false)), debug(env_flag("IMP_B200_DEBUG_FORWARD", false)) {}
Diagnostics::~Diagnostics() {
    for (auto e : events_) cudaEventDestroy(e);
}

void Diagnostics::begin(Step& st) {
    n_stamps_ = 0;
    names_.clear();
    last_stats = Json::array();
    if (profile) stamp(st, "start");
}

void Diagnostics::stamp(Step& st, const std::string& name) {
    if ((size_t)n_stamps_ == events_.size()) {
        cudaEvent_t e;
        IMP_CUDA(cudaEventCreate(&e));
        events_.push_back(e);
    }
    IMP_CUDA(cudaEventRecord(events_[(size_t)n_stamps_++], st.rt->stream));
    names_.push_back(name);
}

void Diagnostics::stage(Step& st, const std::string& name, const Tensor& t) {
    if (profile) stamp(st, name);
    if (debug && t.data && numel(t) > 0 && (t.dtype == F32 || t.dtype == BF16) && contiguous(t)) {
        if (!stats_.data()) {
            stats_ = DeviceBuffer(5 * sizeof(float));
        }
        check_launch(imp_tensor_stats(t.data, t.dtype, numel(t), (float*)stats_.data(), st.rt->stream), "tensor_stats");
        float s[5];
        IMP_CUDA(cudaMemcpyAsync(s, stats_.data(), sizeof s, cudaMemcpyDeviceToHost, st.rt->stream));
        IMP_CUDA(cudaStreamSynchronize(st.rt->stream));
        const double n = (double)numel(t) - s[4];
        Json o = Json::object();
        o["stage"] = name;
        o["shape"] = shape_string(t);
        o["min"] = (double)s[0];
        o["max"] = (double)s[1];
        o["mean"] = n > 0 ? s[2] / n : 0.0;
        o["l2"] = std::sqrt((double)s[3]);
        o["nan"] = (int64_t)s[4];
        last_stats.push(o);
        fprintf(stderr, "[debug_forward] %-24s %-16s min %+.5g max %+.5g mean %+.5g l2 %.5g nan %d\n", name.c_str(),
                shape_string(t).c_str(), s[0], s[1], n > 0 ? s[2] / n : 0.0, std::sqrt((double)s[3]), (int)s[4]);
    }
}

void Diagnostics::end(Step& st, const Tensor& logits) {
    if (debug && logits.data && rows(logits) > 0) {
        // the ten largest logits of the first wanted row
        const int64_t V = cols(logits);
        std::vector<float> row((size_t)V);
        IMP_CUDA(cudaMemcpyAsync(row.data(), logits.data, (size_t)V * 4, cudaMemcpyDeviceToHost, st.rt->stream));
        IMP_CUDA(cudaStreamSynchronize(st.rt->stream));
        std::vector<int> idx((size_t)V);
        for (int64_t i = 0; i < V; ++i) idx[(size_t)i] = (int)i;
        const size_t k = (size_t)std::min<int64_t>(10, V);
        std::partial_sort(idx.begin(), idx.begin() + (long)k, idx.end(), [&](int a, int b) { return row[(size_t)a] > row[(size_t)b] || (row[(size_t)a] == row[(size_t)b] && a < b); });
        Json top = Json::array();
        std::string line = "[debug_forward] top logits:";
        for (size_t i = 0; i < k; ++i) {
            Json o = Json::object();
            o["token"] = idx[i];
            o["logit"] = (double)row[(size_t)idx[i]];
            top.push(o);
            char buf[64];
            snprintf(buf, sizeof buf, " %d:%.4f", idx[i], row[(size_t)idx[i]]);
            line += buf;
        }
        last_top = top;
        fprintf(stderr, "%s\n", line.c_str());
    }
    if (!profile || n_stamps_ < 2) return;
    IMP_CUDA(cudaEventSynchronize(events_[(size_t)n_stamps_ - 1]));
    float total = 0.f;
    IMP_CUDA(cudaEventElapsedTime(&total, events_[0], events_[(size_t)n_stamps_ - 1]));
    if (sums_.size() != (size_t)n_stamps_ - 1 || sum_names_ != names_) {
        sums_.assign((size_t)n_stamps_ - 1, 0.0);
        sum_names_ = names_;
        steps_ = 0;
        total_ms_ = 0;
    }
    for (int i = 1; i < n_stamps_; ++i) {
        float ms = 0.f;
        IMP_CUDA(cudaEventElapsedTime(&ms, events_[(size_t)i - 1], events_[(size_t)i]));
        sums_[(size_t)i - 1] += ms;
    }
    total_ms_ += total;
    ++steps_;
    last_step_ms = total;
    if (steps_ % 32 == 0) print_profile();
}

Json Diagnostics::profile_json() const {
    Json j = Json::object();
    j["steps"] = steps_;
    j["ms_per_step"] = steps_ ? total_ms_ / steps_ : 0.0;
    j["last_step_ms"] = (double)last_step_ms;
    Json st = Json::array();
    for (size_t i = 0; i < sums_.size(); ++i) {
        Json o = Json::object();
        o["stage"] = sum_names_[i + 1];
        o["ms"] = steps_ ? sums_[i] / steps_ : 0.0;
        st.push(o);
    }
    j["stages"] = st;
    return j;
}

void Diagnostics::print_profile() const {
    fprintf(stderr, "[profile] %d steps, %.3f ms per step\n", steps_, steps_ ? total_ms_ / steps_ : 0.0);
    // embedding, per-layer mixer and feed-forward, head: averaged, as the reference prints them
    // (src/graph/executor_forward.cu:3093-3139)
    for (size_t i = 0; i < sums_.size(); ++i)
        fprintf(stderr, "[profile]   %-28s %9.4f ms\n", sum_names_[i + 1].c_str(), sums_[i] / steps_);
}

void stage(Step& st, const char* name, const Tensor& t) {
    if (!st.diag) return;
    st.diag->stage(st, st.layer >= 0 ? "layer" + std::to_string(st.layer) + "." + name : std::string(name), t);
}

void stage(Step& st, const char* name, const Branch& b) {
    if (st.diag) stage(st, name, b.split() ? Tensor{} : b.t);
}

// -------------------------------------------------------------------------------- device model
DeviceModel::DeviceModel(const HostModel& host, Runtime* rt) : plan_(host.plan), rt_(rt), factory_(rt, &store_) {
    std::vector<std::pair<std::string, Tensor>> placed;
    const std::string stored_default = host.config->torch_dtype == "float32" ? "F32" : "BF16";
    for (const auto& e : host.expected) {
        if (host.random) {
            placed.emplace_back(e.first, random_device_tensor(e.first, e.second, host.seed, host.std, host.norm_std, stored_default,
                                                              rt->dtype, store_, rt->stream));
        } else {
            auto it = host.stored.find(e.first);
            if (it == host.stored.end()) continue;   // optional and absent
            placed.emplace_back(e.first, place_tensor(it->second, e.second.role, rt->dtype, store_, rt->stream));
        }
    }
    IMP_CUDA(cudaStreamSynchronize(rt->stream));
    build(placed);
}

DeviceModel::DeviceModel(const ModelPlan& plan, const std::vector<std::pair<std::string, Tensor>>& tensors, Runtime* rt)
    : plan_(plan), rt_(rt), factory_(rt, &store_) {
    const auto expected = plan_.expected_tensors();
    std::map<std::string, FoundTensor> found;
    for (const auto& kv : tensors)
        found[kv.first] = FoundTensor{std::vector<int64_t>(kv.second.shape, kv.second.shape + kv.second.ndim),
                                      kv.second.dtype == F32 ? "F32" : kv.second.dtype == BF16 ? "BF16" : "I32"};
    check_checkpoint(expected, found, plan_.ignored_tensors, "(in memory)");
    std::vector<std::pair<std::string, Tensor>> placed;
    for (const auto& e : expected)
        for (const auto& kv : tensors)
            if (kv.first == e.first) placed.emplace_back(e.first, place_device_tensor(kv.second, e.second.role, rt->dtype, store_, rt->stream));
    IMP_CUDA(cudaStreamSynchronize(rt->stream));
    build(placed);
}

DeviceModel::~DeviceModel() = default;

void DeviceModel::build(const std::vector<std::pair<std::string, Tensor>>& placed) {
    auto take = [&](const PartSpec& spec) {
        std::vector<std::pair<std::string, Tensor>> out;
        for (const auto& t : spec.tensors)
            for (const auto& p : placed)
                if (p.first == t.second) out.emplace_back(t.first, p.second);
        return out;
    };
    embedding_ = part_cast<Embedding>(factory_.build("embedding", plan_.embedding, take(plan_.embedding)), "an embedding");
    for (const auto& layer : plan_.layers) {
        const PartClass& bc = part_class("block", layer.block);
        std::vector<std::pair<std::string, Part*>> parts;
        int mixers = 0;
        for (const auto& slot : bc.part_slots(layer.block_params)) {
            const PartSpec* ps = layer.part(slot.name);
            if (!ps) fail(IMP_ERROR_INVALID_MODEL, "block '" + layer.block + "' needs a part in its slot '" + slot.name + "'");
            parts.emplace_back(slot.name, factory_.build(slot.category, *ps, take(*ps)));
            mixers += slot.category == "mixer";
        }
        if (mixers > 1) fail(IMP_ERROR_UNSUPPORTED, "block '" + layer.block + "': a block holds at most one mixer (one cache per layer)");
        PartSpec bs;
        bs.kind = layer.block;
        bs.params = layer.block_params;
        blocks_.push_back(part_cast<Block>(factory_.build("block", bs, {}, parts), "a block"));
    }
    final_norm_ = part_cast<Norm>(factory_.build("norm", plan_.final_norm, take(plan_.final_norm)), "a norm");
    head_ = part_cast<Head>(factory_.build("head", plan_.head, take(plan_.head)), "a head");
    finish_build();
}

void DeviceModel::finish_build() {
    order_ = plan_.run_order();
    // A block may hand on an unsummed branch only if whoever normalises the stream after it, at every place it
    // has in the run order, adds the parts itself.
    std::vector<bool> after_ok(blocks_.size(), true);
    for (size_t j = 0; j < order_.size(); ++j) {
        const bool next_takes = j + 1 < order_.size() ? blocks_[(size_t)order_[j + 1]]->takes_split_sum() : final_norm_->takes_split_sum();
        after_ok[(size_t)order_[j]] = after_ok[(size_t)order_[j]] && next_takes;
    }
    for (size_t i = 0; i < blocks_.size(); ++i) blocks_[i]->defer_pending = after_ok[i];
    // Cache needs per run position, and which position's cache each position uses.
    std::map<int, int> last_position_of_layer;
    for (size_t j = 0; j < order_.size(); ++j) {
        const int i = order_[j];
        const LayerSpec& layer = plan_.layers[(size_t)i];
        if (layer.cache_from < 0) {
            CacheSpec spec;
            const PartClass& bc = part_class("block", layer.block);
            for (const auto& slot : bc.part_slots(layer.block_params))
                if (slot.category == "mixer") {
                    const PartSpec* ps = layer.part(slot.name);
                    const PartClass& mc = part_class("mixer", ps->kind);
                    if (mc.cache_spec) spec = mc.cache_spec(ps->params);
                }
            cache_specs_.push_back(spec);
            cache_position_.push_back((int)j);
            last_position_of_layer[i] = (int)j;
        } else {
            auto it = last_position_of_layer.find(layer.cache_from);
            if (it == last_position_of_layer.end())
                fail(IMP_ERROR_INVALID_MODEL, "layer " + std::to_string(i) + " reads the cache of layer " + std::to_string(layer.cache_from) +
                                                  ", which has not run before it in the run order");
            cache_specs_.push_back(CacheSpec());
            cache_position_.push_back(it->second);
        }
    }
    layer_caches_.assign(order_.size(), LayerCache());
    // The tilings the mixers want of a step, each distinct one once.
    graph_safe_ = embedding_->graph_safe() && final_norm_->graph_safe() && head_->graph_safe();
    for (Block* b : blocks_) {
        graph_safe_ = graph_safe_ && b->graph_safe();
        for (Part* p : b->parts()) graph_safe_ = graph_safe_ && p->graph_safe();
        if (Mixer* m = b->mixer()) {
            m->tiling_ids.clear();
            for (const TilingSpec& t : m->tilings()) {
                auto it = std::find(tilings_.begin(), tilings_.end(), t);
                if (it == tilings_.end()) {
                    tilings_.push_back(t);
                    it = tilings_.end() - 1;
                }
                m->tiling_ids.push_back((int)(it - tilings_.begin()));
            }
        }
    }
    diag_ = std::make_unique<Diagnostics>();
    if (!diag_->profile && !diag_->debug) diag_.reset();
}

void DeviceModel::attach_cache(CacheManager* cache) {
    cache_ = cache;
    for (size_t j = 0; j < order_.size(); ++j) {
        const int src = cache_position_[j];
        LayerCache lc;
        lc.view = cache->layer_view(src, rt_->dtype);
        lc.view.writes = src == (int)j ? 1 : 0;
        lc.group = cache->layer_ref()[(size_t)src].group;
        layer_caches_[j] = lc;
    }
}

Tensor DeviceModel::forward(Step& st) {
    for (auto& lc : layer_caches_)
        if (lc.paged()) {
            lc.view.block_table = st.block_tables.at((size_t)lc.group);
            lc.view.bt_stride = st.bt_stride;
        }
    st.diag = diag_.get();
    st.layer = -1;
    if (diag_) diag_->begin(st);
    Tensor h = embedding_->forward(st);
    stage(st, "embedding", h);
    Branch pending;
    for (size_t j = 0; j < order_.size(); ++j) {
        rt_->arena->next_layer();
        st.layer = order_[j];
        LayerCache* lc = layer_caches_[j].view.kind ? &layer_caches_[j] : nullptr;
        pending = blocks_[(size_t)order_[j]]->forward(st, h, pending, lc);
    }
    st.layer = -1;
    Tensor logits{};
    if (st.R() > 0) {
        Tensor x = final_norm_->add_norm(st, h, pending, st.view.logit_rows, st.R());
        stage(st, "final_norm", x);
        logits = head_->forward(st, x);
        stage(st, "head", logits);
    } else if (!pending.empty() && diag_) {
        stage(st, "last_layer", summed(st, pending));
    }
    if (diag_) diag_->end(st, logits);
    return logits;
}

Json DeviceModel::info_json() const {
    Json j = Json::object();
    j["order"] = Json::array_of(order_);
    j["cache_position"] = Json::array_of(cache_position_);
    Json specs = Json::array();
    for (const auto& s : cache_specs_) specs.push(s.to_json());
    j["cache_specs"] = specs;
    j["graph_safe"] = graph_safe_;
    j["weight_bytes"] = store_.bytes();
    Json tl = Json::array();
    for (const auto& t : tilings_) {
        Json o = Json::object();
        o["tile"] = t.tile;
        o["min_len"] = t.min_len;
        o["max_len"] = t.max_len;
        tl.push(o);
    }
    j["tilings"] = tl;
    Json defer = Json::array(), mixer_defer = Json::array();
    for (const Block* b : blocks_) {
        defer.push(Json(b->defer_pending));
        mixer_defer.push(Json(b->mixer() ? b->mixer()->defer_out : false));
    }
    j["defer_pending"] = defer;
    j["mixer_defer_out"] = mixer_defer;
    if (diag_) {
        if (diag_->profile) j["profile"] = diag_->profile_json();
        if (diag_->debug) {
            j["debug_stages"] = diag_->last_stats;
            j["debug_top_logits"] = diag_->last_top;
        }
    }
    return j;
}

}  // namespace imp
