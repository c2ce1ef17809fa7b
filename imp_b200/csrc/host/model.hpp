// A model: first as a description on the host (configuration, plan, where its tensors come from),
// then assembled on the device from the plan's parts.
//
// DeviceModel::forward(step) is the whole forward pass of one step over the batch the step
// describes: embedding, blocks in their run order, final norm on the wanted rows, head.  It runs
// only the tokens it is given, reads and writes the cache through the per-position LayerCache
// objects, and returns 32-bit logits for the rows that were asked for.  It is the same function for
// whole prompts, portions, single decode tokens and any mix of them (the reference has separate
// prefill and decode paths and no mixed batch: src/graph/executor_forward.cu:568-701).
//
// Cache ownership follows the run order, not the layer list: every position of the run order whose
// layer owns a cache gets a cache of its own (a layer named twice must not overwrite its first
// pass's keys), and a layer with `cache_from` reads the cache of the latest earlier position that ran
// that other layer.
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "cache.hpp"
#include "config.hpp"
#include "weights.hpp"

namespace imp {

// What imp_model_load / imp_model_random make: everything about a model that needs no device.
struct HostModel {
    std::shared_ptr<ModelConfig> config;
    Json config_json;                 // config.json as read
    ModelPlan plan;
    std::vector<std::pair<std::string, TensorSpec>> expected;
    // tensors from files ...
    std::string folder;
    std::vector<std::unique_ptr<SafetensorsFile>> files;
    std::map<std::string, StoredTensor> stored;
    // ... or random
    bool random = false;
    int64_t seed = 0;
    float std = 0.02f, norm_std = 0.01f;
    // strings handed out through the C API
    std::string config_text, plan_text, arch_text;

    static std::unique_ptr<HostModel> load(const std::string& path);
    static std::unique_ptr<HostModel> make_random(const std::string& config, int64_t seed, float std, float norm_std);
    Json tensor_info(int compute_dtype) const;   // name -> stored type, device type, shape
};

// Per-part event timers and per-stage statistics (IMP_B200_PROFILE, IMP_B200_DEBUG_FORWARD).
struct Diagnostics;

class DeviceModel {
public:
    // Places the tensors (from the files, or random ones made on the device) and builds the parts.
    DeviceModel(const HostModel& host, Runtime* rt);
    // From tensors that already live on the device, by checkpoint name (copied).
    DeviceModel(const ModelPlan& plan, const std::vector<std::pair<std::string, Tensor>>& tensors, Runtime* rt);
    ~DeviceModel();

    const ModelPlan& plan() const { return plan_; }
    int64_t hidden_size() const { return plan_.hidden_size; }
    int64_t vocab_size() const { return plan_.vocab_size; }
    const std::vector<int>& order() const { return order_; }
    const std::vector<CacheSpec>& cache_specs() const { return cache_specs_; }      // per run position
    const std::vector<int>& cache_position() const { return cache_position_; }      // which position's cache each uses
    const std::vector<TilingSpec>& tilings() const { return tilings_; }             // what the step function must fill
    bool graph_safe() const { return graph_safe_; }
    size_t weight_bytes() const { return store_.bytes(); }

    void attach_cache(CacheManager* cache);
    // Runs the batch; float32 logits [step.R(), vocab] (data == nullptr when no row was wanted).
    Tensor forward(Step& st);
    Json info_json() const;
    Diagnostics* diagnostics() { return diag_.get(); }

private:
    void build(const std::vector<std::pair<std::string, Tensor>>& placed);
    void finish_build();
    ModelPlan plan_;
    Runtime* rt_;
    WeightStore store_;
    PartFactory factory_;
    Embedding* embedding_ = nullptr;
    std::vector<Block*> blocks_;
    Norm* final_norm_ = nullptr;
    Head* head_ = nullptr;
    std::vector<int> order_, cache_position_;
    std::vector<CacheSpec> cache_specs_;
    std::vector<LayerCache> layer_caches_;
    std::vector<TilingSpec> tilings_;
    bool graph_safe_ = true;
    CacheManager* cache_ = nullptr;
    std::unique_ptr<Diagnostics> diag_;
};

}  // namespace imp
