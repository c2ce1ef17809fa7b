// The data that describes a model: which parts, with which sizes, in which order.
//
// A ModelPlan is what an architecture's plan function makes of its configuration.  It is pure
// data and round-trips through JSON: part kinds are names resolved through the part registry
// (parts.hpp), sizes and constants are parameters, tensor names are the checkpoint's own, a layer
// is a block kind with named part slots that the block class declares, and the order in which
// layers run is a list (which may name a layer twice).  A layer may read another layer's cache
// (`cache_from`).  The reference has no such description: its forward pass is one function that
// switches on tensor presence (src/graph/executor_forward.cu:2701-3140, layer kinds at
// src/graph/executor_workspace.cu:2314-2330).
#pragma once

#include <string>
#include <utility>
#include <vector>

#include "core.hpp"

namespace imp {

// What a part expects of one checkpoint tensor.
struct TensorSpec {
    std::vector<int64_t> shape;
    std::string role = "matrix";   // "matrix" | "norm" | "vector" | "int_table"
    std::string init = "normal";   // random-weights rule: "normal" | "one_plus_normal" | "zeros" | "arange_mod"
    bool optional = false;
    Json to_json() const;
    static TensorSpec from_json(const Json& j);
    int64_t numel() const;
};
using TensorSpecs = std::vector<std::pair<std::string, TensorSpec>>;   // by local name, in a fixed order
Json tensor_specs_to_json(const TensorSpecs& s);
TensorSpecs tensor_specs_from_json(const Json& j);

// One part: its kind, its parameters, and the checkpoint name of each of its tensors.
struct PartSpec {
    std::string kind;
    Json params = Json::object();
    std::vector<std::pair<std::string, std::string>> tensors;   // local name -> checkpoint tensor name
    Json to_json() const;
    static PartSpec from_json(const Json& j, const std::string& where);
    bool empty() const { return kind.empty(); }
};

// One layer: a block kind and the parts that fill the slots the block declares.
struct LayerSpec {
    std::string block = "prenorm";
    Json block_params = Json::object();
    std::vector<std::pair<std::string, PartSpec>> parts;   // slot name -> part
    int cache_from = -1;   // index of the layer whose cache this layer's mixer reads (it writes none)
    const PartSpec* part(const std::string& slot) const;
    PartSpec* part(const std::string& slot);
};

struct ModelPlan {
    std::string architecture;
    int64_t hidden_size = 0, vocab_size = 0, max_positions = 4096;
    PartSpec embedding, final_norm, head;
    std::vector<LayerSpec> layers;
    bool has_order = false;
    std::vector<int> order;                      // run order of layer indices; none = 0..L-1
    std::vector<std::string> ignored_tensors;    // names a checkpoint may hold that the model does not read

    std::vector<int> run_order() const;          // checked against the number of layers
    Json to_json() const;
    static ModelPlan from_json(const Json& j);

    // Checkpoint tensor name -> what is expected of it, over all parts, in plan order.  Two parts
    // may name the same tensor (a tied output head); their shapes must then agree.
    std::vector<std::pair<std::string, TensorSpec>> expected_tensors() const;
};

}  // namespace imp
