// Typed model configurations read from an architecture's own config.json keys, the registry from
// an architecture's name to its configuration class and plan function, and the engine settings.
//
// Every size and constant of a model comes from here; no kernel, part or engine file holds a model
// size of its own.  The reference keeps one struct for every family with defaults in the
// declaration (src/model/model.h:28-76), maps an architecture string to an enum
// (src/model/model.cpp:70-103) and, on the safetensors route, guesses the family from tensor names
// and never reads config.json (src/model/safetensors_loader.cpp:238-263, 297-359); this engine reads
// config.json and refuses what it cannot run.
#pragma once

#include <functional>
#include <string>
#include <vector>

#include "plan.hpp"

namespace imp {

// The keys every decoder has.
struct ModelConfig {
    std::string architecture;
    int64_t vocab_size = 0, hidden_size = 0, num_hidden_layers = 0, max_position_embeddings = 4096;
    std::string torch_dtype = "bfloat16";
    std::vector<int> eos_token_ids;        // config.json's eos_token_id: one id or a list
    int64_t bos_token_id = -1;
    Json raw = Json::object();             // config.json as read (architectures registered from outside read their own keys)

    virtual ~ModelConfig() = default;
    virtual Json to_json() const;          // the typed fields, plus the keys this configuration did not interpret
    static void read_base(ModelConfig& c, const Json& d, const std::string& where);
};

// The Qwen3 dense decoder (architectures[0] == "Qwen3ForCausalLM").  Keys follow the HF config.json
// of this architecture.  The reference reads the GGUF twins of the same fields
// (src/model/gguf_loader.cpp:726-738: block_count, embedding_length, head counts,
// attention.key_length, feed_forward_length, rope.freq_base, layer_norm_rms_epsilon; sliding window
// at :821) into src/model/model.h:28-76.
struct Qwen3Config : ModelConfig {
    int64_t num_attention_heads = 0, num_key_value_heads = 0, head_dim = 0, intermediate_size = 0;
    double rms_norm_eps = 1e-6, rope_theta = 10000.0;
    bool tie_word_embeddings = false, attention_bias = false, use_sliding_window = false;
    std::string hidden_act = "silu";
    int64_t sliding_window = 0;            // 0 = none given
    int64_t max_window_layers = -1;        // -1 = not given
    std::vector<std::string> layer_types;  // empty = not given

    static Qwen3Config from_json(const Json& d, const std::string& where);
    void validate(const std::string& where) const;
    // Window in tokens of `layer` (0 = attends to all earlier tokens).  A query at position p sees keys
    // j with 0 <= p - j < window, the mask of the reference's kernels (src/compute/attention.cu:167;
    // decode: src/compute/attention_paged.cu:163-164).
    int64_t window_of_layer(int layer) const;
    Json to_json() const override;
};

ModelPlan qwen3_plan(const Qwen3Config& cfg);

// ------------------------------------------------------------------------------------ registry
struct Architecture {
    std::string name;
    // config.json (parsed) -> typed, validated configuration
    std::function<std::shared_ptr<ModelConfig>(const Json& d, const std::string& where)> parse_config;
    // config.json (parsed) -> plan
    std::function<ModelPlan(const Json& d)> plan;
};

void register_architecture(Architecture a, bool replace = false);
void unregister_architecture(const std::string& name);
std::vector<std::string> known_architectures();
const Architecture& architecture(const std::string& name);    // throws, listing known names
const Architecture& architecture_of(const Json& config, const std::string& where);

// Reads `path` (a folder holding config.json, or the file itself) or takes `text` as JSON.
Json read_config_json(const std::string& path_or_text, std::string* where, std::string* folder);

// ------------------------------------------------------------------------------ engine config
void validate_engine_config(const ImpConfig& c);

}  // namespace imp
