#include "config.hpp"

#include <sys/stat.h>

#include <fstream>
#include <map>
#include <mutex>
#include <sstream>

#include "parts.hpp"

namespace imp {

namespace {
[[noreturn]] void bad(const std::string& msg) { fail(IMP_ERROR_INVALID_MODEL, msg); }

const Json& require(const Json& d, const std::string& key, const std::string& where) {
    const Json* v = d.find(key);
    if (!v) bad(where + ": missing required key '" + key + "'");
    return *v;
}
int64_t require_int(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = require(d, key, where);
    if (!v.is_int()) bad(where + ": key '" + key + "' must be int, got " + v.type_name());
    return v.as_int();
}
double require_float(const Json& d, const std::string& key, const std::string& where) {
    const Json& v = require(d, key, where);
    if (!v.is_number()) bad(where + ": key '" + key + "' must be float, got " + v.type_name());
    return v.as_double();
}
int64_t positive(const std::string& name, int64_t v, const std::string& where) {
    if (v <= 0) bad(where + ": '" + name + "' must be positive, got " + std::to_string(v));
    return v;
}
}  // namespace

// ------------------------------------------------------------------------------- base config
void ModelConfig::read_base(ModelConfig& c, const Json& d, const std::string& where) {
    const Json* archs = d.find("architectures");
    if (!archs || !archs->is_array() || archs->size() == 0 || !(*archs)[0].is_string())
        bad(where + ": 'architectures' must be a list that names the model class");
    c.architecture = (*archs)[0].as_string();
    c.vocab_size = positive("vocab_size", require_int(d, "vocab_size", where), where);
    c.hidden_size = positive("hidden_size", require_int(d, "hidden_size", where), where);
    c.num_hidden_layers = positive("num_hidden_layers", require_int(d, "num_hidden_layers", where), where);
    c.max_position_embeddings = positive("max_position_embeddings", d.get_int("max_position_embeddings", 4096), where);
    c.torch_dtype = d.get_string("torch_dtype", d.get_string("dtype", "bfloat16"));
    if (const Json* eos = d.find("eos_token_id")) {
        if (eos->is_array()) {
            for (const auto& e : eos->items())
                if (e.is_int()) c.eos_token_ids.push_back((int)e.as_int());
        } else if (eos->is_int()) {
            c.eos_token_ids.push_back((int)eos->as_int());
        }
    }
    c.bos_token_id = d.get_int("bos_token_id", -1);
    c.raw = d;
}

Json ModelConfig::to_json() const {
    Json j = raw.is_object() ? raw : Json::object();
    j["architectures"] = Json::array_of(std::vector<std::string>{architecture});
    j["vocab_size"] = vocab_size;
    j["hidden_size"] = hidden_size;
    j["num_hidden_layers"] = num_hidden_layers;
    j["max_position_embeddings"] = max_position_embeddings;
    j["torch_dtype"] = torch_dtype;
    if (eos_token_ids.size() == 1) j["eos_token_id"] = eos_token_ids[0];
    else if (!eos_token_ids.empty()) j["eos_token_id"] = Json::array_of(eos_token_ids);
    if (bos_token_id >= 0) j["bos_token_id"] = bos_token_id;
    j.erase("dtype");
    return j;
}

// ------------------------------------------------------------------------------------- Qwen3
Qwen3Config Qwen3Config::from_json(const Json& d, const std::string& where) {
    Qwen3Config c;
    // hidden_size and the head counts first, so that a missing one is named before anything derived from it
    const int64_t hidden = positive("hidden_size", require_int(d, "hidden_size", where), where);
    const int64_t heads = positive("num_attention_heads", require_int(d, "num_attention_heads", where), where);
    read_base(c, d, where);
    c.num_attention_heads = heads;
    const Json* kv = d.find("num_key_value_heads");
    c.num_key_value_heads = (kv && kv->is_int()) ? kv->as_int() : heads;
    const Json* hd = d.find("head_dim");
    if (hd && hd->is_int()) {
        c.head_dim = hd->as_int();
    } else {
        if (hidden % heads)
            bad(where + ": no 'head_dim' and hidden_size " + std::to_string(hidden) +
                " is not a multiple of num_attention_heads " + std::to_string(heads));
        c.head_dim = hidden / heads;
    }
    c.intermediate_size = positive("intermediate_size", require_int(d, "intermediate_size", where), where);
    c.rms_norm_eps = require_float(d, "rms_norm_eps", where);
    c.rope_theta = d.get_double("rope_theta", 10000.0);
    c.tie_word_embeddings = d.get_bool("tie_word_embeddings", false);
    c.attention_bias = d.get_bool("attention_bias", false);
    c.hidden_act = d.get_string("hidden_act", "silu");
    c.use_sliding_window = d.get_bool("use_sliding_window", false);
    c.sliding_window = d.get_int("sliding_window", 0);
    c.max_window_layers = d.get_int("max_window_layers", -1);
    if (const Json* lt = d.find("layer_types"))
        if (lt->is_array())
            for (const auto& t : lt->items()) c.layer_types.push_back(t.is_string() ? t.as_string() : std::string("?"));
    if (const Json* rs = d.find("rope_scaling"))
        if (!rs->is_null() && !(rs->is_object() && rs->size() == 0))
            bad(where + ": rope_scaling " + rs->dump() + " is not supported (only the plain rotary encoding)");
    c.validate(where);
    return c;
}

void Qwen3Config::validate(const std::string& where) const {
    if (num_key_value_heads <= 0 || num_attention_heads % num_key_value_heads)
        bad(where + ": num_attention_heads " + std::to_string(num_attention_heads) +
            " must be a positive multiple of num_key_value_heads " + std::to_string(num_key_value_heads));
    if (head_dim <= 0 || head_dim % 16) bad(where + ": head_dim " + std::to_string(head_dim) + " must be a positive multiple of 16");
    if (head_dim > 256) bad(where + ": head_dim " + std::to_string(head_dim) + " exceeds the kernels' limit of 256");
    if (attention_bias) bad(where + ": attention_bias=true is not supported for " + architecture);
    if (hidden_act != "silu") bad(where + ": hidden_act '" + hidden_act + "' is not supported (silu only)");
    if (!(rms_norm_eps > 0)) bad(where + ": rms_norm_eps must be positive");
    if (!(rope_theta > 0)) bad(where + ": rope_theta must be positive");
    if (torch_dtype != "bfloat16" && torch_dtype != "float32")
        bad(where + ": torch_dtype '" + torch_dtype + "' is not supported (bfloat16 or float32)");
    bool any_sliding = false;
    if (!layer_types.empty()) {
        if ((int64_t)layer_types.size() != num_hidden_layers)
            bad(where + ": layer_types has " + std::to_string(layer_types.size()) + " entries for " +
                std::to_string(num_hidden_layers) + " layers");
        for (const auto& t : layer_types) {
            if (t != "full_attention" && t != "sliding_attention") bad(where + ": unknown layer type '" + t + "' in layer_types");
            any_sliding = any_sliding || t == "sliding_attention";
        }
    }
    if ((use_sliding_window || any_sliding) && sliding_window <= 0)
        bad(where + ": sliding window in use but 'sliding_window' is not a positive size");
}

int64_t Qwen3Config::window_of_layer(int layer) const {
    if (!layer_types.empty()) return layer_types[(size_t)layer] == "sliding_attention" ? sliding_window : 0;
    if (!use_sliding_window) return 0;
    const int64_t first = max_window_layers >= 0 ? max_window_layers : 0;
    return layer >= first ? sliding_window : 0;
}

Json Qwen3Config::to_json() const {
    Json j = ModelConfig::to_json();
    j["model_type"] = j.get_string("model_type", "qwen3");
    j["num_attention_heads"] = num_attention_heads;
    j["num_key_value_heads"] = num_key_value_heads;
    j["head_dim"] = head_dim;
    j["intermediate_size"] = intermediate_size;
    j["rms_norm_eps"] = rms_norm_eps;
    j["rope_theta"] = rope_theta;
    j["tie_word_embeddings"] = tie_word_embeddings;
    j["attention_bias"] = attention_bias;
    j["hidden_act"] = hidden_act;
    j["use_sliding_window"] = use_sliding_window;
    if (sliding_window > 0) j["sliding_window"] = sliding_window;
    if (max_window_layers >= 0) j["max_window_layers"] = max_window_layers;
    if (!layer_types.empty()) j["layer_types"] = Json::array_of(layer_types);
    return j;
}

// The Qwen3 dense decoder as a plan of parts: pre-norm blocks of grouped-query attention (per-head
// RMSNorm on q and k before the rotary encoding, no bias, head size independent of the width) and a
// SwiGLU feed-forward; final RMSNorm; output head tied to the embedding or its own (the reference's
// forward pass for this family: src/graph/executor_forward.cu:2701-3140; tensor names:
// src/model/safetensors_loader.cpp:366-401 and, for the q/k norms that binder lacks, the GGUF twins
// at src/model/gguf_loader.cpp:387-388).  Everything here is data.
ModelPlan qwen3_plan(const Qwen3Config& cfg) {
    const int64_t d = cfg.hidden_size;
    Json rotary = Json::object();
    rotary["kind"] = "rotary";
    rotary["params"]["head_dim"] = cfg.head_dim;
    rotary["params"]["theta"] = cfg.rope_theta;
    rotary["params"]["max_positions"] = cfg.max_position_embeddings;
    ModelPlan plan;
    plan.architecture = cfg.architecture;
    plan.hidden_size = d;
    plan.vocab_size = cfg.vocab_size;
    plan.max_positions = cfg.max_position_embeddings;
    auto norm = [&](const std::string& tensor) {
        PartSpec n;
        n.kind = "rmsnorm";
        n.params["size"] = d;
        n.params["eps"] = cfg.rms_norm_eps;
        n.tensors = {{"weight", tensor}};
        return n;
    };
    for (int i = 0; i < cfg.num_hidden_layers; ++i) {
        const std::string p = "model.layers." + std::to_string(i) + ".";
        PartSpec attn;
        attn.kind = "gqa_attention";
        attn.params["hidden_size"] = d;
        attn.params["num_heads"] = cfg.num_attention_heads;
        attn.params["num_kv_heads"] = cfg.num_key_value_heads;
        attn.params["head_dim"] = cfg.head_dim;
        attn.params["window"] = cfg.window_of_layer(i);
        attn.params["qk_norm"] = true;
        attn.params["qk_norm_eps"] = cfg.rms_norm_eps;
        attn.params["position"] = rotary;
        attn.tensors = {{"q_proj", p + "self_attn.q_proj.weight"}, {"k_proj", p + "self_attn.k_proj.weight"},
                        {"v_proj", p + "self_attn.v_proj.weight"}, {"o_proj", p + "self_attn.o_proj.weight"},
                        {"q_norm", p + "self_attn.q_norm.weight"}, {"k_norm", p + "self_attn.k_norm.weight"}};
        PartSpec ffn;
        ffn.kind = "swiglu";
        ffn.params["hidden_size"] = d;
        ffn.params["intermediate_size"] = cfg.intermediate_size;
        ffn.tensors = {{"gate_proj", p + "mlp.gate_proj.weight"}, {"up_proj", p + "mlp.up_proj.weight"},
                       {"down_proj", p + "mlp.down_proj.weight"}};
        LayerSpec layer;
        layer.block = "prenorm";
        layer.parts = {{"mixer_norm", norm(p + "input_layernorm.weight")}, {"mixer", attn},
                       {"ffn_norm", norm(p + "post_attention_layernorm.weight")}, {"feed_forward", ffn}};
        plan.layers.push_back(layer);
    }
    plan.embedding.kind = "token_embedding";
    plan.embedding.params["vocab_size"] = cfg.vocab_size;
    plan.embedding.params["hidden_size"] = d;
    plan.embedding.tensors = {{"weight", "model.embed_tokens.weight"}};
    plan.final_norm = norm("model.norm.weight");
    plan.head.kind = "linear_head";
    plan.head.params["vocab_size"] = cfg.vocab_size;
    plan.head.params["hidden_size"] = d;
    plan.head.tensors = {{"weight", cfg.tie_word_embeddings ? "model.embed_tokens.weight" : "lm_head.weight"}};
    // Published tied checkpoints of this family also store the head; the reference binds it when present and
    // aliases the embedding when absent (src/model/weight_map.cpp:182, 330).  With a tied configuration the
    // stored copy is not read.
    if (cfg.tie_word_embeddings) plan.ignored_tensors.push_back("lm_head.weight");
    return plan;
}

// ------------------------------------------------------------------------------------ registry
namespace {
std::mutex g_arch_mutex;
std::map<std::string, Architecture>& archs() {
    static std::map<std::string, Architecture> a;
    return a;
}
void ensure_builtin_archs() {
    static std::once_flag once;
    std::call_once(once, [] {
        Architecture q;
        q.name = "Qwen3ForCausalLM";
        q.parse_config = [](const Json& d, const std::string& where) -> std::shared_ptr<ModelConfig> {
            return std::make_shared<Qwen3Config>(Qwen3Config::from_json(d, where));
        };
        q.plan = [](const Json& d) { return qwen3_plan(Qwen3Config::from_json(d, "config.json")); };
        archs()[q.name] = q;
    });
}
}  // namespace

void register_architecture(Architecture a, bool replace) {
    ensure_builtin_archs();
    std::lock_guard<std::mutex> lock(g_arch_mutex);
    if (archs().count(a.name) && !replace) fail(IMP_ERROR_INVALID_ARG, "architecture '" + a.name + "' is already registered");
    archs()[a.name] = std::move(a);
}

void unregister_architecture(const std::string& name) {
    std::lock_guard<std::mutex> lock(g_arch_mutex);
    archs().erase(name);
}

std::vector<std::string> known_architectures() {
    ensure_builtin_archs();
    std::lock_guard<std::mutex> lock(g_arch_mutex);
    std::vector<std::string> out;
    for (const auto& kv : archs()) out.push_back(kv.first);
    return out;
}

const Architecture& architecture(const std::string& name) {
    ensure_builtin_archs();
    std::lock_guard<std::mutex> lock(g_arch_mutex);
    auto it = archs().find(name);
    if (it == archs().end()) {
        std::string known;
        for (const auto& kv : archs()) known += (known.empty() ? "" : ", ") + kv.first;
        bad("unknown architecture '" + name + "'; known: " + (known.empty() ? "(none)" : known));
    }
    return it->second;
}

const Architecture& architecture_of(const Json& config, const std::string& where) {
    if (!config.is_object()) bad(where + ": top level must be an object");
    const Json* a = config.find("architectures");
    if (!a || !a->is_array() || a->size() == 0 || !(*a)[0].is_string())
        bad(where + ": 'architectures' must be a list that names the model class");
    return architecture((*a)[0].as_string());
}

Json read_config_json(const std::string& path_or_text, std::string* where, std::string* folder) {
    size_t first = path_or_text.find_first_not_of(" \t\r\n");
    if (first != std::string::npos && path_or_text[first] == '{') {
        if (where) *where = "config";
        if (folder) folder->clear();
        try {
            return Json::parse(path_or_text, "config");
        } catch (const std::exception& e) {
            bad(e.what());
        }
    }
    std::string path = path_or_text;
    struct stat st;
    if (stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode)) {
        if (folder) *folder = path;
        path += "/config.json";
    } else if (folder) {
        size_t slash = path.find_last_of('/');
        *folder = slash == std::string::npos ? "." : path.substr(0, slash);
    }
    std::ifstream f(path, std::ios::binary);
    if (!f) fail(IMP_ERROR_FILE_NOT_FOUND, "no config.json at " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    if (where) *where = path;
    try {
        Json j = Json::parse(ss.str(), path);
        if (!j.is_object()) bad(path + ": top level must be an object");
        return j;
    } catch (const Error&) {
        throw;
    } catch (const std::exception& e) {
        bad(e.what());
    }
}

// ------------------------------------------------------------------------------ engine config
void validate_engine_config(const ImpConfig& c) {
    auto arg = [](const std::string& m) { fail(IMP_ERROR_INVALID_ARG, m); };
    if (c.compute_dtype != IMP_COMPUTE_BF16 && c.compute_dtype != IMP_COMPUTE_FP32)
        arg("compute_dtype must be bfloat16 or float32");
    if (c.max_batch_size <= 0) arg("max_batch_size must be positive");
    if (c.max_seq_len <= 0) arg("max_seq_len must be positive");
    if (c.kv_block_size <= 0) arg("kv_block_size must be positive");
    if (c.max_batch_tokens <= 0) arg("max_batch_tokens must be positive");
    if (c.prefill_chunk_size < 0) arg("prefill_chunk_size must be >= 0");
    if (c.max_batch_tokens < c.max_batch_size)
        arg("max_batch_tokens must be at least max_batch_size (one token per decoding request)");
    if (c.device_id < 0) arg("device_id must be >= 0");
    if (c.state_slots < 0) arg("state_slots must be >= 0");
    if (!(c.gpu_memory_fraction > 0.f) || c.gpu_memory_fraction > 1.f) arg("gpu_memory_fraction must be in (0, 1]");
}

}  // namespace imp
