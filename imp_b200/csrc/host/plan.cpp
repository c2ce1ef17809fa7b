#include "plan.hpp"

#include "parts.hpp"

namespace imp {

// ------------------------------------------------------------------------------- tensor specs
Json TensorSpec::to_json() const {
    Json j = Json::object();
    j["shape"] = Json::array_of(shape);
    j["role"] = role;
    j["init"] = init;
    j["optional"] = optional;
    return j;
}

TensorSpec TensorSpec::from_json(const Json& j) {
    TensorSpec s;
    for (const auto& d : j.at("shape").items()) s.shape.push_back(d.as_int());
    s.role = j.get_string("role", "matrix");
    s.init = j.get_string("init", s.role == "norm" ? "one_plus_normal" : s.role == "int_table" ? "arange_mod" : "normal");
    s.optional = j.get_bool("optional", false);
    static const char* roles[] = {"matrix", "norm", "vector", "int_table"};
    bool ok = false;
    for (const char* r : roles) ok = ok || s.role == r;
    if (!ok) fail(IMP_ERROR_INVALID_ARG, "tensor spec: unknown role '" + s.role + "'");
    return s;
}

int64_t TensorSpec::numel() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
}

Json tensor_specs_to_json(const TensorSpecs& s) {
    Json j = Json::object();
    for (const auto& kv : s) j[kv.first] = kv.second.to_json();
    return j;
}

TensorSpecs tensor_specs_from_json(const Json& j) {
    TensorSpecs out;
    if (j.is_null()) return out;
    for (const auto& m : j.members()) out.emplace_back(m.first, TensorSpec::from_json(m.second));
    return out;
}

// ---------------------------------------------------------------------------------- part spec
Json PartSpec::to_json() const {
    Json j = Json::object();
    j["kind"] = kind;
    j["params"] = params;
    Json t = Json::object();
    for (const auto& kv : tensors) t[kv.first] = kv.second;
    j["tensors"] = t;
    return j;
}

PartSpec PartSpec::from_json(const Json& j, const std::string& where) {
    if (!j.is_object() || !j.has("kind") || !j.at("kind").is_string())
        fail(IMP_ERROR_INVALID_MODEL, "plan: " + where + " must be an object with a 'kind'");
    PartSpec s;
    s.kind = j.at("kind").as_string();
    if (const Json* p = j.find("params")) {
        if (!p->is_object() && !p->is_null()) fail(IMP_ERROR_INVALID_MODEL, "plan: " + where + ".params must be an object");
        if (p->is_object()) s.params = *p;
    }
    if (const Json* t = j.find("tensors")) {
        if (t->is_object())
            for (const auto& m : t->members()) {
                if (!m.second.is_string())
                    fail(IMP_ERROR_INVALID_MODEL, "plan: " + where + ".tensors." + m.first + " must be a tensor name");
                s.tensors.emplace_back(m.first, m.second.as_string());
            }
    }
    return s;
}

const PartSpec* LayerSpec::part(const std::string& slot) const {
    for (const auto& kv : parts)
        if (kv.first == slot) return &kv.second;
    return nullptr;
}
PartSpec* LayerSpec::part(const std::string& slot) {
    return const_cast<PartSpec*>(static_cast<const LayerSpec*>(this)->part(slot));
}

// ----------------------------------------------------------------------------------- the plan
std::vector<int> ModelPlan::run_order() const {
    std::vector<int> o;
    if (!has_order) {
        for (size_t i = 0; i < layers.size(); ++i) o.push_back((int)i);
        return o;
    }
    for (int i : order) {
        if (i < 0 || i >= (int)layers.size())
            fail(IMP_ERROR_INVALID_MODEL, "run order names layer " + std::to_string(i) + ", but the plan has " +
                                              std::to_string(layers.size()) + " layers");
        o.push_back(i);
    }
    return o;
}

Json ModelPlan::to_json() const {
    Json j = Json::object();
    j["architecture"] = architecture;
    j["hidden_size"] = hidden_size;
    j["vocab_size"] = vocab_size;
    j["max_positions"] = max_positions;
    j["embedding"] = embedding.to_json();
    Json ls = Json::array();
    for (const auto& l : layers) {
        Json lj = Json::object();
        lj["block"] = l.block;
        lj["block_params"] = l.block_params;
        Json ps = Json::object();
        for (const auto& kv : l.parts) ps[kv.first] = kv.second.to_json();
        lj["parts"] = ps;
        lj["cache_from"] = l.cache_from < 0 ? Json() : Json(l.cache_from);
        ls.push(lj);
    }
    j["layers"] = ls;
    j["final_norm"] = final_norm.to_json();
    j["head"] = head.to_json();
    j["order"] = has_order ? Json::array_of(order) : Json();
    j["ignored_tensors"] = Json::array_of(ignored_tensors);
    return j;
}

ModelPlan ModelPlan::from_json(const Json& j) {
    if (!j.is_object()) fail(IMP_ERROR_INVALID_MODEL, "plan: must be a JSON object");
    ModelPlan p;
    try {
        p.architecture = j.get_string("architecture", "");
        p.hidden_size = j.at("hidden_size").as_int();
        p.vocab_size = j.at("vocab_size").as_int();
        p.max_positions = j.get_int("max_positions", 4096);
        p.embedding = PartSpec::from_json(j.at("embedding"), "embedding");
        p.final_norm = PartSpec::from_json(j.at("final_norm"), "final_norm");
        p.head = PartSpec::from_json(j.at("head"), "head");
        int li = 0;
        for (const auto& lj : j.at("layers").items()) {
            LayerSpec l;
            const std::string where = "layers[" + std::to_string(li++) + "]";
            l.block = lj.get_string("block", "prenorm");
            if (const Json* bp = lj.find("block_params"))
                if (bp->is_object()) l.block_params = *bp;
            const Json& ps = lj.at("parts");
            if (!ps.is_object()) fail(IMP_ERROR_INVALID_MODEL, "plan: " + where + ".parts must be an object");
            for (const auto& m : ps.members())
                l.parts.emplace_back(m.first, PartSpec::from_json(m.second, where + ".parts." + m.first));
            const Json* cf = lj.find("cache_from");
            l.cache_from = (cf && !cf->is_null()) ? (int)cf->as_int() : -1;
            p.layers.push_back(std::move(l));
        }
        const Json* o = j.find("order");
        if (o && o->is_array()) {
            p.has_order = true;
            for (const auto& i : o->items()) p.order.push_back((int)i.as_int());
        }
        if (const Json* ig = j.find("ignored_tensors"))
            if (ig->is_array())
                for (const auto& n : ig->items()) p.ignored_tensors.push_back(n.as_string());
    } catch (const Error&) {
        throw;
    } catch (const std::exception& e) {
        fail(IMP_ERROR_INVALID_MODEL, std::string("plan: ") + e.what());
    }
    if (p.hidden_size <= 0 || p.vocab_size <= 0) fail(IMP_ERROR_INVALID_MODEL, "plan: hidden_size and vocab_size must be positive");
    p.run_order();
    return p;
}

static void collect(std::vector<std::pair<std::string, TensorSpec>>& out, const std::string& category, const PartSpec& spec) {
    const PartClass& cls = part_class(category, spec.kind);
    if (!cls.tensor_specs) return;
    for (const auto& kv : cls.tensor_specs(spec.params)) {
        const std::string* name = nullptr;
        for (const auto& t : spec.tensors)
            if (t.first == kv.first) name = &t.second;
        if (!name) {
            if (kv.second.optional) continue;
            fail(IMP_ERROR_INVALID_MODEL, "plan error: part '" + spec.kind + "' needs a checkpoint name for its tensor '" + kv.first + "'");
        }
        bool seen = false;
        for (auto& e : out)
            if (e.first == *name) {
                if (e.second.shape != kv.second.shape)
                    fail(IMP_ERROR_INVALID_MODEL, "plan error: tensor '" + *name + "' is used with two different shapes");
                seen = true;
            }
        if (!seen) out.emplace_back(*name, kv.second);
    }
}

std::vector<std::pair<std::string, TensorSpec>> ModelPlan::expected_tensors() const {
    ensure_builtin_parts();
    std::vector<std::pair<std::string, TensorSpec>> out;
    collect(out, "embedding", embedding);
    int li = 0;
    for (const auto& l : layers) {
        const PartClass& bc = part_class("block", l.block);
        if (!bc.part_slots) fail(IMP_ERROR_INVALID_MODEL, "block kind '" + l.block + "' declares no part slots");
        const auto slots = bc.part_slots(l.block_params);
        for (const auto& s : slots) {
            const PartSpec* ps = l.part(s.name);
            if (!ps)
                fail(IMP_ERROR_INVALID_MODEL, "plan error: layer " + std::to_string(li) + ": block '" + l.block +
                                                  "' needs a part in its slot '" + s.name + "'");
            collect(out, s.category, *ps);
        }
        for (const auto& kv : l.parts) {
            bool known = false;
            for (const auto& s : slots) known = known || s.name == kv.first;
            if (!known)
                fail(IMP_ERROR_INVALID_MODEL, "plan error: layer " + std::to_string(li) + ": block '" + l.block +
                                                  "' has no slot '" + kv.first + "'");
        }
        ++li;
    }
    collect(out, "norm", final_norm);
    collect(out, "head", head);
    return out;
}

}  // namespace imp
