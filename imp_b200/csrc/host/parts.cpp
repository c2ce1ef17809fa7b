#include "parts.hpp"

#include "ops.hpp"

#include <algorithm>
#include <cstring>
#include <mutex>

namespace imp {

const char* const PART_CATEGORIES[7] = {"mixer", "feed_forward", "norm", "position", "block", "embedding", "head"};

// -------------------------------------------------------------------------------- cache spec
std::string CacheSpec::key() const {
    if (kind == None) return "none";
    if (kind == Paged)
        return "paged:" + std::to_string(num_kv_heads) + "x" + std::to_string(head_dim) + "w" + std::to_string(window);
    std::string k = "state";
    for (const auto& s : states) {
        k += ":" + s.name + "/" + dtype_name(s.dtype);
        for (int64_t d : s.shape) k += "," + std::to_string(d);
    }
    return k;
}

Json CacheSpec::to_json() const {
    if (kind == None) return Json();
    Json j = Json::object();
    if (kind == Paged) {
        j["kind"] = "paged";
        j["num_kv_heads"] = num_kv_heads;
        j["head_dim"] = head_dim;
        j["window"] = window;
    } else {
        j["kind"] = "state";
        Json ts = Json::array();
        for (const auto& s : states) {
            Json t = Json::object();
            t["name"] = s.name;
            t["shape"] = Json::array_of(s.shape);
            t["dtype"] = dtype_name(s.dtype);
            ts.push(t);
        }
        j["tensors"] = ts;
    }
    return j;
}

CacheSpec CacheSpec::from_json(const Json& j) {
    CacheSpec s;
    if (j.is_null()) return s;
    const std::string kind = j.get_string("kind", "");
    if (kind == "paged") {
        s.kind = Paged;
        s.num_kv_heads = (int)j.at("num_kv_heads").as_int();
        s.head_dim = (int)j.at("head_dim").as_int();
        s.window = (int)j.get_int("window", 0);
        if (s.num_kv_heads <= 0 || s.head_dim <= 0 || s.window < 0)
            fail(IMP_ERROR_INVALID_ARG, "cache spec: kv heads and head size must be positive, the window not negative");
    } else if (kind == "state") {
        s.kind = State;
        for (const auto& t : j.at("tensors").items()) {
            StateTensorSpec ts;
            ts.name = t.get_string("name", "state" + std::to_string(s.states.size()));
            for (const auto& d : t.at("shape").items()) ts.shape.push_back(d.as_int());
            ts.dtype = dtype_from_name(t.get_string("dtype", "float32"));
            s.states.push_back(ts);
        }
        if (s.states.empty() || s.states.size() > 4)
            fail(IMP_ERROR_INVALID_ARG, "cache spec: a state needs one to four tensors");
    } else {
        fail(IMP_ERROR_INVALID_ARG, "cache spec: kind must be 'paged' or 'state', got '" + kind + "'");
    }
    return s;
}

// ------------------------------------------------------------------------------------ registry
namespace {
std::mutex g_reg_mutex;
std::map<std::string, std::map<std::string, PartClass>>& registry() {
    static std::map<std::string, std::map<std::string, PartClass>> r;
    return r;
}
bool known_category(const std::string& c) {
    for (const char* k : PART_CATEGORIES)
        if (c == k) return true;
    return false;
}
}  // namespace

void register_part_class(const std::string& category, const std::string& kind, PartClass cls, bool replace) {
    if (!known_category(category)) {
        std::string all;
        for (const char* k : PART_CATEGORIES) all += std::string(all.empty() ? "" : ", ") + k;
        fail(IMP_ERROR_INVALID_ARG, "unknown part category '" + category + "'; categories: " + all);
    }
    std::lock_guard<std::mutex> lock(g_reg_mutex);
    auto& m = registry()[category];
    if (m.count(kind) && !replace) fail(IMP_ERROR_INVALID_ARG, category + " kind '" + kind + "' is already registered");
    m[kind] = std::move(cls);
}

void unregister_part_class(const std::string& category, const std::string& kind) {
    std::lock_guard<std::mutex> lock(g_reg_mutex);
    auto it = registry().find(category);
    if (it != registry().end()) it->second.erase(kind);
}

const PartClass& part_class(const std::string& category, const std::string& kind) {
    ensure_builtin_parts();
    std::lock_guard<std::mutex> lock(g_reg_mutex);
    auto& m = registry()[category];
    auto it = m.find(kind);
    if (it == m.end()) {
        std::string known;
        for (const auto& kv : m) known += (known.empty() ? "" : ", ") + kv.first;
        fail(IMP_ERROR_INVALID_MODEL, "unknown " + category + " kind '" + kind + "'; known: " + (known.empty() ? "(none)" : known));
    }
    return it->second;
}

std::vector<std::string> known_parts(const std::string& category) {
    ensure_builtin_parts();
    std::lock_guard<std::mutex> lock(g_reg_mutex);
    std::vector<std::string> out;
    for (const auto& kv : registry()[category]) out.push_back(kv.first);
    return out;
}

// -------------------------------------------------------------------------------- weight store
Tensor WeightStore::alloc(int dtype, const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    DeviceBuffer buf((size_t)std::max<int64_t>(n, 1) * elem_size(dtype));
    Tensor t = tensor_nd(buf.data(), dtype, shape);
    bytes_ += buf.bytes();
    buffers_[buf.data()] = std::move(buf);
    return t;
}

void WeightStore::release(const void* data) {
    auto it = buffers_.find(data);
    if (it == buffers_.end()) return;
    bytes_ -= it->second.bytes();
    buffers_.erase(it);
}

// ---------------------------------------------------------------------------------- build args
bool BuildArgs::has(const std::string& name) const {
    for (const auto& kv : tensors)
        if (kv.first == name) return true;
    return false;
}
Tensor BuildArgs::tensor(const std::string& name) const {
    for (const auto& kv : tensors)
        if (kv.first == name) return kv.second;
    fail(IMP_ERROR_INVALID_MODEL, category + " '" + kind + "' was built without its tensor '" + name + "'");
}
Part* BuildArgs::part(const std::string& slot) const {
    for (const auto& kv : parts)
        if (kv.first == slot) return kv.second;
    return nullptr;
}
void BuildArgs::drop(const std::string& name) {
    for (size_t i = 0; i < tensors.size(); ++i)
        if (tensors[i].first == name) {
            if (store) store->release(tensors[i].second.data);
            tensors.erase(tensors.begin() + (long)i);
            return;
        }
}

// ------------------------------------------------------------------------------------- factory
Part* PartFactory::build(const std::string& category, const PartSpec& spec,
                         std::vector<std::pair<std::string, Tensor>> tensors,
                         std::vector<std::pair<std::string, Part*>> parts) {
    const PartClass& cls = part_class(category, spec.kind);
    BuildArgs args;
    args.category = category;
    args.kind = spec.kind;
    args.params = spec.params;
    args.tensors = std::move(tensors);
    args.parts = std::move(parts);
    args.rt = rt_;
    args.store = store_;
    args.factory = this;
    Part* p = cls.create(args);
    if (!p) fail(IMP_ERROR_INTERNAL, category + " '" + spec.kind + "' could not be built");
    owned_.emplace_back(p);
    return p;
}

Part* PartFactory::shared(const std::string& category, const Json& spec_json) {
    const std::string key = category + ":" + spec_json.dump();
    auto it = shared_.find(key);
    if (it != shared_.end()) return it->second;
    PartSpec spec = PartSpec::from_json(spec_json, category);
    Part* p = build(category, spec, {});
    shared_[key] = p;
    return p;
}

// --------------------------------------------------------------- uniform entry (imp_part_forward)
static Branch branch_of(const ImpTensor& t) {
    Branch b;
    if (t.data) b.t = t;
    return b;
}

static void copy_out(Step& st, const Tensor& produced, ImpTensor& out) {
    // The caller may have brought its own output buffer; otherwise hand the produced tensor back.
    if (out.data && out.data != produced.data) {
        const size_t row_bytes = (size_t)cols(produced) * elem_size(produced.dtype);
        IMP_CUDA(cudaMemcpy2DAsync(out.data, (size_t)out.stride0 * elem_size(out.dtype), produced.data,
                                   (size_t)produced.stride0 * elem_size(produced.dtype), row_bytes, (size_t)rows(produced),
                                   cudaMemcpyDeviceToDevice, st.rt->stream));
    } else {
        out = produced;
    }
}

void Norm::call(Step& st, ImpCall& c) {
    copy_out(st, add_norm(st, c.h, branch_of(c.branch), c.rows, c.rows ? c.n_rows : 0), c.out);
}
void Position::apply(Step&, Tensor, Tensor) { fail(IMP_ERROR_UNSUPPORTED, "this position encoding has no unfused path"); }
void Position::call(Step& st, ImpCall& c) { apply(st, c.q, c.k); }
void Mixer::call(Step& st, ImpCall& c) {
    LayerCache lc;
    if (c.cache) lc.view = *c.cache;
    const bool keep = defer_out;
    defer_out = false;
    Branch b = forward(st, c.x, c.cache ? &lc : nullptr);
    defer_out = keep;
    copy_out(st, summed(st, b), c.out);
}
void FeedForward::call(Step& st, ImpCall& c) {
    const bool keep = defer_out;
    defer_out = false;
    Branch b = forward(st, c.x);
    defer_out = keep;
    copy_out(st, summed(st, b), c.out);
}
void Block::call(Step& st, ImpCall& c) {
    LayerCache lc;
    if (c.cache) lc.view = *c.cache;
    const bool keep = defer_pending;
    defer_pending = false;
    Branch b = forward(st, c.h, branch_of(c.branch), c.cache ? &lc : nullptr);
    defer_pending = keep;
    c.has_out = b.empty() ? 0 : 1;
    if (!b.empty()) copy_out(st, summed(st, b), c.out);
}
void Embedding::call(Step& st, ImpCall& c) { copy_out(st, forward(st), c.h); }
void Head::call(Step& st, ImpCall& c) { copy_out(st, forward(st, c.x), c.out); }

}  // namespace imp
