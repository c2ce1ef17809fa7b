// Part kinds implemented outside the library: a table of C functions stands behind each of the
// part interfaces.  Such parts never see unsummed branches, and a model that holds one does not
// capture CUDA graphs (their launches may depend on more than the batch's sizes).
#include <cstring>

#include "ops.hpp"
#include "parts.hpp"

namespace imp {

static thread_local std::string g_part_error;
void set_part_error(const char* m) { g_part_error = m ? m : ""; }

namespace {

struct Foreign {
    ImpPartVTable vt{};
    void* self = nullptr;
    std::string category, kind;
    ~Foreign() {
        if (self && vt.destroy) vt.destroy(self);
    }
    void run(ImpCall& c) const {
        g_part_error.clear();
        const int rc = vt.forward ? vt.forward(self, &c) : -1;
        if (rc != 0)
            fail(IMP_ERROR_INTERNAL, category + " '" + kind + "' failed" + (g_part_error.empty() ? std::string() : ": " + g_part_error));
    }
};

void create_foreign(Foreign& f, const ImpPartVTable& vt, BuildArgs& a) {
    f.vt = vt;
    f.category = a.category;
    f.kind = a.kind;
    std::vector<const char*> names, part_names;
    std::vector<ImpTensor> tensors;
    std::vector<ImpPart> parts;
    for (const auto& kv : a.tensors) {
        names.push_back(kv.first.c_str());
        tensors.push_back(kv.second);
    }
    for (const auto& kv : a.parts) {
        part_names.push_back(kv.first.c_str());
        parts.push_back((ImpPart)kv.second);
    }
    const std::string params = a.params.dump();
    g_part_error.clear();
    if (!vt.create) fail(IMP_ERROR_INVALID_ARG, a.category + " '" + a.kind + "' has no create function");
    f.self = vt.create(vt.user, params.c_str(), (int)names.size(), names.data(), tensors.data(), (int)parts.size(),
                       part_names.data(), parts.data(), a.rt->dtype, a.rt->device);
    if (!f.self)
        fail(IMP_ERROR_INVALID_MODEL, a.category + " '" + a.kind + "' could not be built" + (g_part_error.empty() ? std::string() : ": " + g_part_error));
}

ImpCall base_call(Step& st, const LayerCache* cache) {
    ImpCall c{};
    c.batch = &st.view;
    c.cache = cache ? &cache->view : nullptr;
    return c;
}

struct ForeignNorm : Norm, Foreign {
    bool graph_safe() const override { return false; }
    Tensor add_norm(Step& st, Tensor h, const Branch& branch, const int32_t* rows_idx, int n_rows) override {
        ImpCall c = base_call(st, nullptr);
        c.h = h;
        if (!branch.empty()) c.branch = summed(st, branch);
        c.rows = rows_idx;
        c.n_rows = rows_idx ? n_rows : 0;
        c.out = st.rt->empty(rows_idx ? n_rows : rows(h), cols(h), -1, rows_idx != nullptr);
        run(c);
        return c.out;
    }
};

struct ForeignPosition : Position, Foreign {
    bool graph_safe() const override { return false; }
    void apply(Step& st, Tensor q, Tensor k) override {
        ImpCall c = base_call(st, nullptr);
        c.q = q;
        c.k = k;
        run(c);
    }
};

struct ForeignMixer : Mixer, Foreign {
    bool graph_safe() const override { return false; }
    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        ImpCall c = base_call(st, cache);
        c.x = x;
        c.out = st.rt->empty(rows(x), cols(x));
        run(c);
        return Branch::of(c.out);
    }
};

struct ForeignFeedForward : FeedForward, Foreign {
    bool graph_safe() const override { return false; }
    Branch forward(Step& st, Tensor x) override {
        ImpCall c = base_call(st, nullptr);
        c.x = x;
        c.out = st.rt->empty(rows(x), cols(x));
        run(c);
        return Branch::of(c.out);
    }
};

struct ForeignBlock : Block, Foreign {
    std::vector<Part*> parts_;
    Mixer* mixer_ = nullptr;
    bool graph_safe() const override { return false; }
    Mixer* mixer() const override { return mixer_; }
    std::vector<Part*> parts() const override { return parts_; }
    Branch forward(Step& st, Tensor h, const Branch& pending, LayerCache* cache) override {
        ImpCall c = base_call(st, cache);
        c.h = h;
        if (!pending.empty()) c.branch = summed(st, pending);
        c.out = st.rt->empty(rows(h), cols(h));
        c.has_out = 1;
        run(c);
        return c.has_out ? Branch::of(c.out) : Branch();
    }
};

struct ForeignEmbedding : Embedding, Foreign {
    int64_t hidden = 0;
    bool graph_safe() const override { return false; }
    Tensor forward(Step& st) override {
        ImpCall c = base_call(st, nullptr);
        c.h = st.rt->empty(st.T(), hidden, F32, true);
        run(c);
        return c.h;
    }
};

struct ForeignHead : Head, Foreign {
    int64_t vocab = 0;
    bool graph_safe() const override { return false; }
    Tensor forward(Step& st, Tensor x) override {
        ImpCall c = base_call(st, nullptr);
        c.x = x;
        c.out = st.rt->empty(rows(x), vocab, F32, true);
        run(c);
        return c.out;
    }
};

std::string call_string(const char* (*fn)(void*, const char*), void* user, const Json& params, const std::string& what) {
    g_part_error.clear();
    const std::string p = params.dump();
    const char* r = fn(user, p.c_str());
    if (!r) fail(IMP_ERROR_INVALID_MODEL, what + " failed" + (g_part_error.empty() ? std::string() : ": " + g_part_error));
    return r;
}

}  // namespace

void register_foreign_part(const std::string& category, const std::string& kind, const ImpPartVTable& vt) {
    PartClass cls;
    const std::string label = category + " '" + kind + "'";
    if (vt.tensor_specs)
        cls.tensor_specs = [vt, label](const Json& p) {
            return tensor_specs_from_json(Json::parse(call_string(vt.tensor_specs, vt.user, p, label + ": tensor_specs"), label));
        };
    if (vt.cache_spec)
        cls.cache_spec = [vt, label](const Json& p) {
            return CacheSpec::from_json(Json::parse(call_string(vt.cache_spec, vt.user, p, label + ": cache_spec"), label));
        };
    if (vt.part_slots)
        cls.part_slots = [vt, label](const Json& p) {
            std::vector<Slot> out;
            int mixers = 0;
            const Json list = Json::parse(call_string(vt.part_slots, vt.user, p, label + ": part_slots"), label);
            for (const auto& s : list.items()) {
                out.push_back(Slot{s.at("name").as_string(), s.at("category").as_string()});
                mixers += out.back().category == "mixer";
            }
            if (mixers > 1) fail(IMP_ERROR_UNSUPPORTED, label + ": a block holds at most one mixer (one cache per layer)");
            return out;
        };
    cls.create = [vt, category](BuildArgs& a) -> Part* {
        if (category == "norm") { auto* p = new ForeignNorm; std::unique_ptr<ForeignNorm> g(p); create_foreign(*p, vt, a); return g.release(); }
        if (category == "position") { auto* p = new ForeignPosition; std::unique_ptr<ForeignPosition> g(p); create_foreign(*p, vt, a); return g.release(); }
        if (category == "mixer") { auto* p = new ForeignMixer; std::unique_ptr<ForeignMixer> g(p); create_foreign(*p, vt, a); return g.release(); }
        if (category == "feed_forward") { auto* p = new ForeignFeedForward; std::unique_ptr<ForeignFeedForward> g(p); create_foreign(*p, vt, a); return g.release(); }
        if (category == "block") {
            auto* p = new ForeignBlock;
            std::unique_ptr<ForeignBlock> g(p);
            for (const auto& kv : a.parts) {
                p->parts_.push_back(kv.second);
                if (auto* m = dynamic_cast<Mixer*>(kv.second)) p->mixer_ = m;
            }
            create_foreign(*p, vt, a);
            return g.release();
        }
        if (category == "embedding") {
            auto* p = new ForeignEmbedding;
            std::unique_ptr<ForeignEmbedding> g(p);
            p->hidden = a.params.get_int("hidden_size", 0);
            if (p->hidden <= 0) fail(IMP_ERROR_INVALID_MODEL, "an embedding needs the parameter 'hidden_size'");
            create_foreign(*p, vt, a);
            return g.release();
        }
        if (category == "head") {
            auto* p = new ForeignHead;
            std::unique_ptr<ForeignHead> g(p);
            p->vocab = a.params.get_int("vocab_size", 0);
            if (p->vocab <= 0) fail(IMP_ERROR_INVALID_MODEL, "a head needs the parameter 'vocab_size'");
            create_foreign(*p, vt, a);
            return g.release();
        }
        fail(IMP_ERROR_INVALID_ARG, "unknown part category '" + category + "'");
    };
    register_part_class(category, kind, cls, false);
}

}  // namespace imp
