// The built-in part kinds: RMSNorm, rotary positions, grouped-query attention over the paged cache,
// SwiGLU feed-forward, the pre-norm block, token embedding and the linear output head.  Formulas
// follow the reference's Qwen3 forward pass (src/graph/executor_forward.cu:252-820 attention,
// :826-1179 feed-forward, :2701-3140 the whole step); each class cites the lines it restates.
#include <cmath>
#include <mutex>

#include "ops.hpp"
#include "parts.hpp"

namespace imp {

namespace {

int64_t need_int(const Json& p, const char* key, const char* part) {
    const Json* v = p.find(key);
    if (!v || !v->is_number()) fail(IMP_ERROR_INVALID_MODEL, std::string(part) + ": parameter '" + key + "' is missing");
    return v->as_int();
}

// --------------------------------------------------------------------------------------- norm
// y = x * rsqrt(mean(x^2) + eps) * (w + weight_offset), statistics in 32-bit
// (src/compute/layernorm.cu:50-82).  params: size, eps, weight_offset (default 0).
struct RMSNorm : Norm {
    Tensor weight;
    float eps, offset;
    explicit RMSNorm(BuildArgs& a)
        : weight(a.tensor("weight")), eps((float)a.params.get_double("eps", 1e-6)),
          offset((float)a.params.get_double("weight_offset", 0.0)) {}
    bool takes_split_sum() const override { return true; }
    Tensor add_norm(Step& st, Tensor h, const Branch& branch, const int32_t* rows_idx, int n_rows) override {
        const int64_t n = rows_idx ? n_rows : rows(h);
        Tensor out = st.rt->empty(n, cols(h), -1, /*step=*/rows_idx != nullptr);
        if (st.rt->without('n') && !rows_idx) return out;
        add_rmsnorm(*st.rt, h, branch, weight, out, eps, offset, rows_idx, n_rows);
        return out;
    }
};

// ----------------------------------------------------------------------------------- position
// Rotary encoding over pairs (i, i + rot/2) with angle pos * theta^(-2i/rot) (src/compute/rope.cu:84-101).
// The cos/sin table is made in double precision on the host, once.
// params: head_dim, theta, max_positions, rotary_dim (default head_dim).
struct RotaryPosition : Position {
    DeviceBuffer cos_, sin_;
    int rot, max_pos;
    explicit RotaryPosition(BuildArgs& a) {
        const int head_dim = (int)need_int(a.params, "head_dim", "rotary");
        rot = (int)a.params.get_int("rotary_dim", head_dim);
        if (rot <= 0) rot = head_dim;
        if (rot % 2 || rot > head_dim)
            fail(IMP_ERROR_INVALID_MODEL, "rotary_dim " + std::to_string(rot) + " must be even and within head_dim " + std::to_string(head_dim));
        const double theta = a.params.get_double("theta", 10000.0);
        max_pos = (int)need_int(a.params, "max_positions", "rotary");
        const int half = rot / 2;
        std::vector<float> c((size_t)max_pos * half), s((size_t)max_pos * half);
        std::vector<double> inv((size_t)half);
        for (int i = 0; i < half; ++i) inv[(size_t)i] = std::pow(theta, -2.0 * i / rot);
        for (int p = 0; p < max_pos; ++p)
            for (int i = 0; i < half; ++i) {
                const double ang = (double)p * inv[(size_t)i];
                c[(size_t)p * half + i] = (float)std::cos(ang);
                s[(size_t)p * half + i] = (float)std::sin(ang);
            }
        cos_ = DeviceBuffer(c.size() * 4);
        sin_ = DeviceBuffer(s.size() * 4);
        IMP_CUDA(cudaMemcpy(cos_.data(), c.data(), c.size() * 4, cudaMemcpyHostToDevice));
        IMP_CUDA(cudaMemcpy(sin_.data(), s.data(), s.size() * 4, cudaMemcpyHostToDevice));
    }
    bool rotary(Rotary* out) const override {
        out->cos = (const float*)cos_.data();
        out->sin = (const float*)sin_.data();
        out->rot_dim = rot;
        out->max_pos = max_pos;
        return true;
    }
};

// -------------------------------------------------------------------------------------- mixer
// Grouped-query softmax attention over the paged cache.
//
// q,k,v = x Wq^T, x Wk^T, x Wv^T without bias (src/graph/executor_forward.cu:429-470); optional
// per-head RMSNorm on q and k with one [head_dim] weight each, before the position encoding
// (:536-546); keys and values go to the pages first, then every new token attends to its sequence's
// cached positions up to its own, within `window` if set; scale 1/sqrt(head_dim) (:566);
// out = attn Wo^T (:773-777).
//
// params: hidden_size, num_heads, num_kv_heads, head_dim, window (0 = all), qk_norm (bool),
//         qk_norm_eps, position ({"kind", "params"} or null), scale (optional).
struct GQAAttention : Mixer {
    AttentionGeometry g;
    Tensor w_qkv, w_o;
    bool has_norm = false;
    Tensor q_norm, k_norm, q_norm_f32, k_norm_f32;
    float norm_eps;
    Position* position = nullptr;

    static TensorSpecs specs(const Json& p) {
        const int64_t d = need_int(p, "hidden_size", "gqa_attention"), hq = need_int(p, "num_heads", "gqa_attention"),
                      hkv = need_int(p, "num_kv_heads", "gqa_attention"), dh = need_int(p, "head_dim", "gqa_attention");
        TensorSpecs s;
        s.emplace_back("q_proj", TensorSpec{{hq * dh, d}});
        s.emplace_back("k_proj", TensorSpec{{hkv * dh, d}});
        s.emplace_back("v_proj", TensorSpec{{hkv * dh, d}});
        s.emplace_back("o_proj", TensorSpec{{d, hq * dh}});
        if (p.get_bool("qk_norm", false)) {
            s.emplace_back("q_norm", TensorSpec{{dh}, "norm", "one_plus_normal"});
            s.emplace_back("k_norm", TensorSpec{{dh}, "norm", "one_plus_normal"});
        }
        return s;
    }
    static CacheSpec cache(const Json& p) {
        return CacheSpec::paged((int)need_int(p, "num_kv_heads", "gqa_attention"), (int)need_int(p, "head_dim", "gqa_attention"),
                                (int)p.get_int("window", 0));
    }

    explicit GQAAttention(BuildArgs& a) {
        const Json& p = a.params;
        g.hq = (int)need_int(p, "num_heads", "gqa_attention");
        g.hkv = (int)need_int(p, "num_kv_heads", "gqa_attention");
        g.dh = (int)need_int(p, "head_dim", "gqa_attention");
        if (g.hkv <= 0 || g.hq % g.hkv)
            fail(IMP_ERROR_INVALID_MODEL, std::to_string(g.hq) + " query heads are not a multiple of " + std::to_string(g.hkv) + " kv heads");
        if (g.dh % 16 || g.dh <= 0 || g.dh > 256)
            fail(IMP_ERROR_INVALID_MODEL, "head_dim " + std::to_string(g.dh) + " must be a multiple of 16 in (0, 256]");
        g.window = (int)p.get_int("window", 0);
        const double scale = p.get_double("scale", 0.0);
        g.scale = scale > 0 ? (float)scale : (float)(1.0 / std::sqrt((double)g.dh));
        Runtime& rt = *a.rt;
        w_qkv = cat_rows(rt, *a.store, {a.tensor("q_proj"), a.tensor("k_proj"), a.tensor("v_proj")});
        w_o = a.tensor("o_proj");
        norm_eps = (float)p.get_double("qk_norm_eps", 1e-6);
        if (p.get_bool("qk_norm", false)) {
            has_norm = true;
            q_norm = a.tensor("q_norm");
            k_norm = a.tensor("k_norm");
            // 32-bit copies of the two small weight vectors for the fused kernels
            q_norm_f32 = to_float32(rt, *a.store, q_norm);
            k_norm_f32 = to_float32(rt, *a.store, k_norm);
            if (q_norm.dtype != k_norm.dtype) {
                q_norm = q_norm_f32;
                k_norm = k_norm_f32;
            }
        }
        if (const Json* pos = p.find("position"))
            if (pos->is_object()) position = part_cast<Position>(a.factory->shared("position", *pos), "a position encoding");
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        // the separate q/k/v matrices are not kept
        a.drop("q_proj");
        a.drop("k_proj");
        a.drop("v_proj");
    }

    std::vector<TilingSpec> tilings() const override { return attention_tilings(); }

    Branch forward(Step& st, Tensor x, LayerCache* cache) override {
        Runtime& rt = *st.rt;
        if (!cache || !cache->paged()) fail(IMP_ERROR_INTERNAL, "gqa_attention runs against a paged cache");
        const int64_t T = rows(x);
        const int64_t qd = (int64_t)g.hq * g.dh, kd = (int64_t)g.hkv * g.dh;
        Position::Rotary rot{};
        const bool rotary = position && position->rotary(&rot);
        const bool writes = cache->view.writes != 0;
        const QkNorm qk{has_norm ? (const float*)q_norm_f32.data : nullptr, has_norm ? (const float*)k_norm_f32.data : nullptr, norm_eps};
        const bool fusable = rotary && writes && !rt.is_f32() && rot.rot_dim == g.dh;
        if (fusable) {
            // long portions: projection, norm, rotation and cache write in one kernel
            Tensor q = rt.empty(T, qd);
            if (linear_qkv_rope(st, q, x, w_qkv, g, *cache, qk, rot)) {
                Tensor attn = rt.empty(T, qd);
                paged_attention(st, attn, q, g, *cache, tiling_ids);
                return linear(rt, rt.empty(T, rows(w_o)), attn, w_o, defer_out);
            }
        }
        Tensor qkv = rt.empty(T, qd + 2 * kd);
        if (!rt.without('q')) linear(rt, qkv, x, w_qkv);
        if (fusable && st.decode_only()) {
            // decode steps: the attention kernel normalises and rotates q and the new key itself and writes the new
            // key and value into their pages (no rotary kernel)
            Tensor attn = rt.empty(T, qd);
            if (rt.without('a') || decode_attention_fused(st, attn, qkv, g, *cache, qk, rot)) {
                if (rt.without('o')) return Branch::of(rt.empty(T, rows(w_o)));
                return linear(rt, rt.empty(T, rows(w_o)), attn, w_o, defer_out);
            }
        }
        if (position && !rotary) {
            // An encoding the fused kernel does not know: norm, then let the part rewrite q and k, then a plain write.
            if (has_norm) qk_norm_rope_kv_write(st, qkv, g, &q_norm, &k_norm, norm_eps, nullptr, nullptr);
            Tensor q3 = tensor_nd(qkv.data, qkv.dtype, {T, g.hq, g.dh});
            q3.stride0 = qkv.stride0;
            Tensor k3 = tensor_nd((char*)qkv.data + (size_t)qd * elem_size(qkv.dtype), qkv.dtype, {T, g.hkv, g.dh});
            k3.stride0 = qkv.stride0;
            position->apply(st, q3, k3);
            qk_norm_rope_kv_write(st, qkv, g, nullptr, nullptr, norm_eps, nullptr, writes ? cache : nullptr);
        } else {
            qk_norm_rope_kv_write(st, qkv, g, has_norm ? &q_norm : nullptr, has_norm ? &k_norm : nullptr, norm_eps,
                                  rotary ? &rot : nullptr, writes ? cache : nullptr);
        }
        Tensor attn = rt.empty(T, qd);
        paged_attention(st, attn, col_slice(qkv, 0, qd), g, *cache, tiling_ids);
        return linear(rt, rt.empty(T, rows(w_o)), attn, w_o, defer_out);
    }
};

// ------------------------------------------------------------------------------- feed-forward
// down( silu(x Wg^T) * (x Wu^T) ), activation in 32-bit (src/graph/executor_forward.cu:933-951,
// 1124-1140; src/compute/activation.cu:67-87).  params: hidden_size, intermediate_size.
struct SwiGLU : FeedForward {
    int64_t f;
    bool interleaved;
    Tensor w_gu, w_down;
    static TensorSpecs specs(const Json& p) {
        const int64_t d = need_int(p, "hidden_size", "swiglu"), f = need_int(p, "intermediate_size", "swiglu");
        TensorSpecs s;
        s.emplace_back("gate_proj", TensorSpec{{f, d}});
        s.emplace_back("up_proj", TensorSpec{{f, d}});
        s.emplace_back("down_proj", TensorSpec{{d, f}});
        return s;
    }
    explicit SwiGLU(BuildArgs& a) {
        f = need_int(a.params, "intermediate_size", "swiglu");
        Runtime& rt = *a.rt;
        Tensor gate = a.tensor("gate_proj"), up = a.tensor("up_proj");
        // Gate and up rows alternate in runs of 8 so that one kernel can produce the activation from the fused
        // product; a width that is no multiple of 8 keeps the two halves apart.
        interleaved = f % SWIGLU_INTERLEAVE == 0 && gate.dtype == up.dtype;
        w_gu = interleaved ? interleave_gate_up(rt, *a.store, gate, up) : cat_rows(rt, *a.store, {gate, up});
        w_down = a.tensor("down_proj");
        IMP_CUDA(cudaStreamSynchronize(rt.stream));
        a.drop("gate_proj");
        a.drop("up_proj");
    }
    Branch forward(Step& st, Tensor x) override {
        Runtime& rt = *st.rt;
        const int64_t T = rows(x);
        Tensor act = rt.empty(T, f);
        if (interleaved) {
            if (!rt.without('g')) linear_swiglu(rt, act, x, w_gu);
        } else {
            Tensor gu = rt.empty(T, 2 * f);
            linear(rt, gu, x, w_gu);
            swiglu(rt, act, gu, 0);
        }
        if (rt.without('d')) return Branch::of(rt.empty(T, rows(w_down)));
        return linear(rt, rt.empty(T, rows(w_down)), act, w_down, defer_out);
    }
};

// -------------------------------------------------------------------------------------- block
// h += mixer(norm1(h)); h += ffn(norm2(h))  (pre-norm, src/model/model.h:66).  The second sum is handed
// on as `pending` and added by whoever normalises the stream next (the next block's first norm, or the
// final norm), in the same kernel.  Slots: mixer_norm, mixer, ffn_norm, feed_forward.
struct PreNormBlock : Block {
    Mixer* mixer_;
    FeedForward* ffn;
    Norm *norm1, *norm2;
    explicit PreNormBlock(BuildArgs& a)
        : mixer_(part_cast<Mixer>(a.part("mixer"), "a mixer")), ffn(part_cast<FeedForward>(a.part("feed_forward"), "a feed-forward")),
          norm1(part_cast<Norm>(a.part("mixer_norm"), "a norm")), norm2(part_cast<Norm>(a.part("ffn_norm"), "a norm")) {
        // the mixer's output goes to this block's second norm and nowhere else
        if (norm2->takes_split_sum()) mixer_->defer_out = true;
    }
    static std::vector<Slot> slots(const Json&) {
        return {{"mixer_norm", "norm"}, {"mixer", "mixer"}, {"ffn_norm", "norm"}, {"feed_forward", "feed_forward"}};
    }
    bool takes_split_sum() const override { return norm1->takes_split_sum(); }
    Mixer* mixer() const override { return mixer_; }
    std::vector<Part*> parts() const override { return {norm1, mixer_, norm2, ffn}; }
    bool graph_safe() const override { return norm1->graph_safe() && mixer_->graph_safe() && norm2->graph_safe() && ffn->graph_safe(); }
    Branch forward(Step& st, Tensor h, const Branch& pending, LayerCache* cache) override {
        Tensor x = norm1->add_norm(st, h, pending);
        Branch a = mixer_->forward(st, x, cache);
        stage(st, "mixer", a);                  // time since the stage before: first norm and mixer
        x = norm2->add_norm(st, h, a);
        ffn->defer_out = defer_pending;
        Branch f = ffn->forward(st, x);
        stage(st, "feed_forward", f);           // second norm and feed-forward
        return f;
    }
};

// ---------------------------------------------------------------------------- embedding, head
// h[t] = E[id[t]] * scale into the 32-bit stream (src/graph/executor_forward.cu:2786-2797).
// params: vocab_size, hidden_size, scale (default 1).
struct TokenEmbedding : Embedding {
    Tensor weight;
    float scale;
    explicit TokenEmbedding(BuildArgs& a) : weight(a.tensor("weight")), scale((float)a.params.get_double("scale", 1.0)) {}
    static TensorSpecs specs(const Json& p) {
        TensorSpecs s;
        s.emplace_back("weight", TensorSpec{{need_int(p, "vocab_size", "token_embedding"), need_int(p, "hidden_size", "token_embedding")}});
        return s;
    }
    Tensor forward(Step& st) override {
        Tensor out = st.rt->empty(st.T(), cols(weight), F32, /*step=*/true);
        embedding(*st.rt, out, weight, st.view.token_ids, st.T(), scale);
        return out;
    }
};

// logits = x W^T in 32-bit (src/graph/executor_forward.cu:2953, 3075).  params: vocab_size, hidden_size.
// The weight may be the embedding's own tensor.
struct LinearHead : Head {
    Tensor weight;
    explicit LinearHead(BuildArgs& a) : weight(a.tensor("weight")) {}
    static TensorSpecs specs(const Json& p) {
        TensorSpecs s;
        s.emplace_back("weight", TensorSpec{{need_int(p, "vocab_size", "linear_head"), need_int(p, "hidden_size", "linear_head")}});
        return s;
    }
    Tensor forward(Step& st, Tensor x) override {
        Tensor out = st.rt->empty(rows(x), rows(weight), F32, /*step=*/true);
        linear(*st.rt, out, x, weight);
        return out;
    }
};

template <typename T> PartClass simple_class(TensorSpecs (*specs)(const Json&)) {
    PartClass c;
    if (specs) c.tensor_specs = specs;
    c.create = [](BuildArgs& a) -> Part* { return new T(a); };
    return c;
}

}  // namespace

void ensure_builtin_parts() {
    static std::once_flag once;
    std::call_once(once, [] {
        PartClass norm = simple_class<RMSNorm>(nullptr);
        norm.tensor_specs = [](const Json& p) {
            TensorSpecs s;
            s.emplace_back("weight", TensorSpec{{need_int(p, "size", "rmsnorm")}, "norm", "one_plus_normal"});
            return s;
        };
        register_part_class("norm", "rmsnorm", norm, true);
        register_part_class("position", "rotary", simple_class<RotaryPosition>(nullptr), true);
        PartClass attn = simple_class<GQAAttention>(&GQAAttention::specs);
        attn.cache_spec = &GQAAttention::cache;
        register_part_class("mixer", "gqa_attention", attn, true);
        register_part_class("feed_forward", "swiglu", simple_class<SwiGLU>(&SwiGLU::specs), true);
        PartClass block = simple_class<PreNormBlock>(nullptr);
        block.part_slots = &PreNormBlock::slots;
        register_part_class("block", "prenorm", block, true);
        register_part_class("embedding", "token_embedding", simple_class<TokenEmbedding>(&TokenEmbedding::specs), true);
        register_part_class("head", "linear_head", simple_class<LinearHead>(&LinearHead::specs), true);
    });
}

}  // namespace imp
