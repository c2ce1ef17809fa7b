#include "sampler.hpp"

#include <algorithm>
#include <cmath>

#include "kernels.h"

namespace imp {

std::map<int32_t, float> dry_penalties(const std::vector<int32_t>& t, float multiplier, float base, int allowed_length, int last_n) {
    std::map<int32_t, float> out;
    const int n = (int)t.size();
    if (multiplier <= 0.f || n < 2) return out;
    const int start = last_n > 0 ? std::max(0, n - last_n) : 0;
    std::map<int32_t, int> best;
    // only positions preceded by the sequence's last token can match at all
    for (int pos = start + 1; pos < n; ++pos) {
        if (t[(size_t)pos - 1] != t[(size_t)n - 1]) continue;
        int a = pos - 1, b = n - 1, m = 0;
        while (a >= start && t[(size_t)a] == t[(size_t)b]) {
            ++m;
            --a;
            --b;
        }
        if (m > allowed_length) {
            int& cur = best[t[(size_t)pos]];
            cur = std::max(cur, m);
        }
    }
    for (const auto& kv : best) out[kv.first] = multiplier * (float)std::pow((double)base, (double)(kv.second - allowed_length));
    return out;
}

Sampler::Sampler(int64_t vocab_size, int max_rows, Runtime* rt) : V_(vocab_size), max_rows_(max_rows), rt_(rt) {
    for (auto& o : out_) o = DeviceBuffer((size_t)max_rows * 4, true);
    argmax_scratch_ = DeviceBuffer((size_t)imp_argmax_scratch_words(max_rows) * 4);
}

template <typename T> T* Sampler::upload(const std::vector<T>& host) {
    if (host.empty()) return nullptr;
    T* d = (T*)rt_->arena->alloc_step(host.size() * sizeof(T));
    IMP_CUDA(cudaMemcpyAsync(d, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice, rt_->stream));
    return d;
}

void Sampler::penalties(Tensor logits, const std::vector<Request*>& rows_) {
    const int R = (int)rows_.size();
    std::vector<int32_t> flat, start{0};
    std::vector<float> rep, freq, pres;
    int max_hist = 0;
    for (Request* r : rows_) {
        const SamplingParams& p = r->params;
        std::vector<int32_t> h;
        if (p.has_penalties()) {
            h = r->all_tokens();
            if (p.repeat_last_n > 0 && (int)h.size() > p.repeat_last_n) h.erase(h.begin(), h.end() - p.repeat_last_n);
        }
        flat.insert(flat.end(), h.begin(), h.end());
        start.push_back((int32_t)flat.size());
        max_hist = std::max(max_hist, (int)h.size());
        rep.push_back(p.repetition_penalty);
        freq.push_back(p.frequency_penalty);
        pres.push_back(p.presence_penalty);
    }
    if (max_hist == 0) return;
    if (!counts_.data()) counts_ = DeviceBuffer((size_t)max_rows_ * (size_t)V_ * 4);
    ++rt_->launches;
    check_launch(imp_apply_penalties((float*)logits.data, logits.stride0, R, (int)V_, upload(flat), upload(start), max_hist, upload(rep),
                                     upload(freq), upload(pres), (int*)counts_.data(), rt_->stream),
                 "apply_penalties");
}

void Sampler::dry(Tensor logits, const std::vector<Request*>& rows_) {
    std::vector<int32_t> rows, toks;
    std::vector<float> vals;
    for (size_t r = 0; r < rows_.size(); ++r) {
        const SamplingParams& p = rows_[r]->params;
        if (!p.has_dry()) continue;
        for (const auto& kv : dry_penalties(rows_[r]->all_tokens(), p.dry_multiplier, p.dry_base, p.dry_allowed_length, p.dry_penalty_last_n))
            if (kv.first >= 0 && kv.first < V_) {
                rows.push_back((int32_t)r);
                toks.push_back(kv.first);
                vals.push_back(kv.second);
            }
    }
    if (rows.empty()) return;
    ++rt_->launches;
    check_launch(imp_sparse_subtract((float*)logits.data, logits.stride0, (int)rows_.size(), (int)V_, upload(rows), upload(toks),
                                     upload(vals), (int)rows.size(), rt_->stream),
                 "sparse_subtract");
}

const int32_t* Sampler::sample_device(Tensor logits, const std::vector<Request*>& rows_, const std::vector<int64_t>& steps) {
    const int R = (int)rows_.size();
    if (R == 0) return nullptr;
    if (R > max_rows_) fail(IMP_ERROR_INTERNAL, "more rows to sample than the sampler was made for");
    int32_t* out = (int32_t*)out_[turn_].data();
    turn_ ^= 1;
    bool any_pen = false, any_dry = false, any_typ = false, all_greedy = true, any_miro = false;
    for (Request* r : rows_) {
        any_pen = any_pen || r->params.has_penalties();
        any_dry = any_dry || r->params.has_dry();
        any_typ = any_typ || r->params.has_typical();
        all_greedy = all_greedy && r->params.is_greedy();
        any_miro = any_miro || r->params.mirostat == 2;
    }
    float* lg = (float*)logits.data;
    if (any_pen) penalties(logits, rows_);
    if (any_dry) dry(logits, rows_);
    if (any_typ) {
        std::vector<float> tp, mp;
        for (Request* r : rows_) {
            tp.push_back(r->params.has_typical() ? r->params.typical_p : 1.0f);
            mp.push_back(r->params.min_p);
        }
        ++rt_->launches;
        check_launch(imp_typical_filter(lg, logits.stride0, R, (int)V_, upload(tp), upload(mp), rt_->stream), "typical_filter");
    }
    if (all_greedy) {
        ++rt_->launches;
        check_launch(imp_argmax(lg, logits.stride0, R, (int)V_, out, V_ >= 8192 ? argmax_scratch_.data() : nullptr, rt_->stream), "argmax");
        return out;
    }
    std::vector<float> temp, top_p, min_p, uni, mu, miro_temp;
    std::vector<int32_t> top_k, active;
    for (int r = 0; r < R; ++r) {
        Request* q = rows_[(size_t)r];
        const SamplingParams& p = q->params;
        temp.push_back((p.is_greedy() || p.mirostat == 2) ? 0.f : p.temperature);
        top_p.push_back((p.top_p > 0.f && p.top_p < 1.f) ? p.top_p : 1.f);
        min_p.push_back(p.min_p);
        uni.push_back(uniform_for(q->seed, steps[(size_t)r]));
        top_k.push_back(p.top_k);
        if (p.mirostat == 2 && !q->has_mu) {
            q->has_mu = true;
            q->mirostat_mu = 2.0f * p.mirostat_tau;
        }
        mu.push_back(p.mirostat == 2 ? q->mirostat_mu : 0.f);
        active.push_back(p.mirostat == 2 ? 1 : 0);
        miro_temp.push_back(p.temperature);
    }
    const float* d_uni = upload(uni);
    ++rt_->launches;
    check_launch(imp_sample(lg, logits.stride0, R, (int)V_, upload(temp), upload(top_k), upload(top_p), upload(min_p), d_uni, out, rt_->stream),
                 "sample");
    if (any_miro) {
        float* surprise = (float*)rt_->arena->alloc_step((size_t)R * 4);
        IMP_CUDA(cudaMemsetAsync(surprise, 0, (size_t)R * 4, rt_->stream));
        ++rt_->launches;
        check_launch(imp_sample_mirostat(lg, logits.stride0, R, (int)V_, upload(active), upload(miro_temp), upload(mu), d_uni, out,
                                         surprise, rt_->stream),
                     "sample_mirostat");
        std::vector<float> sur((size_t)R);
        IMP_CUDA(cudaMemcpyAsync(sur.data(), surprise, (size_t)R * 4, cudaMemcpyDeviceToHost, rt_->stream));
        IMP_CUDA(cudaStreamSynchronize(rt_->stream));   // waits for the device: mu is host state
        for (int r = 0; r < R; ++r) {
            Request* q = rows_[(size_t)r];
            if (q->params.mirostat == 2) q->mirostat_mu -= q->params.mirostat_eta * (sur[(size_t)r] - q->params.mirostat_tau);
        }
    }
    return out;
}

}  // namespace imp
