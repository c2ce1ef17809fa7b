// Runs the reference's own kernels (kekzl/imp, unmodified, compiled from its source tree beside this
// file by make_reference_anchor.py) on tiny inputs and prints inputs and outputs as one JSON object.
// The outputs pin the formulas of the plain implementation under tests/plain on what the reference
// computes: rmsnorm (src/compute/layernorm.cu), rope_forward and qknorm_rope_fused
// (src/compute/rope.cu), swiglu (src/compute/activation.cu), embedding_lookup
// (src/compute/embedding.cu), sample_greedy (src/compute/sampling.cu) and flash_attention_prefill
// (src/compute/attention.cu, half precision only).  Everything here is this repository's code; it
// only calls the reference's public functions.  One launch per case, no loops on the device.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "compute/activation.h"
#include "compute/attention.h"
#include "compute/embedding.h"
#include "compute/layernorm.h"
#include "compute/rope.h"
#include "compute/sampling.h"
#include "core/tensor.h"

using imp::DType;
using imp::Tensor;

#define CK(x)                                                                          \
    do {                                                                               \
        cudaError_t e = (x);                                                           \
        if (e != cudaSuccess) {                                                        \
            fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e));                    \
            exit(2);                                                                   \
        }                                                                              \
    } while (0)

static uint32_t g_state = 12345u;
static float uniform() {   // in [-1, 1)
    g_state = g_state * 1664525u + 1013904223u;
    return (float)(g_state >> 8) / 8388608.0f - 1.0f;
}
static std::vector<float> randoms(size_t n, float scale, float shift = 0.f) {
    std::vector<float> v(n);
    for (auto& x : v) x = shift + scale * uniform();
    return v;
}

template <typename T> struct Dev {
    T* p = nullptr;
    size_t n = 0;
    explicit Dev(const std::vector<T>& h) : n(h.size()) {
        CK(cudaMalloc(&p, n * sizeof(T)));
        CK(cudaMemcpy(p, h.data(), n * sizeof(T), cudaMemcpyHostToDevice));
    }
    explicit Dev(size_t count) : n(count) {
        CK(cudaMalloc(&p, n * sizeof(T)));
        CK(cudaMemset(p, 0, n * sizeof(T)));
    }
    ~Dev() { cudaFree(p); }
    std::vector<T> host() const {
        std::vector<T> h(n);
        CK(cudaDeviceSynchronize());
        CK(cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost));
        return h;
    }
};

static Tensor tensor(void* p, DType dt, std::vector<int64_t> shape) {
    return Tensor(p, dt, (int)shape.size(), shape.data(), true);
}
static std::vector<__half> to_half(const std::vector<float>& v) {
    std::vector<__half> h(v.size());
    for (size_t i = 0; i < v.size(); ++i) h[i] = __float2half(v[i]);
    return h;
}
static std::vector<float> to_float(const std::vector<__half>& v) {
    std::vector<float> f(v.size());
    for (size_t i = 0; i < v.size(); ++i) f[i] = __half2float(v[i]);
    return f;
}

static bool g_first = true;
template <typename T> static void emit(const char* name, const std::vector<T>& v, const char* fmt) {
    printf("%s\"%s\": [", g_first ? "" : ",\n ", name);
    g_first = false;
    for (size_t i = 0; i < v.size(); ++i) {
        if (i) printf(", ");
        printf(fmt, v[i]);
    }
    printf("]");
}
static void emit_f(const char* name, const std::vector<float>& v) { emit(name, v, "%.9g"); }
static void emit_i(const char* name, const std::vector<int>& v) { emit(name, v, "%d"); }

int main() {
    printf("{");
    {   // RMSNorm, float32: two eps values and a weight offset
        const int rows = 5, d = 48;
        auto x = randoms(rows * d, 2.0f), w = randoms(d, 0.3f, 1.0f);
        Dev<float> dx(x), dw(w), dout((size_t)rows * d);
        Tensor tx = tensor(dx.p, DType::FP32, {rows, d}), tw = tensor(dw.p, DType::FP32, {d}), to = tensor(dout.p, DType::FP32, {rows, d});
        emit_f("rmsnorm_x", x);
        emit_f("rmsnorm_w", w);
        imp::rmsnorm(tx, tw, to, 1e-5f);
        emit_f("rmsnorm_eps1e-5", dout.host());
        imp::rmsnorm(tx, tw, to, 0.5f);
        emit_f("rmsnorm_eps0.5", dout.host());
        imp::rmsnorm(tx, tw, to, 1e-6f, nullptr, 1.0f);
        emit_f("rmsnorm_offset1", dout.host());
    }
    {   // rotary encoding, float32, pairs (i, i + Dh/2), whole head and the first 8 of 16 components
        const int T = 6, Hq = 3, Hkv = 2, Dh = 16;
        auto q = randoms((size_t)T * Hq * Dh, 1.0f), k = randoms((size_t)T * Hkv * Dh, 1.0f);
        std::vector<int> pos = {0, 1, 5, 17, 100, 1000};
        Dev<int> dpos(pos);
        emit_f("rope_q", q);
        emit_f("rope_k", k);
        emit_i("rope_positions", pos);
        for (int rope_dim : {0, 8}) {
            Dev<float> dq(q), dk(k);
            Tensor tq = tensor(dq.p, DType::FP32, {1, T, Hq, Dh}), tk = tensor(dk.p, DType::FP32, {1, T, Hkv, Dh});
            imp::rope_forward(tq, tk, dpos.p, Dh, 10000.0f, 1.0f, rope_dim, /*neox=*/true);
            emit_f(rope_dim ? "rope_q_out_dim8" : "rope_q_out", dq.host());
            emit_f(rope_dim ? "rope_k_out_dim8" : "rope_k_out", dk.host());
        }
    }
    {   // per-head RMSNorm on q and k, then the rotary encoding, in the reference's one-token kernel (half)
        const int Hq = 4, Hkv = 2, Dh = 32;
        auto q = randoms((size_t)Hq * Dh, 1.5f), k = randoms((size_t)Hkv * Dh, 1.5f);
        auto qw = randoms(Dh, 0.3f, 1.0f), kw = randoms(Dh, 0.3f, 1.0f);
        std::vector<int> pos = {37};
        Dev<__half> dq(to_half(q)), dk(to_half(k)), dqw(to_half(qw)), dkw(to_half(kw));
        Dev<int> dpos(pos);
        emit_f("qknorm_q", to_float(to_half(q)));
        emit_f("qknorm_k", to_float(to_half(k)));
        emit_f("qknorm_qw", to_float(to_half(qw)));
        emit_f("qknorm_kw", to_float(to_half(kw)));
        imp::qknorm_rope_fused(dq.p, dk.p, dqw.p, dkw.p, Hq, Hkv, Dh, 1e-3f, dpos.p, 1000000.0f, 1.0f, 0, /*neox=*/true, nullptr,
                               0.0f, 0.0f, 1.0f, nullptr, nullptr);
        emit_f("qknorm_q_out", to_float(dq.host()));
        emit_f("qknorm_k_out", to_float(dk.host()));
    }
    {   // SwiGLU, float32
        const int T = 4, F = 24;
        auto g = randoms((size_t)T * F, 4.0f), u = randoms((size_t)T * F, 2.0f);
        Dev<float> dg(g), du(u), dout((size_t)T * F);
        Tensor tg = tensor(dg.p, DType::FP32, {T, F}), tu = tensor(du.p, DType::FP32, {T, F}), to = tensor(dout.p, DType::FP32, {T, F});
        imp::swiglu(tg, tu, to);
        emit_f("swiglu_gate", g);
        emit_f("swiglu_up", u);
        emit_f("swiglu_out", dout.host());
    }
    {   // embedding lookup, float32
        const int V = 11, d = 8;
        auto table = randoms((size_t)V * d, 1.0f);
        std::vector<int> ids = {0, 10, 3, 3, 7};
        Dev<float> dt(table), dout(ids.size() * d);
        Dev<int> dids(ids);
        Tensor tt = tensor(dt.p, DType::FP32, {V, d}), to = tensor(dout.p, DType::FP32, {(int64_t)ids.size(), d});
        imp::embedding_lookup(tt, dids.p, (int)ids.size(), to);
        emit_f("embedding_table", table);
        emit_i("embedding_ids", ids);
        emit_f("embedding_out", dout.host());
    }
    {   // greedy sampling: ties go to the lowest index
        std::vector<int> picks;
        std::vector<float> all;
        for (int c = 0; c < 3; ++c) {
            const int V = c == 2 ? 40000 : 503;
            auto lg = randoms((size_t)V, 3.0f);
            if (c == 0) lg[77] = lg[400] = 9.0f;               // a tie
            if (c == 1) lg[V - 1] = 11.0f;                     // the last entry
            if (c == 2) lg[123] = lg[39999] = lg[20000] = 8.5f;   // a tie across the blocks of the two-stage kernel
            Dev<float> dl(lg);
            Tensor tl = tensor(dl.p, DType::FP32, {V});   // the reference takes the vocabulary size from shape[0]
            picks.push_back(imp::sample_greedy(tl));
            if (c < 2) all.insert(all.end(), lg.begin(), lg.end());
        }
        emit_f("greedy_logits_503x2", all);
        emit_i("greedy_picks", picks);
    }
    {   // causal attention, half precision: 12 tokens, 4 query heads on 2 kv heads of 16
        const int T = 12, Hq = 4, Hkv = 2, Dh = 16;
        auto q = randoms((size_t)T * Hq * Dh, 1.0f), k = randoms((size_t)T * Hkv * Dh, 1.0f), v = randoms((size_t)T * Hkv * Dh, 1.0f);
        Dev<__half> dq(to_half(q)), dk(to_half(k)), dv(to_half(v)), dout((size_t)T * Hq * Dh);
        Tensor tq = tensor(dq.p, DType::FP16, {1, T, Hq, Dh}), tk = tensor(dk.p, DType::FP16, {1, T, Hkv, Dh}),
               tv = tensor(dv.p, DType::FP16, {1, T, Hkv, Dh}), to = tensor(dout.p, DType::FP16, {1, T, Hq, Dh});
        imp::flash_attention_prefill(tq, tk, tv, to, 0.25f, /*causal=*/true);
        emit_f("attention_q", to_float(to_half(q)));
        emit_f("attention_k", to_float(to_half(k)));
        emit_f("attention_v", to_float(to_half(v)));
        emit_f("attention_out", to_float(dout.host()));
        Dev<__half> dwin((size_t)T * Hq * Dh);
        Tensor tw = tensor(dwin.p, DType::FP16, {1, T, Hq, Dh});
        imp::flash_attention_prefill(tq, tk, tv, tw, 0.25f, /*causal=*/true, /*sliding_window=*/5);
        emit_f("attention_out_window5", to_float(dwin.host()));
    }
    printf("}\n");
    CK(cudaDeviceSynchronize());
    return 0;
}
