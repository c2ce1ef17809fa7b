// Matrix products, norms and the other tensor-level operations: checks and kernel choice.
#include <cstring>

#include "kernels.h"
#include "ops.hpp"

namespace imp {

namespace {
constexpr int SMALL_M_MAX = 16;     // most rows the weight-streaming kernel takes
// Rows up to which it is the first choice; IMP_B200_STREAM_ROWS moves it.  Whole decode steps of the 8B shape measured
// with both kernels: one row 3.39 ms against 3.47 with the tcgen05 swap-AB kernel, two rows 3.55 / 3.53, four 3.76 / 3.72,
// six 4.03 / 3.91, seven 4.06 / 4.00.
static int stream_m_max() {
    static const int v = [] { const std::string e = env_string("IMP_B200_STREAM_ROWS", ""); return e.empty() ? 1 : std::atoi(e.c_str()); }();
    return v;
}
constexpr int TC_SWAP_MAX_M = 128;  // rows up to which the weights take the M side of the tcgen05 product

// "tcgen05": this library's TMA + tcgen05 kernels.  "cublas": the library GEMM for products of more than 16
// rows (a yardstick; see cublas_arm.cpp).
bool use_library_gemm() {
    static int v = -1;
    if (v < 0) {
        const std::string s = env_string("IMP_B200_GEMM", "tcgen05");
        if (s != "tcgen05" && s != "cublas") fail(IMP_ERROR_INVALID_ARG, "IMP_B200_GEMM must be 'tcgen05' or 'cublas', got '" + s + "'");
        v = s == "cublas" ? 1 : 0;
    }
    return v == 1;
}
bool defer_split_sums() {
    static int v = -1;
    if (v < 0) v = (env_flag("IMP_B200_DEFER_SUM", true) && !env_flag("IMP_B200_DEBUG_FORWARD", false)) ? 1 : 0;
    return v == 1;
}

void need(bool cond, const char* what) {
    if (!cond) fail(IMP_ERROR_INVALID_ARG, what);
}

int64_t M_of(const Tensor& t) { return rows(t); }
}  // namespace

bool library_gemm_bf16(Runtime& rt, Tensor out, const Tensor& x, const Tensor& w);   // cublas_arm.cpp

void cast(Runtime& rt, Tensor dst, const Tensor& src) {
    need(numel(dst) == numel(src) && contiguous(dst) && contiguous(src), "cast: tensors must be dense and of equal size");
    ++rt.launches;
    check_launch(imp_cast(dst.data, dst.dtype, src.data, src.dtype, numel(src), rt.stream), "cast");
}

void swiglu(Runtime& rt, Tensor out, const Tensor& gate_up, int interleave) {
    need(cols(gate_up) == 2 * cols(out) && rows(gate_up) == rows(out) && gate_up.dtype == out.dtype && contiguous(out) &&
             contiguous(gate_up),
         "swiglu: gate_up must be [T, 2F] beside out [T, F], both dense");
    ++rt.launches;
    check_launch(imp_swiglu(out.data, gate_up.data, (int)rows(out), (int)cols(out), interleave, out.dtype, rt.stream), "swiglu");
}

void embedding(Runtime& rt, Tensor out, const Tensor& table, const int32_t* ids, int n, float scale) {
    need(out.dtype == F32 && contiguous(out) && rows(out) == n && cols(out) == cols(table) && contiguous(table),
         "embedding: out must be dense float32 [T, d] and the table dense [vocab, d]");
    ++rt.launches;
    check_launch(imp_embedding((float*)out.data, table.data, ids, n, (int)cols(out), (int)rows(table), table.dtype, scale,
                               rt.status, rt.stream),
                 "embedding");
}

// ----------------------------------------------------------------------------- matrix products
static void gemm_f32(Runtime& rt, Tensor out, const Tensor& a, const Tensor& w) {
    ++rt.launches;
    check_launch(imp_gemm_f32((float*)out.data, out.stride0, (const float*)a.data, a.stride0, (const float*)w.data, w.stride0,
                              (int)rows(a), (int)rows(w), (int)cols(a), rt.stream),
                 "gemm_f32");
}

static void gemm_plain(Runtime& rt, Tensor out, const Tensor& a, const Tensor& w) {
    ++rt.launches;
    ++rt.fallback_calls;
    check_launch(imp_gemm_bf16_plain(out.data, out.stride0, out.dtype, a.data, a.stride0, w.data, w.stride0, (int)rows(a),
                                     (int)rows(w), (int)cols(a), rt.stream),
                 "gemm_bf16_plain");
}

static void gemm_stream(Runtime& rt, Tensor out, const Tensor& a, const Tensor& w) {
    const int M = (int)rows(a), N = (int)rows(w), K = (int)cols(a);
    ++rt.launches;
    int rc = imp_gemm_bf16_stream(out.data, out.stride0, out.dtype, a.data, a.stride0, w.data, w.stride0, M, N, K, rt.stream);
    if (rc == -2) rc = imp_gemm_bf16_small_m(out.data, out.stride0, out.dtype, a.data, a.stride0, w.data, w.stride0, M, N, K, rt.stream);
    if (rc == -2) {
        --rt.launches;
        gemm_plain(rt, out, a, w);
        return;
    }
    check_launch(rc, "gemm_bf16_stream");
}

static bool gemm_tc(Runtime& rt, Tensor out, const Tensor& a, const Tensor& w, int epilogue = -1) {
    if (epilogue < 0) epilogue = out.dtype == F32 ? TC_OUT_F32 : TC_OUT_BF16;
    if (epilogue != TC_OUT_SWIGLU) {
        // few 256 x 256 tiles for the device's CTA pairs (a portion of a prompt): the K range in parts, then their sum
        const int M = (int)rows(a), N = (int)rows(w), K = (int)cols(a);
        const int n_splits = imp_gemm_bf16_tc_splits(M, N, K);
        if (n_splits > 1) {
            const Arena::Mark mark = rt.arena->mark();
            float* parts = (float*)rt.arena->alloc((size_t)n_splits * M * N * 4);
            const int rc = imp_gemm_bf16_tc_partials(parts, a.data, a.stride0, w.data, w.stride0, M, N, K, rt.status, rt.stream);
            if (rc != -2) {
                check_launch(rc, "gemm_bf16_tc_partials");
                check_launch(imp_gemm_bf16_tc_swap_sum(out.data, out.stride0, epilogue, parts, M, N, n_splits, rt.stream), "gemm_bf16_tc_sum");
                rt.launches += 2;
                return true;
            }
            rt.arena->restore(mark);
        }
    }
    const int rc = imp_gemm_bf16_tc(out.data, out.stride0, epilogue, a.data, a.stride0, w.data, w.stride0, (int)rows(a),
                                    (int)rows(w), (int)cols(a), rt.status, rt.stream);
    if (rc == -2) return false;
    ++rt.launches;
    check_launch(rc, "gemm_bf16_tc");
    return true;
}

static bool gemm_tc_swap(Runtime& rt, Tensor out, const Tensor& a, const Tensor& w, int epilogue = -1) {
    if (epilogue < 0) epilogue = out.dtype == F32 ? TC_OUT_F32 : TC_OUT_BF16;
    const int M = (int)rows(a), N = (int)rows(w), K = (int)cols(a);
    const int64_t n_scratch = imp_gemm_bf16_tc_swap_scratch_floats(M, N, K, epilogue);
    float* scratch = n_scratch > 0 ? (float*)rt.arena->alloc((size_t)n_scratch * 4) : nullptr;
    const int rc = imp_gemm_bf16_tc_swap(out.data, out.stride0, epilogue, a.data, a.stride0, w.data, w.stride0, M, N, K, scratch,
                                         rt.status, rt.stream);
    if (rc == -2) return false;
    rt.launches += n_scratch > 0 ? 2 : 1;
    check_launch(rc, "gemm_bf16_tc_swap");
    return true;
}

static bool gemm_tc_swap_partials(Runtime& rt, Tensor out, const Tensor& a, const Tensor& w, Branch* result) {
    const int M = (int)rows(a), N = (int)rows(w), K = (int)cols(a);
    const int n_splits = imp_gemm_bf16_tc_swap_splits(M, N, K);
    if (n_splits < 2) return false;
    float* parts = (float*)rt.arena->alloc((size_t)n_splits * M * N * 4);
    const int rc = imp_gemm_bf16_tc_swap_partials(parts, a.data, a.stride0, w.data, w.stride0, M, N, K, rt.status, rt.stream);
    if (rc == -2) return false;
    ++rt.launches;
    check_launch(rc, "gemm_bf16_tc_swap_partials");
    result->t = out;
    result->parts = parts;
    result->n_splits = n_splits;
    return true;
}

Tensor summed(Runtime& rt, const Branch& b) {
    if (!b.split()) return b.t;
    const int epi = b.t.dtype == F32 ? TC_OUT_F32 : TC_OUT_BF16;
    ++rt.launches;
    check_launch(imp_gemm_bf16_tc_swap_sum(b.t.data, b.t.stride0, epi, b.parts, (int)rows(b.t), (int)cols(b.t), b.n_splits, rt.stream),
                 "gemm_bf16_tc_swap_sum");
    return b.t;
}

Branch linear(Runtime& rt, Tensor out, const Tensor& x, const Tensor& w, bool may_defer) {
    const int64_t M = M_of(x);
    need(cols(x) == cols(w) && rows(out) == M && cols(out) == rows(w), "linear: shapes do not agree");
    if (M == 0) return Branch::of(out);
    if (w.dtype == F32) {
        Tensor xf = x;
        if (x.dtype != F32) {
            need(contiguous(x), "linear: activations must be dense to be widened");
            xf = rt.empty(M, cols(x), F32);
            cast(rt, xf, x);
        }
        if (out.dtype == F32) {
            gemm_f32(rt, out, xf, w);
            return Branch::of(out);
        }
        Tensor tmp = rt.empty(M, cols(out), F32);
        gemm_f32(rt, tmp, xf, w);
        if (contiguous(out)) {
            cast(rt, out, tmp);
        } else {
            Tensor dense = rt.empty(M, cols(out), out.dtype);
            cast(rt, dense, tmp);
            IMP_CUDA(cudaMemcpy2DAsync(out.data, (size_t)out.stride0 * elem_size(out.dtype), dense.data,
                                       (size_t)cols(out) * elem_size(out.dtype), (size_t)cols(out) * elem_size(out.dtype),
                                       (size_t)M, cudaMemcpyDeviceToDevice, rt.stream));
        }
        return Branch::of(out);
    }
    if (x.dtype != BF16 || w.dtype != BF16)
        fail(IMP_ERROR_INVALID_ARG, "bfloat16 weights need bfloat16 activations (the float32 path widens weights at load)");
    const bool lib = use_library_gemm();
    const bool defer = may_defer && defer_split_sums() && contiguous(out);
    const int64_t N = rows(w), K = cols(w);
    Branch b;
    if (M <= SMALL_M_MAX) {
        // The weight-streaming kernel, except where the swap-AB tcgen05 kernel measured faster: from 8 rows up,
        // and at any row count for products with a long contraction and few output columns (K split over CTAs).
        if (!lib && (M > stream_m_max() || (K >= 2 * N && N >= 1024))) {
            if (defer && gemm_tc_swap_partials(rt, out, x, w, &b)) return b;
            if (gemm_tc_swap(rt, out, x, w)) return Branch::of(out);
        }
        gemm_stream(rt, out, x, w);
        return Branch::of(out);
    }
    if (!lib) {
        if (M <= TC_SWAP_MAX_M) {
            if (defer && gemm_tc_swap_partials(rt, out, x, w, &b)) return b;
            if (gemm_tc_swap(rt, out, x, w)) return Branch::of(out);
        }
        if (gemm_tc(rt, out, x, w)) return Branch::of(out);
    } else if (library_gemm_bf16(rt, out, x, w)) {
        return Branch::of(out);
    }
    gemm_plain(rt, out, x, w);
    return Branch::of(out);
}

void linear_swiglu(Runtime& rt, Tensor out, const Tensor& x, const Tensor& w) {
    const int64_t M = M_of(x), F = cols(out);
    if (M == 0) return;
    const bool bf16 = x.dtype == BF16 && w.dtype == BF16 && out.dtype == BF16;
    const bool lib = use_library_gemm();
    if (bf16 && M > stream_m_max() && M <= SMALL_M_MAX && !lib && gemm_tc_swap(rt, out, x, w, TC_OUT_SWIGLU)) return;
    if (bf16 && M <= SMALL_M_MAX) {
        const int rc = imp_gemm_bf16_stream_swiglu(out.data, out.stride0, x.data, x.stride0, w.data, w.stride0, (int)M, (int)(2 * F),
                                                   (int)cols(x), rt.stream);
        if (rc != -2) {
            ++rt.launches;
            check_launch(rc, "gemm_bf16_stream_swiglu");
            return;
        }
    }
    if (bf16 && !lib) {
        if (M <= TC_SWAP_MAX_M && gemm_tc_swap(rt, out, x, w, TC_OUT_SWIGLU)) return;
        if (gemm_tc(rt, out, x, w, TC_OUT_SWIGLU)) return;
    }
    Tensor gu = rt.empty(M, 2 * F, x.dtype);
    linear(rt, gu, x, w);
    swiglu(rt, out, gu, SWIGLU_INTERLEAVE);
}

// ---------------------------------------------------------------------------------------- norm
void add_rmsnorm(Runtime& rt, Tensor h, const Branch& branch, const Tensor& weight, Tensor out, float eps, float offset,
                 const int32_t* rows_idx, int n_rows) {
    const int d = (int)cols(h);
    need(h.dtype == F32 && contiguous(h) && contiguous(out) && cols(out) == d && numel(weight) == d,
         "add_rmsnorm: the stream must be dense float32 [T, d], out [n, d], the weight [d]");
    const int n_out = (int)rows(out);
    need(rows_idx ? n_out == n_rows : n_out == rows(h), "add_rmsnorm: out has the wrong number of rows");
    const int write_h = rows_idx ? 0 : 1;
    const void* plain = nullptr;
    if (branch.split()) {
        need(rows(branch.t) == rows(h) && cols(branch.t) == d && branch.t.dtype == out.dtype, "add_rmsnorm: branch shape or type");
        const int rc = imp_add_rmsnorm_split((float*)h.data, branch.parts, rows(h) * (int64_t)d, branch.n_splits, weight.data, out.data,
                                             rows_idx, n_out, d, eps, offset, out.dtype, weight.dtype, write_h, rt.stream);
        if (rc != -2) {
            ++rt.launches;
            ++rt.split_norm_calls;
            check_launch(rc, "add_rmsnorm_split");
            return;
        }
        plain = summed(rt, branch).data;
    } else if (!branch.empty()) {
        need(rows(branch.t) == rows(h) && cols(branch.t) == d && branch.t.dtype == out.dtype && contiguous(branch.t),
             "add_rmsnorm: the branch must be dense, of the stream's shape and the output's type");
        plain = branch.t.data;
    }
    ++rt.launches;
    check_launch(imp_add_rmsnorm((float*)h.data, plain, weight.data, out.data, rows_idx, n_out, d, eps, offset, out.dtype,
                                 weight.dtype, write_h, rt.stream),
                 "add_rmsnorm");
}

// -------------------------------------------------------------------------- weight rearrangement
Tensor to_float32(Runtime& rt, WeightStore& store, const Tensor& t) {
    std::vector<int64_t> shape(t.shape, t.shape + t.ndim);
    Tensor f = store.alloc(F32, shape);
    if (t.dtype == F32) IMP_CUDA(cudaMemcpyAsync(f.data, t.data, (size_t)numel(t) * 4, cudaMemcpyDeviceToDevice, rt.stream));
    else cast(rt, f, t);
    return f;
}

Tensor cat_rows(Runtime& rt, WeightStore& store, const std::vector<Tensor>& parts) {
    int dt = parts.at(0).dtype;
    int64_t total = 0;
    const int64_t K = cols(parts[0]);
    for (const auto& p : parts) {
        if (p.dtype != dt) dt = F32;
        need(cols(p) == K && contiguous(p), "cat_rows: matrices must be dense and of equal width");
        total += rows(p);
    }
    Tensor out = store.alloc(dt, {total, K});
    int64_t r = 0;
    for (const auto& p : parts) {
        Tensor dst = tensor2d((char*)out.data + (size_t)(r * K) * elem_size(dt), dt, rows(p), K);
        if (p.dtype == dt) IMP_CUDA(cudaMemcpyAsync(dst.data, p.data, (size_t)numel(p) * elem_size(dt), cudaMemcpyDeviceToDevice, rt.stream));
        else cast(rt, dst, p);
        r += rows(p);
    }
    return out;
}

Tensor interleave_gate_up(Runtime& rt, WeightStore& store, const Tensor& gate, const Tensor& up) {
    const int64_t F = rows(gate), d = cols(gate);
    const int b = SWIGLU_INTERLEAVE;
    need(rows(up) == F && cols(up) == d && F % b == 0 && gate.dtype == up.dtype && contiguous(gate) && contiguous(up),
         "interleave_gate_up: gate and up must be dense [F, d] of one type with F a multiple of 8");
    Tensor out = store.alloc(gate.dtype, {2 * F, d});
    const size_t run = (size_t)b * (size_t)d * elem_size(gate.dtype);
    // runs of 8 gate rows land 16 rows apart, their 8 up rows right behind them
    IMP_CUDA(cudaMemcpy2DAsync(out.data, 2 * run, gate.data, run, run, (size_t)(F / b), cudaMemcpyDeviceToDevice, rt.stream));
    IMP_CUDA(cudaMemcpy2DAsync((char*)out.data + run, 2 * run, up.data, run, run, (size_t)(F / b), cudaMemcpyDeviceToDevice, rt.stream));
    return out;
}

}  // namespace imp
