// Tensor-level operations of the host as C entry points: the kernel choice the engine makes for a
// matrix product, a fused SwiGLU product and a norm, callable on caller-owned tensors and the
// caller's stream.  Tools and kernel tests use them so that what they measure is the engine's own
// choice, not a restatement of it.
#include <memory>

#include "kernels.h"
#include "ops.hpp"

using namespace imp;

namespace {
thread_local std::string g_ops_message;
thread_local std::unique_ptr<Arena> g_arena;
thread_local int64_t g_fallbacks = 0;

Runtime runtime_for(void* stream, int32_t* status) {
    if (!g_arena) g_arena = std::make_unique<Arena>(0, (size_t)1 << 22);
    // scratch of one call stays valid during the next one (unsummed parts travel from a product to a norm)
    g_arena->next_layer();
    Runtime rt;
    rt.stream = (cudaStream_t)stream;
    rt.status = status;
    rt.arena = g_arena.get();
    rt.sm_count = imp_device_sm_count();
    return rt;
}

template <typename F> int guarded(F&& f) {
    try {
        f();
        g_ops_message.clear();
        return IMP_SUCCESS;
    } catch (const Error& e) {
        g_ops_message = e.what();
        return e.code;
    } catch (const std::exception& e) {
        g_ops_message = e.what();
        return IMP_ERROR_INTERNAL;
    }
}
}  // namespace

extern "C" {

IMP_EXPORT const char* imp_op_error_message(void) { return g_ops_message.c_str(); }
IMP_EXPORT int64_t imp_op_fallback_calls(void) { return g_fallbacks; }

// out = x w^T.  With may_defer != 0 a product that the tcgen05 kernel splits over K is left unsummed:
// *parts_out [n_splits, M, N] float32 and *n_splits_out > 0 then describe it (valid until the call
// after next on this thread); otherwise *n_splits_out is 0 and `out` holds the result.
IMP_EXPORT int imp_op_linear(const ImpTensor* out, const ImpTensor* x, const ImpTensor* w, int may_defer, float** parts_out,
                             int* n_splits_out, void* stream, int32_t* status) {
    return guarded([&] {
        if (!out || !x || !w) fail(IMP_ERROR_INVALID_ARG, "imp_op_linear: null tensor");
        Runtime rt = runtime_for(stream, status);
        rt.dtype = x->dtype;
        Branch b = linear(rt, *out, *x, *w, may_defer != 0);
        g_fallbacks += rt.fallback_calls;
        if (parts_out) *parts_out = b.parts;
        if (n_splits_out) *n_splits_out = b.split() ? b.n_splits : 0;
        if (b.split() && !(parts_out && n_splits_out)) summed(rt, b);
    });
}

IMP_EXPORT int imp_op_linear_swiglu(const ImpTensor* out, const ImpTensor* x, const ImpTensor* w_interleaved, void* stream,
                                    int32_t* status) {
    return guarded([&] {
        if (!out || !x || !w_interleaved) fail(IMP_ERROR_INVALID_ARG, "imp_op_linear_swiglu: null tensor");
        Runtime rt = runtime_for(stream, status);
        rt.dtype = x->dtype;
        linear_swiglu(rt, *out, *x, *w_interleaved);
        g_fallbacks += rt.fallback_calls;
    });
}

// h (+= branch); out = rmsnorm(h) * (weight + offset).  `branch` may be null; with parts != NULL the branch
// is the unsummed product imp_op_linear left (branch then names where its sum belongs).
IMP_EXPORT int imp_op_add_rmsnorm(const ImpTensor* h, const ImpTensor* branch, const float* parts, int n_splits,
                                  const ImpTensor* weight, const ImpTensor* out, float eps, float offset, const int32_t* rows,
                                  int n_rows, void* stream) {
    return guarded([&] {
        if (!h || !weight || !out) fail(IMP_ERROR_INVALID_ARG, "imp_op_add_rmsnorm: null tensor");
        Runtime rt = runtime_for(stream, nullptr);
        rt.dtype = out->dtype;
        Branch b;
        if (branch && branch->data) b.t = *branch;
        if (parts && n_splits > 0) {
            b.parts = const_cast<float*>(parts);
            b.n_splits = n_splits;
        }
        add_rmsnorm(rt, *h, b, *weight, *out, eps, offset, rows, rows ? n_rows : 0);
    });
}

IMP_EXPORT int imp_op_decode_splits(int n_tokens, int n_kv_heads, int group, int page_size, int sm_count, int context) {
    return decode_splits(n_tokens, n_kv_heads, group, page_size, sm_count, context);
}

}  // extern "C"
