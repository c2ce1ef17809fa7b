// The library arm of the matrix products: cuBLASLt, loaded at run time, for IMP_B200_GEMM=cublas.
// It exists as a yardstick (the reference's engine sends its T>1 products to cublasLtMatmul,
// src/compute/gemm.cu:303-445); the default path never comes here, and the library is not a
// link-time dependency: without libcublasLt the arm is simply not there.
#include <cublasLt.h>
#include <dlfcn.h>

#include <map>
#include <mutex>
#include <tuple>

#include "ops.hpp"

namespace imp {

namespace {

struct Lt {
    void* so = nullptr;
    decltype(&cublasLtCreate) create = nullptr;
    decltype(&cublasLtMatmulDescCreate) desc_create = nullptr;
    decltype(&cublasLtMatmulDescDestroy) desc_destroy = nullptr;
    decltype(&cublasLtMatmulDescSetAttribute) desc_set = nullptr;
    decltype(&cublasLtMatrixLayoutCreate) layout_create = nullptr;
    decltype(&cublasLtMatrixLayoutDestroy) layout_destroy = nullptr;
    decltype(&cublasLtMatmulPreferenceCreate) pref_create = nullptr;
    decltype(&cublasLtMatmulPreferenceDestroy) pref_destroy = nullptr;
    decltype(&cublasLtMatmulPreferenceSetAttribute) pref_set = nullptr;
    decltype(&cublasLtMatmulAlgoGetHeuristic) heuristic = nullptr;
    decltype(&cublasLtMatmul) matmul = nullptr;
    cublasLtHandle_t handle = nullptr;
    DeviceBuffer workspace;
    std::map<std::tuple<int64_t, int64_t, int64_t, int, int64_t, int64_t, int64_t>, cublasLtMatmulAlgo_t> algos;
    bool ok = false;
};

std::mutex g_mutex;
Lt g_lt;
bool g_tried = false;

template <typename F> bool sym(void* so, const char* name, F& fn) {
    fn = (F)dlsym(so, name);
    return fn != nullptr;
}

bool load_lt() {
    if (g_tried) return g_lt.ok;
    g_tried = true;
    for (const char* name : {"libcublasLt.so.12", "libcublasLt.so", "/usr/local/cuda/lib64/libcublasLt.so.12"}) {
        g_lt.so = dlopen(name, RTLD_NOW | RTLD_LOCAL);
        if (g_lt.so) break;
    }
    if (!g_lt.so) {
        log_line(LOG_WARN, "IMP_B200_GEMM=cublas: libcublasLt cannot be loaded (%s); the library arm is not available", dlerror());
        return false;
    }
    Lt& l = g_lt;
    bool all = sym(l.so, "cublasLtCreate", l.create) && sym(l.so, "cublasLtMatmulDescCreate", l.desc_create) &&
               sym(l.so, "cublasLtMatmulDescDestroy", l.desc_destroy) && sym(l.so, "cublasLtMatmulDescSetAttribute", l.desc_set) &&
               sym(l.so, "cublasLtMatrixLayoutCreate", l.layout_create) && sym(l.so, "cublasLtMatrixLayoutDestroy", l.layout_destroy) &&
               sym(l.so, "cublasLtMatmulPreferenceCreate", l.pref_create) && sym(l.so, "cublasLtMatmulPreferenceDestroy", l.pref_destroy) &&
               sym(l.so, "cublasLtMatmulPreferenceSetAttribute", l.pref_set) && sym(l.so, "cublasLtMatmulAlgoGetHeuristic", l.heuristic) &&
               sym(l.so, "cublasLtMatmul", l.matmul);
    if (!all || l.create(&l.handle) != CUBLAS_STATUS_SUCCESS) return false;
    l.workspace = DeviceBuffer((size_t)64 << 20);
    l.ok = true;
    return true;
}

}  // namespace

// out[M,N] = x[M,K] w[N,K]^T, bfloat16 operands, 32-bit accumulation, bfloat16 or float32 output.  Row-major
// C = A W^T is the column-major product C^T [N x M] = op_T(W as [K x N]) * (A as [K x M]).
bool library_gemm_bf16(Runtime& rt, Tensor out, const Tensor& x, const Tensor& w) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!load_lt()) return false;
    Lt& l = g_lt;
    const int64_t M = rows(x), N = rows(w), K = cols(x);
    const cudaDataType_t ctype = out.dtype == F32 ? CUDA_R_32F : CUDA_R_16BF;
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
    bool done = false;
    if (l.desc_create(&op, CUBLAS_COMPUTE_32F, CUDA_R_32F) == CUBLAS_STATUS_SUCCESS) {
        const cublasOperation_t T = CUBLAS_OP_T, Nn = CUBLAS_OP_N;
        l.desc_set(op, CUBLASLT_MATMUL_DESC_TRANSA, &T, sizeof T);
        l.desc_set(op, CUBLASLT_MATMUL_DESC_TRANSB, &Nn, sizeof Nn);
        if (l.layout_create(&la, CUDA_R_16BF, (uint64_t)K, (uint64_t)N, w.stride0) == CUBLAS_STATUS_SUCCESS &&
            l.layout_create(&lb, CUDA_R_16BF, (uint64_t)K, (uint64_t)M, x.stride0) == CUBLAS_STATUS_SUCCESS &&
            l.layout_create(&lc, ctype, (uint64_t)N, (uint64_t)M, out.stride0) == CUBLAS_STATUS_SUCCESS) {
            const auto key = std::make_tuple(M, N, K, out.dtype, (int64_t)w.stride0, (int64_t)x.stride0, (int64_t)out.stride0);
            auto it = l.algos.find(key);
            bool have = it != l.algos.end();
            if (!have) {
                cublasLtMatmulPreference_t pref = nullptr;
                if (l.pref_create(&pref) == CUBLAS_STATUS_SUCCESS) {
                    const size_t ws = l.workspace.bytes();
                    l.pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws, sizeof ws);
                    cublasLtMatmulHeuristicResult_t res{};
                    int found = 0;
                    if (l.heuristic(l.handle, op, la, lb, lc, lc, pref, 1, &res, &found) == CUBLAS_STATUS_SUCCESS && found > 0) {
                        it = l.algos.emplace(key, res.algo).first;
                        have = true;
                    }
                    l.pref_destroy(pref);
                }
            }
            if (have) {
                const float alpha = 1.f, beta = 0.f;
                done = l.matmul(l.handle, op, &alpha, w.data, la, x.data, lb, &beta, out.data, lc, out.data, lc, &it->second,
                                l.workspace.data(), l.workspace.bytes(), rt.stream) == CUBLAS_STATUS_SUCCESS;
            }
        }
    }
    if (la) l.layout_destroy(la);
    if (lb) l.layout_destroy(lb);
    if (lc) l.layout_destroy(lc);
    if (op) l.desc_destroy(op);
    if (done) ++rt.launches;
    return done;
}

}  // namespace imp
