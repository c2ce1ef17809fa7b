// A part kind written against the C extension interface alone (include/imp_b200/imp_parts.h), in CUDA, with no
// Python in it: an RMS norm of its own, registered as norm kind "toy_c_rmsnorm".  The test compiles this file
// with nvcc, loads it beside the engine's library, calls toy_c_register() and builds a model whose plan names the kind.
// Nothing here is part of the framework; it shows what a part outside the framework has to provide:
//   tensor_specs  what tensors it wants, as JSON;
//   create        keep the device views of its tensors and its parameters;
//   forward       launch on the step's stream: add the branch into the 32-bit stream, normalise, write `out`;
//   destroy.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "imp_b200/imp_parts.h"

namespace {

struct ToyNorm {
    ImpTensor weight;
    float eps;
    int size;
};

__device__ float load(const float* p, int64_t i) { return p[i]; }
__device__ float load(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
__device__ void store(float* p, int64_t i, float v) { p[i] = v; }
__device__ void store(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// One block per output row.  rows == nullptr: out row i is stream row i, and the branch is added into the stream;
// else out row i is stream row rows[i] (plus its branch row) and the stream is left as it is.
template <typename TB, typename TW, typename TO>
__global__ void toy_rmsnorm_kernel(float* h, int64_t h_ld, const TB* branch, int64_t b_ld, const TW* w, TO* out, int64_t o_ld, int d,
                                   const int32_t* rows, float eps) {
    __shared__ float partial[32];
    const int i = blockIdx.x;
    const int64_t r = rows ? rows[i] : i;
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float v = h[r * h_ld + c];
        if (branch) v += load(branch, r * b_ld + c);
        if (branch && !rows) h[r * h_ld + c] = v;
        ss += v * v;
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.f;
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) partial[0] = rsqrtf(t / (float)d + eps);
    }
    __syncthreads();
    const float inv = partial[0];
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float v = h[r * h_ld + c];
        if (branch && rows) v += load(branch, r * b_ld + c);      // (without rows the stream already holds the sum)
        store(out, (int64_t)i * o_ld + c, v * inv * load(w, c));
    }
}

// "key": number in a flat JSON object (all this file needs of JSON)
double number_of(const char* json, const char* key, double dflt) {
    char pat[64];
    snprintf(pat, sizeof pat, "\"%s\"", key);
    const char* p = strstr(json, pat);
    if (!p) return dflt;
    p = strchr(p + strlen(pat), ':');
    return p ? strtod(p + 1, nullptr) : dflt;
}

char g_specs[256];

const char* tensor_specs(void*, const char* params_json) {
    snprintf(g_specs, sizeof g_specs, "{\"weight\": {\"shape\": [%d], \"role\": \"norm\", \"init\": \"one_plus_normal\"}}",
             (int)number_of(params_json, "size", 0));
    return g_specs;
}

void* create(void*, const char* params_json, int n_tensors, const char* const* names, const ImpTensor* tensors, int, const char* const*,
             const ImpPart*, int, int) {
    for (int i = 0; i < n_tensors; ++i)
        if (strcmp(names[i], "weight") == 0) {
            ToyNorm* n = new ToyNorm{tensors[i], (float)number_of(params_json, "eps", 1e-6), (int)number_of(params_json, "size", 0)};
            return n;
        }
    imp_part_set_error("toy_c_rmsnorm: no tensor named weight");
    return nullptr;
}

template <typename TB, typename TW, typename TO>
void launch(const ToyNorm* n, ImpCall* c, int n_out) {
    toy_rmsnorm_kernel<TB, TW, TO><<<n_out, 256, 0, (cudaStream_t)c->batch->stream>>>(
        (float*)c->h.data, c->h.stride0, (const TB*)c->branch.data, c->branch.stride0, (const TW*)n->weight.data, (TO*)c->out.data,
        c->out.stride0, n->size, c->rows, n->eps);
}

int forward(void* self, ImpCall* c) {
    const ToyNorm* n = (const ToyNorm*)self;
    const int n_out = c->rows ? c->n_rows : (int)c->h.shape[0];
    if (n_out == 0) return 0;
    if (c->h.dtype != IMP_ELEM_F32 || (int)c->h.shape[1] != n->size) {
        imp_part_set_error("toy_c_rmsnorm: the stream is not float32 of the part's width");
        return 1;
    }
    const bool b16 = c->branch.data ? c->branch.dtype == IMP_ELEM_BF16 : c->out.dtype == IMP_ELEM_BF16;
    const bool w16 = n->weight.dtype == IMP_ELEM_BF16, o16 = c->out.dtype == IMP_ELEM_BF16;
    if (b16 != o16) {
        imp_part_set_error("toy_c_rmsnorm: branch and output of different types");
        return 1;
    }
    if (o16 && w16) launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(n, c, n_out);
    else if (o16) launch<__nv_bfloat16, float, __nv_bfloat16>(n, c, n_out);
    else if (w16) launch<float, __nv_bfloat16, float>(n, c, n_out);
    else launch<float, float, float>(n, c, n_out);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        imp_part_set_error(cudaGetErrorString(e));
        return 1;
    }
    return 0;
}

void destroy(void* self) { delete (ToyNorm*)self; }

int g_created = 0;

}  // namespace

extern "C" int toy_c_register(void) {
    static ImpPartVTable vt;
    memset(&vt, 0, sizeof vt);
    vt.tensor_specs = tensor_specs;
    vt.create = create;
    vt.forward = forward;
    vt.destroy = destroy;
    (void)g_created;
    return (int)imp_register_part("norm", "toy_c_rmsnorm", &vt);
}

extern "C" int toy_c_unregister(void) { return (int)imp_unregister_part("norm", "toy_c_rmsnorm"); }
