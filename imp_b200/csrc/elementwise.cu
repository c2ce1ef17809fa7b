// Embedding gather, SwiGLU and dtype casts.
//
// Reference counterparts: embedding_lookup_* (src/compute/embedding.cu:15-112),
// swiglu_* (src/compute/activation.cu:15-87).  Differences: the gather writes
// the 32-bit residual stream directly, the activation uses the IEEE expf
// (the reference compiles __expf under --use_fast_math), and both take any
// width.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                 const int* __restrict__ ids, int d, int vocab, float scale,
                                 int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (int64_t)t * d;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) imp_report(status, IMP_BAD_TOKEN_ID);
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const TW* row = table + (int64_t)id * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

// out[t, :] = table[ids[t], :] * scale, as 32-bit floats.
IMP_API int imp_embedding(float* out, const void* table, const int* ids, int n_tokens, int d, int vocab,
                          int table_dtype, float scale, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(out && table && ids && d > 0 && vocab > 0, "imp_embedding: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const int block = d >= 1024 ? 256 : 128;
    if (table_dtype == IMP_F32)
        embedding_kernel<float><<<n_tokens, block, 0, s>>>(out, (const float*)table, ids, d, vocab, scale, status);
    else
        embedding_kernel<__nv_bfloat16><<<n_tokens, block, 0, s>>>(out, (const __nv_bfloat16*)table, ids, d,
                                                                  vocab, scale, status);
    IMP_RETURN_LAUNCH();
}

// ------------------------------------------------------------------- swiglu
// out[t, f] = silu(gate) * up; the activation is computed in 32-bit.  Layout of gu[t, 2F]:
// block == 0: gate columns 0..F-1, then up columns F..2F-1;
// block == b: gate and up interleaved in runs of b columns (b gate, b up, b gate, ...).
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t n_tokens, int F, int block) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t total = n_tokens * (int64_t)F;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / F;
        const int f = (int)(i - t * F);
        const int gi = block ? (f / block) * 2 * block + f % block : f;
        const int ui = block ? gi + block : F + f;
        const float g = to_float(gu[t * 2 * F + gi]);
        const float u = to_float(gu[t * 2 * F + ui]);
        const float a = g / (1.f + expf(-g));
        out[i] = from_float<T>(a * u);
    }
}

// bfloat16, F a multiple of 8, 16-byte aligned rows: a thread turns 8 gate and 8 up values into 8 outputs.
__global__ void swiglu_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu,
                                       int64_t n_tokens, int F, int block) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t total = n_tokens * (int64_t)(F >> 3);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / (F >> 3);
        const int f = (int)(i - t * (F >> 3)) << 3;
        const int gi = block ? (f / block) * 2 * block + f % block : f;   // block is a multiple of 8 here
        const int ui = block ? gi + block : F + f;
        const uint4 gv = *reinterpret_cast<const uint4*>(gu + t * 2 * F + gi);
        const uint4 uv = *reinterpret_cast<const uint4*>(gu + t * 2 * F + ui);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            o2[j] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + t * F + f) = ov;
    }
}

IMP_API int imp_swiglu(void* out, const void* gate_up, int n_tokens, int F, int block, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    IMP_CHECK_ARG(out && gate_up && F > 0, "imp_swiglu: bad argument");
    IMP_CHECK_ARG(block >= 0 && (block == 0 || F % block == 0), "imp_swiglu: width %d is not a multiple of the interleave %d", F, block);
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t total = (int64_t)n_tokens * F;
    const int threads = 256;
    const int64_t sms = imp_sm_count();
    const int grid = (int)((total + threads - 1) / threads < sms * 16 ? (total + threads - 1) / threads : sms * 16);
    if (dtype == IMP_BF16 && F % 8 == 0 && block % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gate_up % 16 == 0) {
        const int64_t work = total >> 3;
        const int g8 = (int)((work + threads - 1) / threads < sms * 32 ? (work + threads - 1) / threads : sms * 32);
        swiglu_bf16_vec_kernel<<<g8, threads, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, n_tokens, F, block);
    } else if (dtype == IMP_F32)
        swiglu_kernel<float><<<grid, threads, 0, s>>>((float*)out, (const float*)gate_up, n_tokens, F, block);
    else
        swiglu_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up,
                                                               n_tokens, F, block);
    IMP_RETURN_LAUNCH();
}

// --------------------------------------------------------------------- cast
template <typename TS, typename TD>
__global__ void cast_kernel(TD* __restrict__ dst, const TS* __restrict__ src, int64_t n) {
    pdl_wait();
    pdl_launch_dependents();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = from_float<TD>(to_float(src[i]));
}

IMP_API int imp_cast(void* dst, int dst_dtype, const void* src, int src_dtype, int64_t n, void* stream) {
    if (n == 0) return 0;
    IMP_CHECK_ARG(dst && src, "imp_cast: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    const int block = 256;
    const int64_t want = (n + block - 1) / block;
    const int64_t cap = (int64_t)imp_sm_count() * 16;
    const int grid = (int)(want < cap ? want : cap);
    if (src_dtype == IMP_F32 && dst_dtype == IMP_BF16)
        cast_kernel<float, __nv_bfloat16><<<grid, block, 0, s>>>((__nv_bfloat16*)dst, (const float*)src, n);
    else if (src_dtype == IMP_BF16 && dst_dtype == IMP_F32)
        cast_kernel<__nv_bfloat16, float><<<grid, block, 0, s>>>((float*)dst, (const __nv_bfloat16*)src, n);
    else if (src_dtype == IMP_F32 && dst_dtype == IMP_F32)
        cast_kernel<float, float><<<grid, block, 0, s>>>((float*)dst, (const float*)src, n);
    else
        cast_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, block, 0, s>>>((__nv_bfloat16*)dst,
                                                                       (const __nv_bfloat16*)src, n);
    IMP_RETURN_LAUNCH();
}
