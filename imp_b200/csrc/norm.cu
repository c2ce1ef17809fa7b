// RMSNorm fused with the residual sum, and a plain row RMSNorm.
//
// Formula (src/compute/layernorm.cu:50-82 in the reference):
//   y = x * rsqrt(mean(x^2) + eps) * (w + weight_offset)
// with the sum of squares, the rsqrt and the product in 32-bit.  The residual
// stream itself is 32-bit here in both precisions (the reference keeps it in
// fp16 and has a separate rmsnorm_residual kernel, src/compute/layernorm.cu:
// 167-300): a branch output is added into it in the same pass that normalises
// it for the next matrix product, so the residual sum is never rounded to
// bfloat16.  One block per row, a fixed block size: the order of additions of
// a row does not depend on the batch it is in.
#include "common.cuh"

constexpr int NORM_BLOCK = 256;

// h: [n_rows_total, d] 32-bit residual stream.
// branch: optional [n_rows_total, d] (TA) to add first.
// rows: optional gather list; output row r reads stream row rows[r].
// write_h: store h + branch back (never with a gather list that may repeat rows).
template <typename TA, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TA* __restrict__ branch,
                                   const TW* __restrict__ w, TA* __restrict__ out,
                                   const int* __restrict__ rows, int d, float eps, float weight_offset,
                                   int write_h) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = rows ? rows[r] : r;
    float* hrow = h + src * d;
    const TA* brow = branch ? branch + src * d : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += NORM_BLOCK) {
        float v = hrow[i];
        if (brow) v += to_float(brow[i]);
        if (write_h && brow) hrow[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)d + eps);
    TA* orow = out + (int64_t)r * d;
    for (int i = threadIdx.x; i < d; i += NORM_BLOCK) {
        float v = hrow[i];
        if (brow && !write_h) v += to_float(brow[i]);
        orow[i] = from_float<TA>(v * inv * (to_float(w[i]) + weight_offset));
    }
}

// Fast path for rows of up to 8192 floats whose width is a multiple of 4: the row is read once
// with 16-byte loads issued together, kept in registers, and written from there.  The per-thread
// partial sums and the block reduction add in an order fixed by the width alone.
constexpr int NORM_MAX_V4 = 8;   // float4 per thread: 256 threads x 8 x 4 = 8192 columns

template <typename T> struct Vec4 {};
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a);
        u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <typename TA, typename TW>
__global__ void __launch_bounds__(NORM_BLOCK) add_rmsnorm_vec_kernel(float* __restrict__ h, const TA* __restrict__ branch,
                                                                     const TW* __restrict__ w, TA* __restrict__ out,
                                                                     const int* __restrict__ rows, int d, float eps,
                                                                     float weight_offset, int write_h) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = rows ? rows[r] : r;
    float* hrow = h + src * d;
    const TA* brow = branch ? branch + src * d : nullptr;
    const int nv = d >> 2;
    float4 v[NORM_MAX_V4], wv[NORM_MAX_V4];
#pragma unroll
    for (int i = 0; i < NORM_MAX_V4; ++i) {
        const int c = threadIdx.x + i * NORM_BLOCK;
        if (c < nv) {
            v[i] = Vec4<float>::load(hrow + 4 * c);
            wv[i] = Vec4<TW>::load(w + 4 * c);
        }
    }
    if (brow) {
#pragma unroll
        for (int i = 0; i < NORM_MAX_V4; ++i) {
            const int c = threadIdx.x + i * NORM_BLOCK;
            if (c < nv) {
                const float4 b = Vec4<TA>::load(brow + 4 * c);
                v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAX_V4; ++i) {
        const int c = threadIdx.x + i * NORM_BLOCK;
        if (c < nv) {
            if (write_h && brow) Vec4<float>::store(hrow + 4 * c, v[i]);
            ss += v[i].x * v[i].x;
            ss += v[i].y * v[i].y;
            ss += v[i].z * v[i].z;
            ss += v[i].w * v[i].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)d + eps);
    TA* orow = out + (int64_t)r * d;
#pragma unroll
    for (int i = 0; i < NORM_MAX_V4; ++i) {
        const int c = threadIdx.x + i * NORM_BLOCK;
        if (c < nv) {
            float4 o;
            o.x = v[i].x * inv * (wv[i].x + weight_offset);
            o.y = v[i].y * inv * (wv[i].y + weight_offset);
            o.z = v[i].z * inv * (wv[i].z + weight_offset);
            o.w = v[i].w * inv * (wv[i].w + weight_offset);
            Vec4<TA>::store(orow + 4 * c, o);
        }
    }
}

IMP_API int imp_add_rmsnorm(float* h, const void* branch, const void* w, void* out, const int* rows,
                            int n_out_rows, int d, float eps, float weight_offset, int act_dtype,
                            int w_dtype, int write_h, void* stream) {
    if (n_out_rows == 0) return 0;
    IMP_CHECK_ARG(h && w && out && d > 0, "imp_add_rmsnorm: bad argument");
    IMP_CHECK_ARG(!(rows && write_h), "imp_add_rmsnorm: write_h with a row list is not allowed");
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = d % 4 == 0 && d <= NORM_BLOCK * NORM_MAX_V4 * 4 && (uintptr_t)h % 16 == 0 &&
                     (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0 && (!branch || (uintptr_t)branch % 16 == 0);
#define LAUNCH(TA, TW)                                                                                     \
    do {                                                                                                   \
        if (vec)                                                                                           \
            imp_launch(add_rmsnorm_vec_kernel<TA, TW>, dim3(n_out_rows), dim3(NORM_BLOCK), 0, s, h,        \
                       (const TA*)branch, (const TW*)w, (TA*)out, rows, d, eps, weight_offset, write_h);   \
        else                                                                                               \
            add_rmsnorm_kernel<TA, TW><<<n_out_rows, NORM_BLOCK, 0, s>>>(                                  \
                h, (const TA*)branch, (const TW*)w, (TA*)out, rows, d, eps, weight_offset, write_h);       \
    } while (0)
    if (act_dtype == IMP_F32 && w_dtype == IMP_F32) LAUNCH(float, float);
    else if (act_dtype == IMP_F32) LAUNCH(float, __nv_bfloat16);
    else if (w_dtype == IMP_F32) LAUNCH(__nv_bfloat16, float);
    else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
    IMP_RETURN_LAUNCH();
}

// Plain RMSNorm over rows of `x` (row stride in elements), any element type.
template <typename TA, typename TW>
__global__ void rmsnorm_rows_kernel(const TA* __restrict__ x, int64_t x_stride, const TW* __restrict__ w,
                                    TA* __restrict__ out, int64_t out_stride, int d, float eps,
                                    float weight_offset) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const TA* xr = x + (int64_t)blockIdx.x * x_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += NORM_BLOCK) {
        const float v = to_float(xr[i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)d + eps);
    TA* orow = out + (int64_t)blockIdx.x * out_stride;
    for (int i = threadIdx.x; i < d; i += NORM_BLOCK)
        orow[i] = from_float<TA>(to_float(xr[i]) * inv * (to_float(w[i]) + weight_offset));
}

IMP_API int imp_rmsnorm_rows(const void* x, int64_t x_stride, const void* w, void* out, int64_t out_stride,
                             int n_rows, int d, float eps, float weight_offset, int act_dtype, int w_dtype,
                             void* stream) {
    if (n_rows == 0) return 0;
    IMP_CHECK_ARG(x && w && out && d > 0, "imp_rmsnorm_rows: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH(TA, TW)                                                                                 \
    rmsnorm_rows_kernel<TA, TW><<<n_rows, NORM_BLOCK, 0, s>>>((const TA*)x, x_stride, (const TW*)w,    \
                                                              (TA*)out, out_stride, d, eps, weight_offset)
    if (act_dtype == IMP_F32 && w_dtype == IMP_F32) LAUNCH(float, float);
    else if (act_dtype == IMP_F32) LAUNCH(float, __nv_bfloat16);
    else if (w_dtype == IMP_F32) LAUNCH(__nv_bfloat16, float);
    else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
    IMP_RETURN_LAUNCH();
}
