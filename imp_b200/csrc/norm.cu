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

IMP_API int imp_add_rmsnorm(float* h, const void* branch, const void* w, void* out, const int* rows,
                            int n_out_rows, int d, float eps, float weight_offset, int act_dtype,
                            int w_dtype, int write_h, void* stream) {
    if (n_out_rows == 0) return 0;
    IMP_CHECK_ARG(h && w && out && d > 0, "imp_add_rmsnorm: bad argument");
    IMP_CHECK_ARG(!(rows && write_h), "imp_add_rmsnorm: write_h with a row list is not allowed");
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH(TA, TW)                                                                               \
    add_rmsnorm_kernel<TA, TW><<<n_out_rows, NORM_BLOCK, 0, s>>>(h, (const TA*)branch, (const TW*)w, \
                                                                 (TA*)out, rows, d, eps, weight_offset, write_h)
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
