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

IMP_TL_DEFINE(norm)

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
// with 16-byte loads issued together, kept in registers (NV float4 a thread: 1, 2, 4 or 8, the least that
// holds the row, so that narrow rows leave room for more blocks on an SM), and written from there.  The per-thread
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

// SPLIT: the branch has not been summed yet.  `part` holds n_splits 32-bit partial results [n_rows_total, d] of a
// product whose contraction was cut over CTAs, split_stride floats apart; the branch value is their sum in split
// order rounded to TA, bit for bit what the summing kernel would have stored.
template <typename TA, typename TW, bool SPLIT, int NV>
__global__ void __launch_bounds__(NORM_BLOCK) add_rmsnorm_vec_kernel(float* __restrict__ h, const TA* __restrict__ branch,
                                                                     const TW* __restrict__ w, TA* __restrict__ out,
                                                                     const int* __restrict__ rows, int d, float eps,
                                                                     float weight_offset, int write_h,
                                                                     const float* __restrict__ part, int64_t split_stride,
                                                                     int n_splits) {
    IMP_TL_BEGIN(6)
    pdl_wait();
    IMP_TL_WAITED()
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = rows ? rows[r] : r;
    float* hrow = h + src * d;
    const TA* brow = (SPLIT || branch) ? branch + src * d : nullptr;   // with SPLIT only its null-ness is used
    const int nv = d >> 2;
    float4 v[NV], wv[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * NORM_BLOCK;
        if (c < nv) {
            v[i] = Vec4<float>::load(hrow + 4 * c);
            wv[i] = Vec4<TW>::load(w + 4 * c);     // with the row, not after the sum: one trip to the L2 less on the way
        }
    }
    if (SPLIT) {
        const float* prow = part + src * d;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = threadIdx.x + i * NORM_BLOCK;
            if (c < nv) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                constexpr int NB = 8;                 // parts requested together, added in split order
                for (int s0 = 0; s0 < n_splits; s0 += NB) {
                    float4 b[NB];
#pragma unroll
                    for (int j = 0; j < NB; ++j)
                        if (s0 + j < n_splits) b[j] = Vec4<float>::load(prow + (s0 + j) * split_stride + 4 * c);
#pragma unroll
                    for (int j = 0; j < NB; ++j)
                        if (s0 + j < n_splits) { acc.x += b[j].x; acc.y += b[j].y; acc.z += b[j].z; acc.w += b[j].w; }
                }
                v[i].x += to_float(from_float<TA>(acc.x));
                v[i].y += to_float(from_float<TA>(acc.y));
                v[i].z += to_float(from_float<TA>(acc.z));
                v[i].w += to_float(from_float<TA>(acc.w));
            }
        }
    } else if (brow) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = threadIdx.x + i * NORM_BLOCK;
            if (c < nv) {
                const float4 b = Vec4<TA>::load(brow + 4 * c);
                v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
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
    for (int i = 0; i < NV; ++i) {
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
    IMP_TL_END()
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
// the vector kernel with the fewest float4 a thread that hold a row of d floats
#define VEC_BY_WIDTH(TA, TW, SPLIT, BRANCH, PART, STRIDE, NSPLITS)                                               \
    do {                                                                                                         \
        const int per_thread = (d / 4 + NORM_BLOCK - 1) / NORM_BLOCK;                                            \
        if (per_thread <= 1)                                                                                     \
            imp_launch(add_rmsnorm_vec_kernel<TA, TW, SPLIT, 1>, dim3(n_out_rows), dim3(NORM_BLOCK), 0, s, h,    \
                       BRANCH, (const TW*)w, (TA*)out, rows, d, eps, weight_offset, write_h, PART, STRIDE, NSPLITS); \
        else if (per_thread <= 2)                                                                                \
            imp_launch(add_rmsnorm_vec_kernel<TA, TW, SPLIT, 2>, dim3(n_out_rows), dim3(NORM_BLOCK), 0, s, h,    \
                       BRANCH, (const TW*)w, (TA*)out, rows, d, eps, weight_offset, write_h, PART, STRIDE, NSPLITS); \
        else if (per_thread <= 4)                                                                                \
            imp_launch(add_rmsnorm_vec_kernel<TA, TW, SPLIT, 4>, dim3(n_out_rows), dim3(NORM_BLOCK), 0, s, h,    \
                       BRANCH, (const TW*)w, (TA*)out, rows, d, eps, weight_offset, write_h, PART, STRIDE, NSPLITS); \
        else                                                                                                     \
            imp_launch(add_rmsnorm_vec_kernel<TA, TW, SPLIT, 8>, dim3(n_out_rows), dim3(NORM_BLOCK), 0, s, h,    \
                       BRANCH, (const TW*)w, (TA*)out, rows, d, eps, weight_offset, write_h, PART, STRIDE, NSPLITS); \
    } while (0)

#define LAUNCH(TA, TW)                                                                                     \
    do {                                                                                                   \
        if (vec)                                                                                           \
            VEC_BY_WIDTH(TA, TW, false, (const TA*)branch, (const float*)nullptr, (int64_t)0, 0);          \
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

// The unsummed branch for few rows: one row is shared by a cluster of CTAs, 512 columns each (a thread holds
// one float4, or two for rows of more than 4096 columns), so that the n_splits partial rows are fetched by
// enough threads at once.  Each CTA adds up its squares, stores the sum into every CTA of the cluster (shared
// memory of the cluster), and after one cluster barrier all of them add the same numbers in rank order.
constexpr int CN_THREADS = 128, CN_MAX_C = 8, CN_MAX_V = 2;

template <typename TA, typename TW>
__global__ void __launch_bounds__(CN_THREADS) add_rmsnorm_split_cluster_kernel(
    float* __restrict__ h, const TW* __restrict__ w, TA* __restrict__ out, const int* __restrict__ rows, int d, float eps,
    float weight_offset, int write_h, const float* __restrict__ part, int64_t split_stride, int n_splits) {
    __shared__ float scratch[33];
    __shared__ float slots[CN_MAX_C];
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int C = gridDim.x;
    // first half of "every CTA of the cluster is running"; the wait stands before the first remote store
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    IMP_TL_BEGIN(4)
    pdl_wait();
    IMP_TL_WAITED()
    pdl_launch_dependents();
    const int r = blockIdx.y;
    const int64_t src = rows ? rows[r] : r;
    float* hrow = h + src * d;
    const float* prow = part + src * d;
    const int nv = d >> 2;
    float4 v[CN_MAX_V], wv[CN_MAX_V];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < CN_MAX_V; ++i) {
        const int c = (int)rank * CN_THREADS + threadIdx.x + i * C * CN_THREADS;
        if (c < nv) {
            v[i] = Vec4<float>::load(hrow + 4 * c);
            wv[i] = Vec4<TW>::load(w + 4 * c);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            const float* p = prow + 4 * c;
            // up to twelve partial rows requested together (one trip to the L2 for the usual 6 to 9 splits), added in
            // split order
            constexpr int NB = 12;
            for (int sp0 = 0; sp0 < n_splits; sp0 += NB) {
                float4 b[NB];
#pragma unroll
                for (int j = 0; j < NB; ++j)
                    if (sp0 + j < n_splits) b[j] = Vec4<float>::load(p + (sp0 + j) * split_stride);
#pragma unroll
                for (int j = 0; j < NB; ++j)
                    if (sp0 + j < n_splits) { acc.x += b[j].x; acc.y += b[j].y; acc.z += b[j].z; acc.w += b[j].w; }
            }
            v[i].x += to_float(from_float<TA>(acc.x));
            v[i].y += to_float(from_float<TA>(acc.y));
            v[i].z += to_float(from_float<TA>(acc.z));
            v[i].w += to_float(from_float<TA>(acc.w));
            if (write_h) Vec4<float>::store(hrow + 4 * c, v[i]);
            ss += v[i].x * v[i].x;
            ss += v[i].y * v[i].y;
            ss += v[i].z * v[i].z;
            ss += v[i].w * v[i].w;
        }
    }
    ss = block_sum(ss, scratch);
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (threadIdx.x < C) {
        const uint32_t local = (uint32_t)__cvta_generic_to_shared(&slots[rank]);
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((uint32_t)threadIdx.x));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(ss) : "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    float total = 0.f;
    for (int k = 0; k < C; ++k) total += slots[k];
    const float inv = rsqrtf(total / (float)d + eps);
    TA* orow = out + (int64_t)r * d;
#pragma unroll
    for (int i = 0; i < CN_MAX_V; ++i) {
        const int c = (int)rank * CN_THREADS + threadIdx.x + i * C * CN_THREADS;
        if (c < nv) {
            float4 o;
            o.x = v[i].x * inv * (wv[i].x + weight_offset);
            o.y = v[i].y * inv * (wv[i].y + weight_offset);
            o.z = v[i].z * inv * (wv[i].z + weight_offset);
            o.w = v[i].w * inv * (wv[i].w + weight_offset);
            Vec4<TA>::store(orow + 4 * c, o);
        }
    }
    IMP_TL_END()
}

template <typename TA, typename TW>
static cudaError_t launch_split_cluster(int C, int n_out_rows, cudaStream_t s, float* h, const void* w, void* out, const int* rows,
                                        int d, float eps, float weight_offset, int write_h, const float* part,
                                        int64_t split_stride, int n_splits) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(C, n_out_rows);
    cfg.blockDim = dim3(CN_THREADS);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = imp_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, add_rmsnorm_split_cluster_kernel<TA, TW>, h, (const TW*)w, (TA*)out, rows, d, eps,
                              weight_offset, write_h, part, split_stride, n_splits);
}

// h += (sum of the n_splits partial results, rounded to the activation type); out = rmsnorm(h) * (w + offset).
// part: [n_splits][n_rows_total, d] 32-bit, split_stride floats apart.  IMP_ERR_UNSUPPORTED for widths the
// register-resident kernel does not take (the caller then sums first).
IMP_API int imp_add_rmsnorm_split(float* h, const float* part, int64_t split_stride, int n_splits, const void* w, void* out,
                                  const int* rows, int n_out_rows, int d, float eps, float weight_offset, int act_dtype,
                                  int w_dtype, int write_h, void* stream) {
    if (n_out_rows == 0) return 0;
    IMP_CHECK_ARG(h && part && w && out && d > 0 && n_splits >= 1, "imp_add_rmsnorm_split: bad argument");
    IMP_CHECK_ARG(!(rows && write_h), "imp_add_rmsnorm_split: write_h with a row list is not allowed");
    if (!(d % 4 == 0 && d <= NORM_BLOCK * NORM_MAX_V4 * 4 && (uintptr_t)h % 16 == 0 && (uintptr_t)w % 16 == 0 &&
          (uintptr_t)out % 16 == 0 && (uintptr_t)part % 16 == 0 && split_stride % 4 == 0))
        return IMP_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    static int use_cluster = -1;    // IMP_B200_NORM_CLUSTER=0: one CTA per row whatever the number of rows
    if (use_cluster < 0) { const char* e = getenv("IMP_B200_NORM_CLUSTER"); use_cluster = e ? atoi(e) : 1; }
    if (use_cluster && n_out_rows <= 128 && d >= 1024) {
        // a row over several CTAs while the rows alone would leave most of the device idle
        const int nv = d / 4;
        int C = (nv + CN_THREADS - 1) / CN_THREADS;
        if (C > CN_MAX_C) C = CN_MAX_C;
        if (nv <= C * CN_THREADS * CN_MAX_V) {
            cudaError_t e;
            if (act_dtype == IMP_F32 && w_dtype == IMP_F32)
                e = launch_split_cluster<float, float>(C, n_out_rows, s, h, w, out, rows, d, eps, weight_offset, write_h, part, split_stride, n_splits);
            else if (act_dtype == IMP_F32)
                e = launch_split_cluster<float, __nv_bfloat16>(C, n_out_rows, s, h, w, out, rows, d, eps, weight_offset, write_h, part, split_stride, n_splits);
            else if (w_dtype == IMP_F32)
                e = launch_split_cluster<__nv_bfloat16, float>(C, n_out_rows, s, h, w, out, rows, d, eps, weight_offset, write_h, part, split_stride, n_splits);
            else
                e = launch_split_cluster<__nv_bfloat16, __nv_bfloat16>(C, n_out_rows, s, h, w, out, rows, d, eps, weight_offset, write_h, part, split_stride, n_splits);
            if (e != cudaSuccess) { imp_set_error("imp_add_rmsnorm_split: %s", cudaGetErrorString(e)); return (int)e; }
            return 0;
        }
    }
#define LAUNCH(TA, TW) VEC_BY_WIDTH(TA, TW, true, (const TA*)out, part, split_stride, n_splits)
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
