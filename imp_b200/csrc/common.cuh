// Shared helpers of the sm_100a kernels: element types, loads/stores through
// float, block reductions with a fixed order, and the device status word.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define IMP_API extern "C" __attribute__((visibility("default")))

// Element type codes used across the C ABI.
enum ImpDType : int { IMP_F32 = 0, IMP_BF16 = 1 };

// Codes written to the device status word (first error wins; 0 = ok).
enum ImpStatus : int {
    IMP_OK = 0,
    IMP_BAD_TOKEN_ID = 1,      // embedding: id outside [0, vocab)
    IMP_BAD_PAGE = 2,          // cache write / attention: page id outside the pool
    IMP_BAD_POSITION = 3,      // position outside the rotary table or the block table
    IMP_BAD_SEQUENCE = 4,      // token names a sequence outside the batch
    IMP_WAIT_TIMEOUT = 5,      // a bounded device-side wait ran out
};

// Host-side error codes returned by launchers (negative = argument errors, positive = cudaError_t).
#define IMP_ERR_ARG (-1)
#define IMP_ERR_UNSUPPORTED (-2)

void imp_set_error(const char* fmt, ...);
// Streaming multiprocessors of the current device (asked once per device); launch heuristics size their
// grids by it.  1 when the device cannot be asked: the launch that follows reports the real error.
int imp_sm_count();

#define IMP_CHECK_ARG(cond, ...)            \
    do {                                    \
        if (!(cond)) {                      \
            imp_set_error(__VA_ARGS__);     \
            return IMP_ERR_ARG;             \
        }                                   \
    } while (0)

#define IMP_RETURN_LAUNCH()                                            \
    do {                                                               \
        cudaError_t e__ = cudaGetLastError();                          \
        if (e__ != cudaSuccess) {                                      \
            imp_set_error("%s: %s", __func__, cudaGetErrorString(e__)); \
            return (int)e__;                                           \
        }                                                              \
        return 0;                                                      \
    } while (0)

// ---- programmatic dependent launch -------------------------------------------------------------
// Every kernel of this library starts with pdl_wait() before it touches memory an earlier kernel
// of the stream may have written, and calls pdl_launch_dependents() so that the next kernel's
// blocks may become resident while this one still runs (they stop at their own pdl_wait()).
// Launched without the attribute (or after a kernel of another library) both are no-ops.
// Kernels call the two in the order wait, launch_dependents.  With IMP_PDL_EARLY (the default) the
// trigger is issued by pdl_wait() itself, before the wait: the next kernel's blocks may then become
// resident (and fetch what does not depend on earlier kernels, e.g. weights) while the kernel before
// this one still runs.  That is safe because every kernel waits for its own predecessor before it
// touches anything an earlier kernel wrote, and completion is transitive along the stream.
#ifndef IMP_PDL_EARLY
#define IMP_PDL_EARLY 1
#endif
__device__ __forceinline__ void pdl_wait() {
#if IMP_PDL_EARLY
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
#if !IMP_PDL_EARLY
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

// ---- timeline of a step (diagnostic build only) ---------------------------------------------------
// -DIMP_TIMELINE: thread 0 of every CTA of the kernels that carry the three marks below records the global timer
// at its start, after its wait for the kernel before it, and at its end, with the SM it ran on.  A file that uses the
// marks says IMP_TL_DEFINE(name) once: that makes its record buffer and the setter imp_tl_set_<name>(records, capacity,
// counter).  A record is four 64-bit words: kernel << 48 | sm << 32 | CTA, then the three times in ns.  Without the
// flag (every product build) the marks are empty.
#ifdef IMP_TIMELINE
struct ImpTl { unsigned long long* buf; unsigned cap; unsigned* count; };
__device__ __forceinline__ unsigned long long imp_tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define IMP_TL_DEFINE(name)                                                                                       \
    static __device__ ImpTl g_imp_tl;                                                                             \
    IMP_API int imp_tl_set_##name(void* buf, unsigned cap, void* count) {                                         \
        ImpTl h{(unsigned long long*)buf, cap, (unsigned*)count};                                                 \
        return (int)cudaMemcpyToSymbol(g_imp_tl, &h, sizeof h);                                                   \
    }
#define IMP_TL_BEGIN(kernel_id)                                                                                   \
    const bool tl_on = threadIdx.x == 0 && threadIdx.y == 0 && g_imp_tl.buf != nullptr;                           \
    const int tl_kernel = (kernel_id);                                                                            \
    unsigned long long tl_t0 = 0, tl_t1 = 0;                                                                      \
    if (tl_on) tl_t0 = tl_t1 = imp_tl_now();
#define IMP_TL_WAITED() if (tl_on) tl_t1 = imp_tl_now();
#define IMP_TL_END()                                                                                              \
    if (tl_on) {                                                                                                  \
        const unsigned long long t2 = imp_tl_now();                                                               \
        const unsigned i = atomicAdd(g_imp_tl.count, 1u);                                                         \
        if (i < g_imp_tl.cap) {                                                                                   \
            unsigned sm;                                                                                          \
            asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));                                                       \
            const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);                  \
            unsigned long long* r = g_imp_tl.buf + 4ull * i;                                                      \
            r[0] = ((unsigned long long)tl_kernel << 48) | ((unsigned long long)sm << 32) | cta;                  \
            r[1] = tl_t0; r[2] = tl_t1; r[3] = t2;                                                                \
        }                                                                                                         \
    }
#else
#define IMP_TL_DEFINE(name)
#define IMP_TL_BEGIN(kernel_id)
#define IMP_TL_WAITED()
#define IMP_TL_END()
#endif

// 1 unless the environment variable IMP_B200_NO_PDL is set (read once).
int imp_pdl_enabled();

// Launch with the programmatic-stream-serialization attribute (when enabled).
template <typename... KArgs, typename... Args>
inline cudaError_t imp_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = imp_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// -DIMP_TAG_STATUS (a diagnostic build): a reported code carries 100 x the tag of the check that raised it.
#ifdef IMP_TAG_STATUS
#define IMP_TAGGED(code, tag) ((code) + 100 * (tag))
#else
#define IMP_TAGGED(code, tag) (code)
#endif
__device__ __forceinline__ void imp_report(int* status, int code) {
    if (status) atomicCAS(status, 0, code);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Load element i of a buffer whose element type is only known at run time.
__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
    return dtype == IMP_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; every thread gets the result.  The order of additions is
// fixed by blockDim alone, so a row reduces the same way in every batch.
// `scratch` holds at least 33 floats.  blockDim.x must be a multiple of 32.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
