// Error text of the last failed launcher call, device queries, and the status word helpers.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

static thread_local char g_last_error[512] = "";

void imp_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

IMP_API const char* imp_last_error(void) { return g_last_error; }

int imp_pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) enabled = getenv("IMP_B200_NO_PDL") ? 0 : 1;
    return enabled;
}

IMP_API int imp_abi_version(void) { return 1; }

// Compute capability of the current device as major*10+minor, or a negative CUDA error.
IMP_API int imp_device_arch(void) {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) {
        imp_set_error("imp_device_arch: %s", cudaGetErrorString(e));
        return -(int)e;
    }
    return major * 10 + minor;
}

IMP_API int imp_device_sm_count(void) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return n;
}

int imp_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 1;
    if (dev < 64 && cached[dev] > 0) return cached[dev];
    const int n = imp_device_sm_count();
    if (n <= 0) return 1;
    if (dev < 64) cached[dev] = n;
    return n;
}

const char* imp_status_name(int code) {
    switch (code) {
        case IMP_OK: return "ok";
        case IMP_BAD_TOKEN_ID: return "token id outside the vocabulary";
        case IMP_BAD_PAGE: return "page id outside the cache pool";
        case IMP_BAD_POSITION: return "position outside the position table or the block table";
        case IMP_BAD_SEQUENCE: return "token names a sequence outside the batch";
        case IMP_WAIT_TIMEOUT: return "a bounded device-side wait ran out";
        default: return "unknown status";
    }
}

IMP_API const char* imp_status_string(int code) { return imp_status_name(code); }
