// Error text and device queries of the kernel library.
#include "common.cuh"
#include <cstdarg>

static thread_local char g_error[512] = "";

void nib_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

NIB_API const char* nib_last_error() { return g_error; }

NIB_API int nib_abi_version() { return 1; }

// Compute capability of the current device as major * 10 + minor, or a negative CUDA error.
NIB_API int nib_device_arch() {
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return -1;
    return major * 10 + minor;
}

NIB_API int nib_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return n;
}

// Programmatic dependent launch of the decode kernels: on unless switched off (nib_set_pdl(0)).
static int g_pdl = 1;
bool nib_pdl_enabled() { return g_pdl != 0; }
NIB_API void nib_set_pdl(int on) { g_pdl = on; }
