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

// cuTensorMapEncodeTiled, looked up once through the runtime; nullptr if this driver does not offer it.
#include "pipeline.cuh"
NibEncodeTiledFn nib_tensor_map_encoder() {
    static NibEncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (NibEncodeTiledFn)p;
    }
    return fn;
}

// The trace buffer of nib_trace_mark: device memory of 1 + 2 * capacity 64-bit words, zeroed by the caller.
static unsigned long long* g_trace_buf = nullptr;
static int g_trace_cap = 0;
unsigned long long* nib_trace_buffer() { return g_trace_buf; }
int nib_trace_capacity() { return g_trace_cap; }
NIB_API void nib_trace_set(void* buf, int capacity) {
    g_trace_buf = static_cast<unsigned long long*>(buf);
    g_trace_cap = buf ? capacity : 0;
}
