// Shared helpers of the kernel library. Every exported function is extern "C", takes raw device
// pointers and a stream, allocates nothing, and returns 0 or a non-zero code whose text
// nib_last_error() gives.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstring>

#define NIB_API extern "C" __attribute__((visibility("default")))

enum NibDType : int { NIB_F32 = 0, NIB_BF16 = 1 };

// Sets the message that nib_last_error() returns (thread-local).
void nib_set_error(const char* fmt, ...);

#define NIB_REQUIRE(cond, ...)            \
    do {                                  \
        if (!(cond)) {                    \
            nib_set_error(__VA_ARGS__);   \
            return 1;                     \
        }                                 \
    } while (0)

#define NIB_CUDA(call)                                                              \
    do {                                                                            \
        cudaError_t e__ = (call);                                                   \
        if (e__ != cudaSuccess) {                                                   \
            nib_set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__),  \
                          __FILE__, __LINE__);                                      \
            return 2;                                                               \
        }                                                                           \
    } while (0)

#define NIB_LAUNCH_CHECK() NIB_CUDA(cudaGetLastError())

template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

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

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Programmatic dependent launch: a kernel launched with launch_pdl may begin while the kernel before it
// in the stream is still running; it must call pdl_wait() before it reads anything that kernel (or any
// earlier one) wrote and before its first write to global memory. What it does before that (index
// arithmetic, loads of weights and of inputs that no kernel writes) overlaps the other kernel's tail.
// In a launch without the attribute both calls do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

bool nib_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
    cfg.numAttrs = nib_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- timeline of a step -------------------------------------------------------------------------------
// Kernels that overlap through programmatic dependent launch cannot be timed from outside (an event between two
// of them would end the overlap). When a trace buffer is set (nib_trace_set), thread 0 of the first CTA of a
// kernel notes the GPU's nanosecond timer at a few points of its life: 0 entry, 1 after the wait for the
// earlier kernels, 2 its results written. buf[0] counts the notes; note i is buf[1 + 2i] = kernel id << 8 | phase
// and buf[2 + 2i] = time. Without a buffer a launch passes nullptr and the kernel does one predictable branch.
enum NibTraceKernel : int {
    NIB_TK_EMBED = 1, NIB_TK_RMSNORM = 2, NIB_TK_ROPE = 3, NIB_TK_GEMM_SMALLM = 4, NIB_TK_GEMM_STREAM = 5,
    NIB_TK_GEMM_TC = 6, NIB_TK_ATTN_DECODE = 7, NIB_TK_ATTN_COMBINE = 8, NIB_TK_ARGMAX = 9, NIB_TK_ATTN_DECODE_MMA = 10,
    NIB_TK_GEMM_PAIR = 11, NIB_TK_ATTN_PREFILL = 12,
};
unsigned long long* nib_trace_buffer();      // nullptr unless a trace is being taken
int nib_trace_capacity();

__device__ __forceinline__ void nib_trace_mark(unsigned long long* buf, int cap, int kernel, int tag, int phase) {
    if (buf == nullptr || (blockIdx.x | blockIdx.y | blockIdx.z) != 0) return;
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
    const unsigned long long i = atomicAdd(buf, 1ULL);
    if ((int)i < cap) {
        buf[1 + 2 * i] = ((unsigned long long)kernel << 16) | ((unsigned long long)(tag & 0xff) << 8) | (unsigned long long)phase;
        buf[2 + 2 * i] = now;
    }
}
