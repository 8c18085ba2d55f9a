// Matrix product for a decode step: out[tokens, N] = A[tokens, K] . W[N, K]^T with at most 64 tokens,
// bfloat16 operands, 32-bit accumulation. The weights are the bulk of the bytes a decode step reads,
// and each is needed once: a warp streams 16 weight rows with 16-byte loads straight from global
// memory into tensor-core fragments (mma.sync m16n8k16, weights as the 16-row operand, tokens as the
// 8-column operand), the few activation rows come from L1/L2. No shared-memory staging, no waits.
//
// K order: within every block of 32 elements thread t of a quad holds elements 8t..8t+7 of its rows
// and feeds them to two instructions as their columns (2t, 2t+1, 2t+8, 2t+9); the activations are
// permuted the same way, so the sum over k is unchanged. A dot product is therefore accumulated in a
// fixed order that depends on K and on the split only: a row's result does not depend on the batch.
//
// Split over K: for narrow outputs (few row groups) the four warps of a CTA take a quarter of K each
// and are summed through shared memory in warp order. Epilogues as in gemm_tcgen05.cu.
// The reference's decode GEMV is a warp per output channel on CUDA cores (cpp/src/cuda/cuda_gemm.cu:47-78).
#include "common.cuh"

namespace {

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_F32 = 2, EPI_SWIGLU = 3 };
constexpr int WARPS = 4;

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg16(const __nv_bfloat16* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
// Weights are read once per step: do not let them push the activations out of L1.
__device__ __forceinline__ uint4 ldg16_stream(const __nv_bfloat16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// NT: token tiles of 8 (tokens <= 8*NT). KSPLIT: 1 (each warp its own 16 rows) or WARPS (the warps share
// 16 rows and split K). grid.x: groups of 16 rows per CTA = WARPS / KSPLIT.
template <int NT, int KSPLIT, int EPI>
__global__ void __launch_bounds__(WARPS * 32)
gemm_smallm_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                   const float* __restrict__ bias, void* __restrict__ out, int tokens, int n_out, int k_dim,
                   int lda, int ldo) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    constexpr int GROUPS = WARPS / KSPLIT;
    __shared__ float part[KSPLIT > 1 ? KSPLIT : 1][DUAL ? 2 : 1][NT][4][32];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int group = blockIdx.x * GROUPS + (KSPLIT > 1 ? 0 : warp);
    const int f0 = group * 16;
    const int ks = KSPLIT > 1 ? warp : 0;

    // K range of this warp, in blocks of 32
    const int blocks = k_dim / 32;                       // K % 32 == 0 is required by the launcher
    const int per = (blocks + KSPLIT - 1) / KSPLIT;
    const int kb_begin = ks * per, kb_end = min(blocks, kb_begin + per);

    float acc[NT][4], acc2[DUAL ? NT : 1][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
    if (DUAL) {
#pragma unroll
        for (int n = 0; n < (DUAL ? NT : 1); ++n) { acc2[n][0] = acc2[n][1] = acc2[n][2] = acc2[n][3] = 0.f; }
    }

    if (f0 < n_out) {
        // rows past the end are clamped (their results are not stored)
        const int r0 = min(f0 + g, n_out - 1), r1 = min(f0 + g + 8, n_out - 1);
        const __nv_bfloat16* w0 = W + (size_t)r0 * k_dim + 8 * t;
        const __nv_bfloat16* w1 = W + (size_t)r1 * k_dim + 8 * t;
        const __nv_bfloat16* u0 = W + (size_t)(n_out + r0) * k_dim + 8 * t;
        const __nv_bfloat16* u1 = W + (size_t)(n_out + r1) * k_dim + 8 * t;
        const __nv_bfloat16* a_row[NT];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int tok = n * 8 + g;
            a_row[n] = tok < tokens ? A + (size_t)tok * lda + 8 * t : nullptr;
        }
#pragma unroll 2
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            const int k0 = kb * 32;
            const uint4 wa = ldg16_stream(w0 + k0), wb = ldg16_stream(w1 + k0);
            uint4 ua, ub;
            if (DUAL) { ua = ldg16_stream(u0 + k0); ub = ldg16_stream(u1 + k0); }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                uint4 x = make_uint4(0u, 0u, 0u, 0u);
                if (a_row[n]) x = ldg16(a_row[n] + k0);
                mma_bf16(acc[n], wa.x, wb.x, wa.y, wb.y, x.x, x.y);
                mma_bf16(acc[n], wa.z, wb.z, wa.w, wb.w, x.z, x.w);
                if (DUAL) {
                    mma_bf16(acc2[n], ua.x, ub.x, ua.y, ub.y, x.x, x.y);
                    mma_bf16(acc2[n], ua.z, ub.z, ua.w, ub.w, x.z, x.w);
                }
            }
        }
    }

    if (KSPLIT > 1) {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                part[ks][0][n][e][lane] = acc[n][e];
                if (DUAL) part[ks][DUAL ? 1 : 0][n][e][lane] = acc2[DUAL ? n : 0][e];
            }
        __syncthreads();
        if (warp != 0) return;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float s = 0.f, s2 = 0.f;
#pragma unroll
                for (int w = 0; w < KSPLIT; ++w) {
                    s += part[w][0][n][e][lane];
                    if (DUAL) s2 += part[w][DUAL ? 1 : 0][n][e][lane];
                }
                acc[n][e] = s;
                if (DUAL) acc2[DUAL ? n : 0][e] = s2;
            }
    }
    if (f0 >= n_out) return;

    // accumulator element e of tile n: feature f0 + g + 8*(e/2), token n*8 + 2t + (e&1)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int f = f0 + g + 8 * (e >> 1), tok = n * 8 + 2 * t + (e & 1);
            if (f >= n_out || tok >= tokens) continue;
            const float x = acc[n][e] + (bias ? bias[f] : 0.f);
            const size_t o = (size_t)tok * ldo + f;
            if (EPI == EPI_STORE) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(x);
            else if (EPI == EPI_ADD) ((float*)out)[o] += x;
            else if (EPI == EPI_F32) ((float*)out)[o] = x;
            else ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(x / (1.0f + __expf(-x)) * acc2[DUAL ? n : 0][e]);
        }
}

template <int NT, int KSPLIT>
int launch_smallm(int epi, const void* A, const void* W, const float* bias, void* out, int tokens, int N, int K,
                  int lda, int ldo, cudaStream_t stream) {
    const int groups = ceil_div(N, 16);
    const int grid = ceil_div(groups, WARPS / KSPLIT);
#define L(E) gemm_smallm_kernel<NT, KSPLIT, E><<<grid, WARPS * 32, 0, stream>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, out, tokens, N, K, lda, ldo)
    switch (epi) {
        case EPI_STORE: L(EPI_STORE); break;
        case EPI_ADD: L(EPI_ADD); break;
        case EPI_F32: L(EPI_F32); break;
        case EPI_SWIGLU: L(EPI_SWIGLU); break;
        default: nib_set_error("gemm (small M): unknown epilogue %d", epi); return 1;
    }
#undef L
    NIB_LAUNCH_CHECK();
    return 0;
}

template <int NT>
int launch_smallm_split(int ksplit, int epi, const void* A, const void* W, const float* bias, void* out, int tokens,
                        int N, int K, int lda, int ldo, cudaStream_t stream) {
    if (ksplit > 1) return launch_smallm<NT, WARPS>(epi, A, W, bias, out, tokens, N, K, lda, ldo, stream);
    return launch_smallm<NT, 1>(epi, A, W, bias, out, tokens, N, K, lda, ldo, stream);
}

}  // namespace

// 1 if the kernel takes these operands: at most 64 tokens, K a multiple of 32, 16-byte aligned rows.
NIB_API int nib_gemm_smallm_supported(const void* A, const void* W, int tokens, int K, int lda) {
    if (tokens <= 0 || tokens > 64 || K <= 0 || K % 32 || lda % 8) return 0;
    return (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) ? 0 : 1;
}

// Same operands and epilogues as nib_gemm_tc. ksplit: 0 = chosen here, 1, or 4.
NIB_API int nib_gemm_smallm(const void* A, const void* W, const float* bias, void* out, int tokens, int N, int K,
                            int lda, int ldo, int epi, int ksplit, cudaStream_t stream) {
    NIB_REQUIRE(N > 0 && lda >= K && ldo >= N, "gemm (small M): bad sizes tokens=%d N=%d K=%d", tokens, N, K);
    NIB_REQUIRE(nib_gemm_smallm_supported(A, W, tokens, K, lda), "gemm (small M): needs 1..64 tokens, K %% 32 == 0 and 16-byte aligned rows (tokens=%d K=%d)", tokens, K);
    NIB_REQUIRE(epi != EPI_SWIGLU || bias == nullptr, "gemm (small M): the swiglu epilogue takes no bias");
    if (ksplit == 0) ksplit = (ceil_div(N, 16) < 4 * 148 && K >= 512) ? WARPS : 1;
    NIB_REQUIRE(ksplit == 1 || ksplit == WARPS, "gemm (small M): ksplit must be 1 or %d", WARPS);
    if (tokens <= 8) return launch_smallm_split<1>(ksplit, epi, A, W, bias, out, tokens, N, K, lda, ldo, stream);
    if (tokens <= 16) return launch_smallm_split<2>(ksplit, epi, A, W, bias, out, tokens, N, K, lda, ldo, stream);
    if (tokens <= 32) return launch_smallm_split<4>(ksplit, epi, A, W, bias, out, tokens, N, K, lda, ldo, stream);
    return launch_smallm_split<8>(ksplit, epi, A, W, bias, out, tokens, N, K, lda, ldo, stream);
}
