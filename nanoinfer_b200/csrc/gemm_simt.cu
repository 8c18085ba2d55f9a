// The general matrix product of the engine: C[M,N] = A[M,K] . W[N,K]^T (+ bias), any M, N, K,
// 32-bit accumulation on the CUDA cores. It is the true 32-bit path (no reduced-precision matrix
// mode) and the fallback of the bfloat16 path for shapes the tensor-core kernel refuses.
//
// Every output element is accumulated by one thread over k = 0..K-1 in ascending order, so a row's
// result does not depend on how many other rows the call has (the reference guarantees the same:
// cpp/src/cuda/cuda_gemm.cu:37-45). Tiling after cpp/src/cuda/cuda_gemm.cu:80-150 in spirit only.
//
// Epilogues: STORE (T out = acc + bias), ADD (float out += acc + bias: the residual sum),
// F32 (float out = acc + bias: logits), SWIGLU (two accumulators, W rows n and n + N:
// T out = silu(gate) * up, silu(g) = g / (1 + exp(-g)), cpp/src/ops.cpp:86-93).
#include "common.cuh"

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_F32 = 2, EPI_SWIGLU = 3 };

template <typename T, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, const float* __restrict__ bias,
                 void* __restrict__ out, int M, int N, int K, int lda, int ldo) {
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    __shared__ float Us[DUAL ? BK : 1][DUAL ? BN + 1 : 1];

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;     // thread's 4x4 micro tile: rows ty*4.., cols tx*4..
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    float acc[TM][TN];
    float acc2[DUAL ? TM : 1][DUAL ? TN : 1];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    if (DUAL) {
#pragma unroll
        for (int i = 0; i < (DUAL ? TM : 1); ++i)
#pragma unroll
            for (int j = 0; j < (DUAL ? TN : 1); ++j) acc2[i][j] = 0.f;
    }

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, kk = e % BK;
            const int gk = k0 + kk;
            float a = 0.f, w = 0.f, u = 0.f;
            if (gk < K) {
                if (m0 + r < M) a = Elem<T>::load(A + (size_t)(m0 + r) * lda + gk);
                if (n0 + r < N) {
                    w = Elem<T>::load(W + (size_t)(n0 + r) * K + gk);
                    if (DUAL) u = Elem<T>::load(W + (size_t)(N + n0 + r) * K + gk);
                }
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
            if (DUAL) Us[kk][r] = u;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
            if (DUAL) {
                float u[TN];
#pragma unroll
                for (int j = 0; j < TN; ++j) u[j] = Us[kk][tx * TN + j];
#pragma unroll
                for (int i = 0; i < (DUAL ? TM : 1); ++i)
#pragma unroll
                    for (int j = 0; j < (DUAL ? TN : 1); ++j) acc2[i][j] = fmaf(a[i], u[j], acc2[i][j]);
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j] + (bias ? bias[n] : 0.f);
            const size_t o = (size_t)m * ldo + n;
            if (EPI == EPI_STORE) {
                Elem<T>::store((T*)out + o, v);
            } else if (EPI == EPI_ADD) {
                ((float*)out)[o] += v;
            } else if (EPI == EPI_F32) {
                ((float*)out)[o] = v;
            } else {
                const float g = v, u = acc2[DUAL ? i : 0][DUAL ? j : 0];
                Elem<T>::store((T*)out + o, g / (1.0f + expf(-g)) * u);
            }
        }
    }
}

template <typename T>
static int launch_simt(const void* A, const void* W, const float* bias, void* out, int M, int N, int K,
                       int lda, int ldo, int epi, cudaStream_t stream) {
    dim3 grid(ceil_div(N, 64), ceil_div(M, 64));
    dim3 block(256);
    switch (epi) {
        case EPI_STORE: gemm_simt_kernel<T, EPI_STORE><<<grid, block, 0, stream>>>((const T*)A, (const T*)W, bias, out, M, N, K, lda, ldo); break;
        case EPI_ADD: gemm_simt_kernel<T, EPI_ADD><<<grid, block, 0, stream>>>((const T*)A, (const T*)W, bias, out, M, N, K, lda, ldo); break;
        case EPI_F32: gemm_simt_kernel<T, EPI_F32><<<grid, block, 0, stream>>>((const T*)A, (const T*)W, bias, out, M, N, K, lda, ldo); break;
        case EPI_SWIGLU: gemm_simt_kernel<T, EPI_SWIGLU><<<grid, block, 0, stream>>>((const T*)A, (const T*)W, bias, out, M, N, K, lda, ldo); break;
        default: nib_set_error("gemm: unknown epilogue %d", epi); return 1;
    }
    NIB_LAUNCH_CHECK();
    return 0;
}

// A [M, K] with row stride lda; W [N, K] (SWIGLU: [2N, K], gate rows then up rows); out [M, N] with
// row stride ldo. epi: 0 store, 1 add into float, 2 store float, 3 swiglu.
NIB_API int nib_gemm_simt(const void* A, const void* W, const float* bias, void* out, int M, int N, int K,
                          int lda, int ldo, int epi, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(M >= 0 && N > 0 && K > 0 && lda >= K && ldo >= N, "gemm: bad sizes M=%d N=%d K=%d lda=%d ldo=%d", M, N, K, lda, ldo);
    NIB_REQUIRE(epi != EPI_SWIGLU || bias == nullptr, "gemm: the swiglu epilogue takes no bias");
    if (M == 0) return 0;
    NIB_REQUIRE(ceil_div(M, 64) <= 65535, "gemm: M=%d is too large for one launch", M);
    if (dtype == NIB_F32) return launch_simt<float>(A, W, bias, out, M, N, K, lda, ldo, epi, stream);
    if (dtype == NIB_BF16) return launch_simt<__nv_bfloat16>(A, W, bias, out, M, N, K, lda, ldo, epi, stream);
    NIB_REQUIRE(false, "gemm: unknown dtype %d", dtype);
}
