// Matrix product for a decode step: out[tokens, N] = A[tokens, K] . W[N, K]^T with at most 64 tokens,
// bfloat16 operands, 32-bit accumulation. The weights are the bulk of the bytes a decode step reads,
// and each is needed once: a warp streams 16 weight rows with 16-byte loads straight from global
// memory into tensor-core fragments (mma.sync m16n8k16, weights as the 16-row operand, tokens as the
// 8-column operand), the few activation rows come from L1/L2. No shared-memory staging, no waits.
//
// K order: within every block of 32 elements thread t of a quad holds elements 8t..8t+7 of its rows
// and feeds them to two instructions as their columns (2t, 2t+1, 2t+8, 2t+9); the activations are
// permuted the same way, so the sum over k is unchanged.
//
// Parallelism. Wide outputs (the head: thousands of 16-row groups): one warp per group, whole K.
// Narrow outputs: the eight warps of a CTA take an eighth of K each (summed through shared memory in
// warp order), and `cross` CTAs split K further: each writes its partial tile to scratch memory, the
// CTA that arrives last at the group's counter adds the partials IN SPLIT ORDER and runs the
// epilogue, then resets the counter. The order of every sum is fixed by (K, splits) alone, so a
// row's result does not depend on the batch and is the same from run to run.
//
// Fused RMSNorm (NORM): the A operand is the 32-bit residual stream x. Since
// sum_k w[f,k] * (x[k] * s * g[k]) = s * sum_k w[f,k] * (x[k] * g[k]) with s = 1/sqrt(mean(x^2) + eps),
// the fragments are built from bfloat16(x * gain), the sum of x^2 is accumulated from the very values
// that are loaded for them (every element of a row is loaded by exactly one thread of the K split),
// reduced along with the accumulators, and s multiplies the accumulator in the epilogue: the norm
// costs no extra pass over the row and no extra wait.
//
// Epilogues as in gemm_tcgen05.cu. The reference's decode GEMV is a warp per output channel on CUDA
// cores (cpp/src/cuda/cuda_gemm.cu:47-78); its RMSNorm is a separate kernel with one thread per row
// (cpp/src/cuda/cuda_elementwise.cu:36-46).
#include "common.cuh"

namespace {

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_F32 = 2, EPI_SWIGLU = 3, EPI_QKV = 4 };
constexpr int WARPS = 8;
constexpr int MAX_TOKENS = 64;

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Weights are read once per step: do not let them push the activations out of L1.
__device__ __forceinline__ uint4 ldg16_stream(const __nv_bfloat16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// The q/k/v epilogue (EPI_QKV): the product's rows are [q heads | k heads | v heads] of head_dim each. A group of 16
// rows is cut so that the rotated dimension d of a query or key head (rows g of the group) and its partner d + rot/2
// (rows g + 8) are the two halves of one thread's accumulator: the rotation needs no exchange between threads.
// After bias and rotation the whole row goes to the activation buffer, and (writes) the rotated key and the value
// into the slot of the token's position in its request's page.
struct QkvEpi {
    int heads, kv_heads, head_dim, rot;
    const int* positions; const int* req_index; const float* cos_t; const float* sin_t;
    const int* block_table; int bt_stride, page_size, num_pages;
    __nv_bfloat16* k_pages; __nv_bfloat16* v_pages; int writes;
};

// First rows of the two halves of row group `group` in the q/k/v form.
__device__ __forceinline__ void qkv_group_rows(const QkvEpi& q, int group, int& a, int& b) {
    const int per_head = q.head_dim >> 4;
    const int hs = group / per_head, i = group - hs * per_head;
    const int base = hs * q.head_dim;
    if (hs < q.heads + q.kv_heads && i < (q.rot >> 4)) { a = base + i * 8; b = a + (q.rot >> 1); }
    else { a = base + i * 16; b = a + 8; }
}

// NT: token tiles of 8. KSPLIT: 1 (each warp its own 16 rows, whole K) or WARPS (the warps of a CTA
// share 16 rows and split K; gridDim.y CTAs split K further). grid.x: CTAs over the row groups.
template <int NT, int KSPLIT, int EPI, bool NORM>
__global__ void __launch_bounds__(WARPS * 32, 2)      // two CTAs per SM: a projection's 300 row groups fit one wave
gemm_smallm_kernel(const void* __restrict__ A, const __nv_bfloat16* __restrict__ W, const float* __restrict__ bias,
                   void* __restrict__ out, int tokens, int n_out, int k_dim, int lda, int ldo,
                   const float* __restrict__ gain, float eps, float* __restrict__ scratch, int* __restrict__ counters,
                   const QkvEpi qe, unsigned long long* trace, int trace_cap) {
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    constexpr int ACCS = DUAL ? 2 : 1;
    constexpr int GROUPS = WARPS / KSPLIT;
    constexpr int E = NORM ? 5 : 4;                      // accumulator elements per tile, plus the row's sum of squares
    extern __shared__ float part[];                      // [KSPLIT][ACCS][NT][E][32] when KSPLIT > 1
    __shared__ int s_last;

    // Up to 16 tokens the kernel behind this one may start only when this kernel's own loads are out (below): measured,
    // dependents that are resident from this kernel's first instruction on take issue slots and bandwidth from it
    // (batch 8: 3 us a step at the 0.5B widths, 30 us at the 1.5B widths). With more tokens the attention behind the
    // q/k/v product wants its keys and values on their way as early as can be (batch 64: 1.53 against 1.56 ms).
    constexpr bool LATE_DEPENDENTS = NT <= 2;
    if (!LATE_DEPENDENTS) pdl_launch_dependents();
    bool waited = false;          // pdl_wait() comes after the first batch of weight loads has been issued
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_GEMM_SMALLM, EPI, 0);
    const int group = blockIdx.x * GROUPS + (KSPLIT > 1 ? 0 : warp);
    const int f0 = group * 16;
    const int cross = gridDim.y;

    // K range of this warp, in blocks of 32, out of KSPLIT * cross equal parts
    const int blocks = k_dim / 32;
    const int parts = KSPLIT * cross;
    const int my_part = (KSPLIT > 1 ? warp : 0) + KSPLIT * blockIdx.y;
    const int per = (blocks + parts - 1) / parts;
    const int kb_begin = min(blocks, my_part * per), kb_end = min(blocks, kb_begin + per);

    // acc[a][n][0..3]: the mma tile; acc[0][n][4] (NORM): sum of x^2 of token n*8+g over this thread's elements
    float acc[ACCS][NT][E];
#pragma unroll
    for (int a = 0; a < ACCS; ++a)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < E; ++e) acc[a][n][e] = 0.f;

    // The q/k/v epilogue's view of the thread's tokens (2t, 2t+1 of every tile): position, page, cos and sin of the
    // thread's rotated dimension. They are inputs of the step, not results of its kernels: read before the wait.
    constexpr bool QSPREAD = KSPLIT > 1 && NT > 1;        // (the q/k/v form never splits K over CTAs: tile n is warp n's)
    constexpr int QN = (EPI == EPI_QKV && !QSPREAD) ? NT : 1;
    int q_ra = 0, q_rb = 0, q_pos[QN][2], q_page[QN][2];
    float q_cs[QN][2], q_sn[QN][2], q_bias[2] = {0.f, 0.f};
    bool q_rot = false;
    if (EPI == EPI_QKV && f0 < n_out) {
        qkv_group_rows(qe, group, q_ra, q_rb);
        const int hs = q_ra / qe.head_dim, d = q_ra - hs * qe.head_dim + g;
        q_rot = hs < qe.heads + qe.kv_heads && q_rb - q_ra == (qe.rot >> 1) && qe.rot > 0 && d < (qe.rot >> 1);
        if (KSPLIT == 1 || (QSPREAD ? warp < NT : warp == 0)) {
            if (bias) { q_bias[0] = __ldg(bias + q_ra + g); q_bias[1] = __ldg(bias + q_rb + g); }
#pragma unroll
            for (int n = 0; n < QN; ++n)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int tok = (QSPREAD ? warp : n) * 8 + 2 * t + j;
                    q_pos[n][j] = 0; q_page[n][j] = -1; q_cs[n][j] = 1.f; q_sn[n][j] = 0.f;
                    if (tok < tokens) {
                        const int pos = __ldg(qe.positions + tok);
                        q_pos[n][j] = pos;
                        if (hs >= qe.heads && qe.writes)
                            q_page[n][j] = __ldg(qe.block_table + (size_t)__ldg(qe.req_index + tok) * qe.bt_stride + pos / qe.page_size);
                        if (q_rot) {
                            q_cs[n][j] = __ldg(qe.cos_t + (size_t)pos * (qe.rot >> 1) + d);
                            q_sn[n][j] = __ldg(qe.sin_t + (size_t)pos * (qe.rot >> 1) + d);
                        }
                    }
                }
        }
    }

    if (f0 < n_out) {
        // rows past the end are clamped (their results are not stored)
        int r0 = min(f0 + g, n_out - 1), r1 = min(f0 + g + 8, n_out - 1);
        if (EPI == EPI_QKV) { r0 = q_ra + g; r1 = q_rb + g; }
        const __nv_bfloat16* w0 = W + (size_t)r0 * k_dim + 8 * t;
        const __nv_bfloat16* w1 = W + (size_t)r1 * k_dim + 8 * t;
        const __nv_bfloat16* u0 = W + (size_t)(n_out + r0) * k_dim + 8 * t;
        const __nv_bfloat16* u1 = W + (size_t)(n_out + r1) * k_dim + 8 * t;
        const void* a_row[NT];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int tok = n * 8 + g;
            a_row[n] = nullptr;
            if (tok < tokens)
                a_row[n] = NORM ? (const void*)(static_cast<const float*>(A) + (size_t)tok * lda)
                                : (const void*)(static_cast<const __nv_bfloat16*>(A) + (size_t)tok * lda);
        }
        // Batches of UN blocks: every load of a batch is issued before the first mma that needs one, so a
        // warp waits for memory once per batch, not once per block (a warp issues in order).
        constexpr int UN = (NORM || DUAL) ? (NT <= 2 ? 4 : 2) : (NT <= 2 ? 8 : (NT == 4 ? 4 : 2));
        for (int base = kb_begin; base < kb_end; base += UN) {
            uint4 wa[UN], wb[UN], ua[DUAL ? UN : 1], ub[DUAL ? UN : 1];
            uint4 xb[NORM ? 1 : UN][NORM ? 1 : NT];
            float4 xf[NORM ? UN : 1][NORM ? NT : 1][2], gf[NORM ? UN : 1][2];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const bool live = base + u < kb_end;
                const int k0 = (live ? base + u : kb_begin) * 32;      // a block past the end re-reads a valid one and is zeroed
                wa[u] = ldg16_stream(w0 + k0);
                wb[u] = ldg16_stream(w1 + k0);
                if (DUAL) { ua[DUAL ? u : 0] = ldg16_stream(u0 + k0); ub[DUAL ? u : 0] = ldg16_stream(u1 + k0); }
                if (NORM) {
                    gf[NORM ? u : 0][0] = __ldg(reinterpret_cast<const float4*>(gain + k0 + 8 * t));
                    gf[NORM ? u : 0][1] = __ldg(reinterpret_cast<const float4*>(gain + k0 + 8 * t + 4));
                }
            }
            if (!waited) {                                  // weights are nobody's output; the activations are
                pdl_wait();
                waited = true;
                if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_GEMM_SMALLM, EPI, 1);
            }
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const bool live = base + u < kb_end;
                const int k0 = (live ? base + u : kb_begin) * 32;
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    if (NORM) {
                        float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                        xf[NORM ? u : 0][NORM ? n : 0][0] = z;
                        xf[NORM ? u : 0][NORM ? n : 0][1] = z;
                        if (a_row[n] && live) {
                            const float* x = static_cast<const float*>(a_row[n]) + k0 + 8 * t;
                            xf[NORM ? u : 0][NORM ? n : 0][0] = __ldcg(reinterpret_cast<const float4*>(x));
                            xf[NORM ? u : 0][NORM ? n : 0][1] = __ldcg(reinterpret_cast<const float4*>(x + 4));
                        }
                    } else {
                        xb[NORM ? 0 : u][NORM ? 0 : n] = make_uint4(0u, 0u, 0u, 0u);
                        if (a_row[n] && live)
                            xb[NORM ? 0 : u][NORM ? 0 : n] = __ldcg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a_row[n]) + k0 + 8 * t));
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < UN; ++u) {
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    uint4 x;
                    if (NORM) {
                        const float4 xa = xf[NORM ? u : 0][NORM ? n : 0][0], xc = xf[NORM ? u : 0][NORM ? n : 0][1];
                        const float4 g0 = gf[NORM ? u : 0][0], g1 = gf[NORM ? u : 0][1];
                        float& ss = acc[0][n][E - 1];
                        ss = fmaf(xa.x, xa.x, ss); ss = fmaf(xa.y, xa.y, ss); ss = fmaf(xa.z, xa.z, ss); ss = fmaf(xa.w, xa.w, ss);
                        ss = fmaf(xc.x, xc.x, ss); ss = fmaf(xc.y, xc.y, ss); ss = fmaf(xc.z, xc.z, ss); ss = fmaf(xc.w, xc.w, ss);
                        x.x = pack2(xa.x * g0.x, xa.y * g0.y);
                        x.y = pack2(xa.z * g0.z, xa.w * g0.w);
                        x.z = pack2(xc.x * g1.x, xc.y * g1.y);
                        x.w = pack2(xc.z * g1.z, xc.w * g1.w);
                    } else {
                        x = xb[NORM ? 0 : u][NORM ? 0 : n];
                    }
                    // a block past the end has zero activations: it adds nothing
                    mma_bf16(*reinterpret_cast<float(*)[4]>(&acc[0][n][0]), wa[u].x, wb[u].x, wa[u].y, wb[u].y, x.x, x.y);
                    mma_bf16(*reinterpret_cast<float(*)[4]>(&acc[0][n][0]), wa[u].z, wb[u].z, wa[u].w, wb[u].w, x.z, x.w);
                    if (DUAL) {
                        mma_bf16(*reinterpret_cast<float(*)[4]>(&acc[ACCS - 1][n][0]), ua[DUAL ? u : 0].x, ub[DUAL ? u : 0].x, ua[DUAL ? u : 0].y, ub[DUAL ? u : 0].y, x.x, x.y);
                        mma_bf16(*reinterpret_cast<float(*)[4]>(&acc[ACCS - 1][n][0]), ua[DUAL ? u : 0].z, ub[DUAL ? u : 0].z, ua[DUAL ? u : 0].w, ub[DUAL ? u : 0].w, x.z, x.w);
                    }
                }
            }
        }
    }
    if (LATE_DEPENDENTS) pdl_launch_dependents();
    if (!waited) pdl_wait();      // before the first write (shared results, scratch, output)
    if (NORM) {
        // the four threads of a quad hold the same token's partial sums: add them (fixed order)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            float v = acc[0][n][E - 1];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            acc[0][n][E - 1] = v;
        }
    }

    // Who finishes what. With K split among the warps of a CTA, each token tile of 8 is summed and finished by a warp
    // of its own (tile n by warp n: there are at most as many tiles as warps), so that 64 tokens are not one warp's
    // work; with K split over CTAs as well, warp 0 of the CTA that arrives last does all of it.
    constexpr bool SPREAD = KSPLIT > 1 && NT > 1;
    const bool spread = SPREAD && cross == 1;
    if (KSPLIT > 1) {
        // the warps of the CTA, in warp order
#pragma unroll
        for (int a = 0; a < ACCS; ++a)
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int e = 0; e < E; ++e) part[(((warp * ACCS + a) * NT + n) * E + e) * 32 + lane] = acc[a][n][e];
        __syncthreads();
        if (spread) {
            if (warp >= NT) return;
        } else if (warp != 0) {
            if (cross == 1) return;
        } else {
#pragma unroll
            for (int a = 0; a < ACCS; ++a)
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        float s = 0.f;
#pragma unroll
                        for (int w = 0; w < KSPLIT; ++w) s += part[(((w * ACCS + a) * NT + n) * E + e) * 32 + lane];
                        acc[a][n][e] = s;
                    }
        }
        if (cross > 1) {
            // the CTAs of the group: partial tiles in scratch, summed in split order by the last to arrive
            constexpr int TILE = ACCS * NT * E * 32;
            float* mine = scratch + ((size_t)blockIdx.x * cross + blockIdx.y) * TILE;
            if (warp == 0) {
#pragma unroll
                for (int a = 0; a < ACCS; ++a)
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int e = 0; e < E; ++e) mine[((a * NT + n) * E + e) * 32 + lane] = acc[a][n][e];
                __threadfence();
                __syncwarp();
                if (lane == 0) s_last = (atomicAdd(&counters[blockIdx.x], 1) == cross - 1) ? 1 : 0;
            }
            __syncthreads();
            if (!s_last || warp != 0) return;
            __threadfence();
            const float* base = scratch + (size_t)blockIdx.x * cross * TILE;
#pragma unroll
            for (int a = 0; a < ACCS; ++a)
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        float s = 0.f;
                        for (int c = 0; c < cross; ++c) s += __ldcg(base + (size_t)c * TILE + ((a * NT + n) * E + e) * 32 + lane);
                        acc[a][n][e] = s;
                    }
            if (lane == 0) counters[blockIdx.x] = 0;     // ready for the next launch
        }
    }
    if (f0 >= n_out) return;

    // ---- one token tile: v[a][0..3] the sums of accumulator a (element e: feature f0 + g + 8*(e/2), token n*8 + 2t + (e&1)),
    // v[0][4] (NORM) the sum of squares, token n*8 + j in the lanes of quad j. qi: the tile's slot in the q/k/v arrays.
    const float bias0 = (EPI != EPI_QKV && bias && f0 + g < n_out) ? bias[f0 + g] : 0.f;
    const float bias1 = (EPI != EPI_QKV && bias && f0 + g + 8 < n_out) ? bias[f0 + g + 8] : 0.f;
    auto emit = [&](const float (&v)[ACCS][E], const int n, const int qi) {
        float scale2[2] = {1.f, 1.f};                    // 1/rms of the thread's two tokens
        if (NORM) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float ss = __shfl_sync(0xffffffffu, v[0][E - 1], (2 * t + j) * 4);
                scale2[j] = 1.0f / sqrtf(ss / (float)k_dim + eps);
            }
        }
        if (EPI == EPI_QKV) {
            // the thread's rows q_ra + g (elements 0, 1) and q_rb + g (elements 2, 3) of tokens n*8 + 2t and + 1
            const int hs = q_ra / qe.head_dim;
            const int d_lo = q_ra - hs * qe.head_dim + g, d_hi = q_rb - hs * qe.head_dim + g;
            const bool is_v = hs >= qe.heads + qe.kv_heads;
            const int kvh = hs - qe.heads - (is_v ? qe.kv_heads : 0);
            __nv_bfloat16* pages = is_v ? qe.v_pages : qe.k_pages;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int tok = n * 8 + 2 * t + j;
                if (tok >= tokens) continue;
                float lo = v[0][j] * scale2[j] + q_bias[0], hi = v[0][2 + j] * scale2[j] + q_bias[1];
                if (q_rot) {
                    const float c = q_cs[qi][j], sn = q_sn[qi][j];
                    const float a = lo * c - hi * sn, b = hi * c + lo * sn;
                    lo = a;
                    hi = b;
                }
                const __nv_bfloat16 blo = __float2bfloat16_rn(lo), bhi = __float2bfloat16_rn(hi);
                __nv_bfloat16* row = (__nv_bfloat16*)out + (size_t)tok * ldo;
                row[q_ra + g] = blo;
                row[q_rb + g] = bhi;
                const int page = q_page[qi][j];
                if (hs >= qe.heads && qe.writes && page >= 0 && page < qe.num_pages) {
                    __nv_bfloat16* dst = pages + (((size_t)page * qe.kv_heads + kvh) * qe.page_size + q_pos[qi][j] % qe.page_size) * qe.head_dim;
                    dst[d_lo] = blo;
                    dst[d_hi] = bhi;
                }
            }
            return;
        }
        float res[4] = {0.f, 0.f, 0.f, 0.f};
        if (EPI == EPI_ADD) {
            // the residual stream is read-modify-written: all loads first, so that they wait together
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int f = f0 + g + 8 * (e >> 1), tok = n * 8 + 2 * t + (e & 1);
                if (f < n_out && tok < tokens) res[e] = __ldcg((const float*)out + (size_t)tok * ldo + f);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int f = f0 + g + 8 * (e >> 1), tok = n * 8 + 2 * t + (e & 1);
            if (f >= n_out || tok >= tokens) continue;
            const float x = v[0][e] * scale2[e & 1] + ((e >> 1) ? bias1 : bias0);
            const size_t o = (size_t)tok * ldo + f;
            if (EPI == EPI_STORE) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(x);
            else if (EPI == EPI_ADD) ((float*)out)[o] = res[e] + x;
            else if (EPI == EPI_F32) ((float*)out)[o] = x;
            else if (EPI == EPI_SWIGLU) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(__fdividef(x, 1.0f + __expf(-x)) * (v[ACCS - 1][e] * scale2[e & 1]));
        }
    };

    if (spread) {
        // this warp's tile: the eight warps' parts, in warp order
        float v[ACCS][E];
#pragma unroll
        for (int a = 0; a < ACCS; ++a)
#pragma unroll
            for (int e = 0; e < E; ++e) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < KSPLIT; ++w) s += part[(((w * ACCS + a) * NT + warp) * E + e) * 32 + lane];
                v[a][e] = s;
            }
        emit(v, warp, 0);
    } else {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            float v[ACCS][E];
#pragma unroll
            for (int a = 0; a < ACCS; ++a)
#pragma unroll
                for (int e = 0; e < E; ++e) v[a][e] = acc[a][n][e];
            emit(v, n, SPREAD ? 0 : n);
        }
    }
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_GEMM_SMALLM, EPI, 2);
}

struct Args {
    const void* A; const void* W; const float* bias; void* out; int tokens, N, K, lda, ldo;
    const float* gain; float eps; float* scratch; int* counters; int cross;
    QkvEpi qe;
};

template <int NT, int KSPLIT, int EPI, bool NORM>
int launch_one(const Args& a, cudaStream_t stream) {
    constexpr int ACCS = (EPI == EPI_SWIGLU) ? 2 : 1;
    const int groups = ceil_div(a.N, 16);
    dim3 grid(ceil_div(groups, WARPS / KSPLIT), KSPLIT > 1 ? a.cross : 1);
    const size_t smem = KSPLIT > 1 ? (size_t)KSPLIT * ACCS * NT * (NORM ? 5 : 4) * 32 * sizeof(float) : 0;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        NIB_CUDA(cudaFuncSetAttribute(gemm_smallm_kernel<NT, KSPLIT, EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    configured = true;
    NIB_CUDA(launch_pdl(gemm_smallm_kernel<NT, KSPLIT, EPI, NORM>, grid, dim3(WARPS * 32), smem, stream,
                        a.A, (const __nv_bfloat16*)a.W, a.bias, a.out, a.tokens, a.N, a.K, a.lda, a.ldo, a.gain, a.eps,
                        a.scratch, a.counters, a.qe, nib_trace_buffer(), nib_trace_capacity()));
    return 0;
}

template <int NT, int KSPLIT, bool NORM>
int launch_epi(int epi, const Args& a, cudaStream_t stream) {
    switch (epi) {
        case EPI_STORE: return launch_one<NT, KSPLIT, EPI_STORE, NORM>(a, stream);
        case EPI_ADD: return launch_one<NT, KSPLIT, EPI_ADD, NORM>(a, stream);
        case EPI_F32: return launch_one<NT, KSPLIT, EPI_F32, NORM>(a, stream);
        case EPI_SWIGLU: return launch_one<NT, KSPLIT, EPI_SWIGLU, NORM>(a, stream);
        case EPI_QKV:
            if constexpr (KSPLIT > 1) return launch_one<NT, KSPLIT, EPI_QKV, NORM>(a, stream);
            break;
    }
    nib_set_error("gemm (small M): unknown epilogue %d", epi);
    return 1;
}

template <int NT, bool NORM>
int launch_split(int ksplit, int epi, const Args& a, cudaStream_t stream) {
    if (ksplit > 1) return launch_epi<NT, WARPS, NORM>(epi, a, stream);
    return launch_epi<NT, 1, NORM>(epi, a, stream);
}

template <bool NORM>
int launch_tokens(int ksplit, int epi, const Args& a, cudaStream_t stream) {
    if (a.tokens <= 8) return launch_split<1, NORM>(ksplit, epi, a, stream);
    if (a.tokens <= 16) return launch_split<2, NORM>(ksplit, epi, a, stream);
    if (a.tokens <= 32) return launch_split<4, NORM>(ksplit, epi, a, stream);
    return launch_split<8, NORM>(ksplit, epi, a, stream);
}

}  // namespace

// 1 if the kernel takes these operands: at most 64 tokens, K a multiple of 32, 16-byte aligned rows.
// elem_bytes: 2 for a bfloat16 A operand, 4 for the 32-bit residual stream of the fused-norm form.
NIB_API int nib_gemm_smallm_supported(const void* A, const void* W, int tokens, int K, int lda, int elem_bytes) {
    if (tokens <= 0 || tokens > MAX_TOKENS || K <= 0 || K % 32) return 0;
    if ((lda * elem_bytes) % 16) return 0;
    return (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) ? 0 : 1;
}

// Floats of scratch and ints of counters that a call with these sizes may use (for the caller's workspace).
NIB_API long long nib_gemm_smallm_scratch_floats(int N, int cross) {
    return (long long)ceil_div(N, 16) * cross * 2 * 8 * 5 * 32;
}

// Same operands and epilogues as nib_gemm_tc. If gain != nullptr, A is the float residual stream
// [tokens, K] and is RMS-normalised with (gain, eps) on the fly. ksplit: 0 = chosen here, 1 or 8.
// cross: CTAs that split K further (needs ksplit 8; 0 = chosen here; > 1 needs scratch of
// nib_gemm_smallm_scratch_floats floats and ceil(N/16) zeroed counters, both reusable between calls).
NIB_API int nib_gemm_smallm(const void* A, const void* W, const float* bias, void* out, int tokens, int N, int K,
                            int lda, int ldo, int epi, const float* gain, float eps, int ksplit, int cross,
                            float* scratch, int* counters, long long scratch_floats, int counter_ints,
                            cudaStream_t stream) {
    NIB_REQUIRE(N > 0 && lda >= K && ldo >= N, "gemm (small M): bad sizes tokens=%d N=%d K=%d", tokens, N, K);
    NIB_REQUIRE(nib_gemm_smallm_supported(A, W, tokens, K, lda, gain ? 4 : 2),
                "gemm (small M): needs 1..64 tokens, K %% 32 == 0 and 16-byte aligned rows (tokens=%d K=%d)", tokens, K);
    NIB_REQUIRE(epi != EPI_SWIGLU || bias == nullptr, "gemm (small M): the swiglu epilogue takes no bias");
    NIB_REQUIRE(gain == nullptr || (((uintptr_t)gain & 15) == 0), "gemm (small M): the gain must be 16-byte aligned");
    const int groups = ceil_div(N, 16), blocks = K / 32;
    if (ksplit == 0) ksplit = (groups < 8 * 148 && blocks >= 8) ? WARPS : 1;   // wide outputs: a warp per row group
    NIB_REQUIRE(ksplit == 1 || ksplit == WARPS, "gemm (small M): ksplit must be 1 or %d", WARPS);
    if (ksplit == 1) cross = 1;
    if (cross == 0) {
        // a warp keeps about eight blocks of K in flight; only a longer K is worth the extra
        // hand-over between CTAs (a fence, a counter and a second read of the partial tiles)
        cross = 1;
        if (scratch && counters) {
            // measured: the hand-over between CTAs (fence, counter, second read of the partials) costs more
            // than it saves until a warp would have to stream more than ~32 blocks of K on its own
            cross = ceil_div(blocks, WARPS * 32);
            if (cross > 16) cross = 16;
            while (cross > 1 && (long long)groups * cross > 8 * 148) --cross;
        }
    }
    if (cross > 1) {
        NIB_REQUIRE(scratch && counters, "gemm (small M): a cross-CTA split needs scratch memory and counters");
        NIB_REQUIRE(nib_gemm_smallm_scratch_floats(N, cross) <= scratch_floats && groups <= counter_ints,
                    "gemm (small M): workspace too small for N=%d cross=%d", N, cross);
    }
    Args a{A, W, bias, out, tokens, N, K, lda, ldo, gain, eps, scratch, counters, cross, QkvEpi{}};
    if (gain) return launch_tokens<true>(ksplit, epi, a, stream);
    return launch_tokens<false>(ksplit, epi, a, stream);
}

// 1 if nib_gemm_smallm_qkv takes these sizes: up to 64 tokens, head size and rotated width multiples of 16.
NIB_API int nib_gemm_smallm_qkv_supported(const void* A, const void* W, int tokens, int K, int lda, int elem_bytes,
                                          int head_dim, int rot) {
    if (tokens > MAX_TOKENS || head_dim <= 0 || head_dim % 16 || rot < 0 || rot > head_dim || rot % 16) return 0;
    return nib_gemm_smallm_supported(A, W, tokens, K, lda, elem_bytes);
}

// The q/k/v projection of a decode step with what follows it, in one kernel: qkv[tokens, (heads + 2 kv_heads) *
// head_dim] = A . W^T + bias (A, gain, eps as in nib_gemm_smallm); query and key heads are rotated by
// positions[token] (tables of rot/2 values per position; the first rot dimensions of a head, halves paired); the whole
// row is stored to ``qkv``; with ``writes`` the rotated key and the value also go to the slot of the token's position
// in its request's page (block_table[req_index[token]][position / page_size]; a negative entry is skipped).
NIB_API int nib_gemm_smallm_qkv(const void* A, const void* W, const float* bias, void* qkv, int tokens, int heads,
                                int kv_heads, int head_dim, int K, int lda, int ldq, const float* gain, float eps,
                                const int* positions, const int* req_index, const float* cos_t, const float* sin_t,
                                int rot, const int* block_table, int bt_stride, int page_size, void* k_pages,
                                void* v_pages, int num_pages, int writes, cudaStream_t stream) {
    const int N = (heads + 2 * kv_heads) * head_dim;
    NIB_REQUIRE(heads > 0 && kv_heads > 0 && lda >= K && ldq >= N, "gemm (small M, q/k/v): bad sizes heads=%d/%d head_dim=%d", heads, kv_heads, head_dim);
    NIB_REQUIRE(nib_gemm_smallm_qkv_supported(A, W, tokens, K, lda, gain ? 4 : 2, head_dim, rot),
                "gemm (small M, q/k/v): needs 1..64 tokens, K %% 32 == 0, head_dim and the rotated width multiples of 16 (tokens=%d K=%d head_dim=%d rot=%d)",
                tokens, K, head_dim, rot);
    NIB_REQUIRE(rot == 0 || (cos_t && sin_t), "gemm (small M, q/k/v): rotation needs the tables");
    NIB_REQUIRE(positions && req_index, "gemm (small M, q/k/v): positions and request rows are needed");
    NIB_REQUIRE(!writes || (block_table && k_pages && v_pages && page_size > 0 && num_pages > 0), "gemm (small M, q/k/v): writing needs pages and a block table");
    NIB_REQUIRE(gain == nullptr || (((uintptr_t)gain & 15) == 0), "gemm (small M, q/k/v): the gain must be 16-byte aligned");
    Args a{A, W, bias, qkv, tokens, N, K, lda, ldq, gain, eps, nullptr, nullptr, 1,
           QkvEpi{heads, kv_heads, head_dim, rot, positions, req_index, cos_t, sin_t, block_table, bt_stride, page_size,
                  num_pages, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, writes}};
    if (gain) return launch_tokens<true>(WARPS, EPI_QKV, a, stream);
    return launch_tokens<false>(WARPS, EPI_QKV, a, stream);
}
