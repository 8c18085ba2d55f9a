// The feed-forward block of a decode step in ONE kernel: RMSNorm, gate/up projection with SiLU(gate)*up,
// down projection, sum into the residual stream; for up to 8 tokens, bfloat16 weights.
//
// As three kernels (norm, gate/up, down) these cost three launches and three dependent chains of memory
// round trips per layer, which is what bounds a small model's decode step. Here one CTA per SM stays
// resident for the whole block:
//   0. before the wait for the previous kernel: the CTA's weight rows (its share of the gate/up rows and of
//      the down rows) are prefetched into L2;
//   1. every CTA normalises the step's tokens into shared memory (the 32-bit residual rows are a few KB);
//   2. gate/up: the CTA's rows (intermediate / CTAs of them, tiles of 16), K split over its 8 warps, weights
//      streamed with 16-byte loads into mma.sync fragments as in gemm_smallm.cu, summed over the warps in
//      warp order, SiLU(gate)*up written as bfloat16 to a scratch [tokens, intermediate];
//   3. a barrier over the grid (one arrival counter; bounded wait; the launch is cooperative, so all CTAs are
//      resident), then
//   4. down: the CTA's rows of the hidden size, K = intermediate split over its warps, the activations read
//      from the scratch through L2; every output element has one owner, which adds it to the residual.
// The order of every sum is fixed by the sizes and the grid alone.
//
// Measured on B200 at the 0.5B sizes (hidden 896, intermediate 4864, 8 tokens, cold weights, chained in a
// graph): 18.6 us per block against 13.2 us for the three kernels, whose prologues overlap through
// programmatic dependent launch: inside one kernel the same dependent round trips (tokens, weights,
// activations through L2, residual) run one after the other and the grid barrier adds its own. The engine
// therefore leaves this path off (Kernels.fuse_ffn); it stays as a tested building block for a decode
// kernel that keeps more of a layer on the SMs.
//
// Reference formulas: cpp/src/ops.cpp:272-292 (rmsnorm), :42-69 (linear), :86-100 (silu, mul);
// cpp/src/model.cpp:217-223 (the block). The reference runs it as five kernels.
#include "common.cuh"

namespace {

constexpr int WARPS = 8, THREADS = WARPS * 32;
constexpr int MAX_TILES = 4;                 // row tiles of 16 per CTA and phase
constexpr unsigned SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg16_stream(const __nv_bfloat16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p)); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Streams `tiles` tiles of 16 weight rows (rows row0 + 16 i + g and + 8, clamped to row_end - 1) over the warp's
// blocks of 32 along K and multiplies them with the 8 token columns that `b_of(k0)` returns for this lane
// (8 consecutive bfloat16 of token g at k0 + 8 t, as a uint4). DUAL: a second matrix `rows2` apart.
template <bool DUAL, typename BOf>
__device__ __forceinline__ void stream_rows(float (&acc)[MAX_TILES][2][4], const __nv_bfloat16* __restrict__ w, size_t ldw,
                                            size_t rows2, int row0, int row_end, int tiles, int kb_begin, int kb_end,
                                            int g, int t, BOf b_of) {
    constexpr int UN = DUAL ? 2 : 4;
    const __nv_bfloat16* p0[MAX_TILES];
    const __nv_bfloat16* p1[MAX_TILES];
#pragma unroll
    for (int i = 0; i < MAX_TILES; ++i) {
        const int r0 = min(row0 + 16 * i + g, row_end - 1), r1 = min(row0 + 16 * i + g + 8, row_end - 1);
        p0[i] = w + (size_t)r0 * ldw + 8 * t;
        p1[i] = w + (size_t)r1 * ldw + 8 * t;
    }
    for (int base = kb_begin; base < kb_end; base += UN) {
        uint4 wa[UN][MAX_TILES], wb[UN][MAX_TILES], ua[DUAL ? UN : 1][MAX_TILES], ub[DUAL ? UN : 1][MAX_TILES], x[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const bool live = base + u < kb_end;
            const int k0 = (live ? base + u : kb_begin) * 32;     // a block past the end re-reads a valid one and is zeroed
#pragma unroll
            for (int i = 0; i < MAX_TILES; ++i) {
                if (i < tiles) {
                    wa[u][i] = ldg16_stream(p0[i] + k0);
                    wb[u][i] = ldg16_stream(p1[i] + k0);
                    if (DUAL) {
                        ua[DUAL ? u : 0][i] = ldg16_stream(p0[i] + rows2 * ldw + k0);
                        ub[DUAL ? u : 0][i] = ldg16_stream(p1[i] + rows2 * ldw + k0);
                    }
                }
            }
            x[u] = live ? b_of(k0) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
#pragma unroll
            for (int i = 0; i < MAX_TILES; ++i) {
                if (i < tiles) {
                    mma_bf16(acc[i][0], wa[u][i].x, wb[u][i].x, wa[u][i].y, wb[u][i].y, x[u].x, x[u].y);
                    mma_bf16(acc[i][0], wa[u][i].z, wb[u][i].z, wa[u][i].w, wb[u][i].w, x[u].z, x[u].w);
                    if (DUAL) {
                        mma_bf16(acc[i][1], ua[DUAL ? u : 0][i].x, ub[DUAL ? u : 0][i].x, ua[DUAL ? u : 0][i].y, ub[DUAL ? u : 0][i].y, x[u].x, x[u].y);
                        mma_bf16(acc[i][1], ua[DUAL ? u : 0][i].z, ub[DUAL ? u : 0][i].z, ua[DUAL ? u : 0][i].w, ub[DUAL ? u : 0][i].w, x[u].z, x[u].w);
                    }
                }
            }
        }
    }
}

// bar[0]: arrivals at the grid barrier, bar[1]: departures; both zero between launches. err: set if a wait ran out.
__global__ void __launch_bounds__(THREADS, 1)
ffn_decode_kernel(float* __restrict__ x32, int ldx, const float* __restrict__ gain, float eps,
                  const __nv_bfloat16* __restrict__ w_gu, const __nv_bfloat16* __restrict__ w_down,
                  __nv_bfloat16* __restrict__ act, int tokens, int hidden, int inter, unsigned* __restrict__ bar,
                  int* __restrict__ err) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int lda = hidden + 32;                                   // bfloat16 elements per row: rows fall 64 bytes apart in the banks
    __nv_bfloat16* s_a = reinterpret_cast<__nv_bfloat16*>(smem);   // [8][lda] normalised tokens
    float* s_part = reinterpret_cast<float*>(smem + (size_t)8 * lda * 2);   // [WARPS][MAX_TILES][2][4][32]
    __shared__ int s_ok;

    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int ctas = gridDim.x, cta = blockIdx.x;
    const int per_gu = (inter + ctas - 1) / ctas, gu0 = min(inter, cta * per_gu), gu1 = min(inter, gu0 + per_gu);
    const int per_d = (hidden + ctas - 1) / ctas, d0 = min(hidden, cta * per_d), d1 = min(hidden, d0 + per_d);
    const int gu_tiles = (gu1 - gu0 + 15) / 16, d_tiles = (d1 - d0 + 15) / 16;

    // 0. this CTA's weights towards L2 (they are nobody's output)
    {
        const size_t row_bytes_gu = (size_t)hidden * 2, row_bytes_d = (size_t)inter * 2;
        const size_t n_gu = (size_t)(gu1 - gu0) * row_bytes_gu / 128, n_d = (size_t)(d1 - d0) * row_bytes_d / 128;
        const char* base_g = reinterpret_cast<const char*>(w_gu + (size_t)gu0 * hidden);
        const char* base_u = reinterpret_cast<const char*>(w_gu + (size_t)(inter + gu0) * hidden);
        const char* base_d = reinterpret_cast<const char*>(w_down + (size_t)d0 * inter);
        for (size_t i = tid; i < n_gu; i += THREADS) { prefetch_l2(base_g + i * 128); prefetch_l2(base_u + i * 128); }
        for (size_t i = tid; i < n_d; i += THREADS) prefetch_l2(base_d + i * 128);
    }
    pdl_wait();

    // 1. RMSNorm of the step's tokens into shared memory (warp w: token w); rows of absent tokens are zero
    {
        __nv_bfloat16* row = s_a + (size_t)warp * lda;
        if (warp < tokens) {
            const float4* xr = reinterpret_cast<const float4*>(x32 + (size_t)warp * ldx);
            float ss = 0.f;
            for (int c = lane; c < hidden / 4; c += 32) {
                const float4 v = __ldcg(xr + c);
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
            ss = warp_sum(ss);
            const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
            for (int c = lane; c < hidden / 4; c += 32) {
                const float4 v = __ldcg(xr + c), gg = __ldg(reinterpret_cast<const float4*>(gain) + c);
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * scale * gg.x, v.y * scale * gg.y);
                __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * scale * gg.z, v.w * scale * gg.w);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned*>(&lo);
                pk.y = *reinterpret_cast<unsigned*>(&hi);
                *reinterpret_cast<uint2*>(row + 4 * c) = pk;
            }
        } else {
            for (int c = lane; c < hidden / 4; c += 32) *reinterpret_cast<uint2*>(row + 4 * c) = make_uint2(0u, 0u);
        }
    }
    __syncthreads();

    float acc[MAX_TILES][2][4];
    auto clear = [&]() {
#pragma unroll
        for (int i = 0; i < MAX_TILES; ++i)
#pragma unroll
            for (int a = 0; a < 2; ++a) acc[i][a][0] = acc[i][a][1] = acc[i][a][2] = acc[i][a][3] = 0.f;
    };
    // partial tiles of the eight warps -> shared memory; afterwards element (i, a, e, lane) is summed in warp order
    auto publish = [&](int tiles, int accs) {
        for (int i = 0; i < tiles; ++i)
            for (int a = 0; a < accs; ++a)
#pragma unroll
                for (int e = 0; e < 4; ++e) s_part[((((size_t)warp * MAX_TILES + i) * 2 + a) * 4 + e) * 32 + lane] = acc[i][a][e];
    };
    auto summed = [&](int i, int a, int e, int ln) -> float {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) s += s_part[((((size_t)w * MAX_TILES + i) * 2 + a) * 4 + e) * 32 + ln];
        return s;
    };

    // 2. gate/up rows gu0..gu1 of this CTA; warp w takes the w-th eighth of K
    {
        clear();
        const int blocks = hidden / 32, per = (blocks + WARPS - 1) / WARPS;
        const int kb_begin = min(blocks, warp * per), kb_end = min(blocks, kb_begin + per);
        if (gu_tiles > 0)
            stream_rows<true>(acc, w_gu, (size_t)hidden, (size_t)inter, gu0, gu1, gu_tiles, kb_begin, kb_end, g, t,
                              [&](int k0) { return *reinterpret_cast<const uint4*>(s_a + (size_t)g * lda + k0 + 8 * t); });
        publish(gu_tiles, 2);
        __syncthreads();
        // element e of tile i in lane (g, t): row gu0 + 16 i + g + 8 (e / 2), token 2 t + (e & 1)
        for (int idx = tid; idx < gu_tiles * 4 * 32; idx += THREADS) {
            const int ln = idx & 31, e = (idx >> 5) & 3, i = idx >> 7;
            const int row = gu0 + 16 * i + (ln >> 2) + 8 * (e >> 1), tok = 2 * (ln & 3) + (e & 1);
            if (row < gu1 && tok < tokens) {
                const float gate = summed(i, 0, e, ln), up = summed(i, 1, e, ln);
                act[(size_t)tok * inter + row] = __float2bfloat16_rn(__fdividef(gate, 1.0f + __expf(-gate)) * up);
            }
        }
    }

    // 3. every CTA's activations are written before any CTA reads them
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        atomicAdd(&bar[0], 1u);
        int ok = 0;
        for (unsigned i = 0; i < SPIN_LIMIT; ++i) {
            if (ld_acquire(&bar[0]) >= (unsigned)ctas) { ok = 1; break; }
            if (i > 64) __nanosleep(40);
        }
        if (!ok) atomicExch(err, 1);
        s_ok = ok;
        // the CTA that leaves last clears the counters for the next launch
        if (atomicAdd(&bar[1], 1u) == (unsigned)ctas - 1) { bar[0] = 0u; bar[1] = 0u; __threadfence(); }
    }
    __syncthreads();
    if (!s_ok) return;

    // 4. down rows d0..d1 of this CTA, K = intermediate; the activations come from the scratch through L2
    {
        clear();
        const int blocks = inter / 32, per = (blocks + WARPS - 1) / WARPS;
        const int kb_begin = min(blocks, warp * per), kb_end = min(blocks, kb_begin + per);
        const __nv_bfloat16* a_row = act + (size_t)g * inter + 8 * t;
        const bool has_tok = g < tokens;
        if (d_tiles > 0)
            stream_rows<false>(acc, w_down, (size_t)inter, 0, d0, d1, d_tiles, kb_begin, kb_end, g, t,
                               [&](int k0) { return has_tok ? __ldcg(reinterpret_cast<const uint4*>(a_row + k0)) : make_uint4(0u, 0u, 0u, 0u); });
        __syncthreads();            // the gate/up sums have been read
        publish(d_tiles, 1);
        __syncthreads();
        for (int idx = tid; idx < d_tiles * 4 * 32; idx += THREADS) {
            const int ln = idx & 31, e = (idx >> 5) & 3, i = idx >> 7;
            const int row = d0 + 16 * i + (ln >> 2) + 8 * (e >> 1), tok = 2 * (ln & 3) + (e & 1);
            if (row < d1 && tok < tokens) x32[(size_t)tok * ldx + row] += summed(i, 0, e, ln);
        }
    }
}

int sm_count_ffn() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 1;
    }
    return sms;
}

size_t ffn_smem(int hidden) { return (size_t)8 * (hidden + 32) * 2 + (size_t)WARPS * MAX_TILES * 2 * 4 * 32 * 4; }

}  // namespace

// 1 if the fused kernel takes these sizes: up to 8 tokens, hidden and intermediate multiples of 32, at most
// 64 rows of either matrix per SM, the normalised tokens fit shared memory, 16-byte aligned rows.
NIB_API int nib_ffn_decode_supported(int tokens, int hidden, int inter, int ldx) {
    if (tokens < 1 || tokens > 8 || hidden % 32 || inter % 32 || hidden <= 0 || inter <= 0 || ldx % 4) return 0;
    const int ctas = sm_count_ffn();
    if (ceil_div(inter, ctas) > 16 * MAX_TILES || ceil_div(hidden, ctas) > 16 * MAX_TILES) return 0;
    return ffn_smem(hidden) <= 200 * 1024;
}

// x32 [tokens, hidden] (row stride ldx) += down( silu(gate(n)) * up(n) ), n = rmsnorm(x32) * gain. w_gate_up
// [2 * inter, hidden] (gate rows, then up rows), w_down [hidden, inter], act: scratch of tokens * inter bfloat16,
// barrier: two zeroed 32-bit counters that the kernel leaves zeroed, err: an int that is set to 1 if the
// barrier's bounded wait ran out (the result is then incomplete).
NIB_API int nib_ffn_decode(float* x32, int ldx, const float* gain, float eps, const void* w_gate_up, const void* w_down,
                           void* act, int tokens, int hidden, int inter, unsigned* barrier, int* err, cudaStream_t stream) {
    NIB_REQUIRE(nib_ffn_decode_supported(tokens, hidden, inter, ldx), "ffn (fused decode): %d tokens, hidden %d, intermediate %d are not supported", tokens, hidden, inter);
    NIB_REQUIRE(((((uintptr_t)x32 | (uintptr_t)gain | (uintptr_t)w_gate_up | (uintptr_t)w_down | (uintptr_t)act) & 15) == 0), "ffn (fused decode): operands must be 16-byte aligned");
    NIB_REQUIRE(barrier != nullptr && err != nullptr, "ffn (fused decode): barrier counters and error word are needed");
    const size_t smem = ffn_smem(hidden);
    static bool configured = false;
    static int resident = 0;
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(ffn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = true;
    }
    NIB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, ffn_decode_kernel, THREADS, smem));
    NIB_REQUIRE(resident >= 1, "ffn (fused decode): a CTA does not fit an SM");
    // cooperative: every CTA of the grid is resident, so the grid barrier cannot wait for a CTA that has no SM
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count_ffn());
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = nib_pdl_enabled() ? 2 : 1;
    NIB_CUDA(cudaLaunchKernelEx(&cfg, ffn_decode_kernel, x32, ldx, gain, eps, (const __nv_bfloat16*)w_gate_up,
                                (const __nv_bfloat16*)w_down, (__nv_bfloat16*)act, tokens, hidden, inter, barrier, err));
    return 0;
}
