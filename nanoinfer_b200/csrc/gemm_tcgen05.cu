// Matrix product on the 5th-generation tensor cores of sm_100a: out[tokens, N] = A[tokens, K] . W[N, K]^T
// for bfloat16 operands, 32-bit accumulation in tensor memory (TMEM).
//
// Orientation: the WEIGHT rows are the M side of the instruction (tiles of 128 output features =
// the 128 TMEM lanes), the TOKENS are its N side (16..256 per tile). A decode step with few tokens
// therefore still fills the 128-row instruction, and streams every weight exactly once; a prefill
// uses token tiles of 128 or 256. One thread of the epilogue owns one output feature, so bias is a
// scalar per thread and the residual sum is a coalesced read-modify-write over 32 features.
//
// Persistent CTAs (at most one per SM) walk over the output tiles. Per CTA (192 threads): warp 0 = TMA
// producer (one lane), warp 1 = MMA issuer (one lane; the warp allocates and frees TMEM), warps 2..5 =
// epilogue (tcgen05.ld of the warp's lane quadrant). Operand tiles are 64 elements (128 bytes) wide in K
// with the 128-byte swizzle, written by TMA and read by tcgen05.mma through shared-memory descriptors;
// STAGES tiles are in flight, tracked by full/empty mbarriers that run on across output tiles;
// tcgen05.commit releases a stage when the MMAs that read it are done. The accumulator is double
// buffered in TMEM: while the epilogue warps drain tile i, the MMA warp already fills tile i+1.
//
// Split K: with few output tiles (a decode step of a narrow projection) the K range of a tile is cut
// into `splits` work items that different CTAs run at the same time, so that all SMs stream weights.
// The ADD epilogue then adds each item's partial sums into the 32-bit output with reductions in
// memory (red.global.add.f32; the order of the additions, and with it the last bit, is not fixed).
// The other epilogues leave the partial sums in a scratch buffer; per (tile, 32-feature quadrant) a
// counter tells the warp that arrives last, and that warp adds the partials in the fixed order of the
// splits and runs the epilogue (chosen for up to 16 tokens only: one warp reads all of them).
// Nobody waits for anybody.
//
// Every wait has an iteration limit; a wait that runs out records a code in an error word, the CTA
// stops issuing, waits (bounded) for its own copies in flight, frees its TMEM and returns.
//
// Epilogues: STORE bf16 (+bias), ADD into a float tensor (the residual sum), F32 store (logits),
// SWIGLU (two accumulators from W rows n and n + N: silu(gate) * up). Reference formulas:
// cpp/src/ops.cpp:42-69 (linear), :86-93 (silu). The reference's tensor-core GEMMs are wmma kernels
// for sm_89 (cpp/src/cuda/cuda_gemm.cu:484-622).
#include "tcgen05.cuh"
#include <mutex>
#include <unordered_map>

using namespace nibp;
using namespace nibt;

namespace {

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_F32 = 2, EPI_SWIGLU = 3, EPI_QKV = 4 };

constexpr int BLOCK_F = 128;     // output features per CTA (UMMA M)
constexpr int BLOCK_K = 64;      // elements of K per stage: 128 bytes, one swizzle atom
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;

__device__ int g_tc_error = 0;   // 0, or (code << 16 | blockIdx.x) of the first wait that ran out

// HD != 0 (the q/k/v form): four stages, and room for the rotation tables' rows of the tile's 128 tokens (cos and sin,
// HD/2 values each, rows padded by one float so that a thread per row reads them without bank conflicts).
template <int TOK, bool DUAL, int HD = 0> struct Cfg {
    static constexpr int W_BYTES = BLOCK_F * BLOCK_K * 2;                 // 16 KB
    static constexpr int A_BYTES = TOK * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * W_BYTES + A_BYTES;
    static constexpr int STAGES = HD ? 4 : ((200 * 1024 / STAGE_BYTES) > 8 ? 8 : (200 * 1024 / STAGE_BYTES));
    static constexpr int TAB_ROW = HD / 2 + 1;                            // floats per staged table row
    static constexpr int TAB_BYTES = HD ? 2 * BLOCK_F * TAB_ROW * 4 : 0;
    static constexpr int OFF_TAB = STAGES * STAGE_BYTES + 256;            // behind the barriers
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */ + TAB_BYTES;
    static constexpr int ACC_COLS = (DUAL ? 2 : 1) * TOK;                 // columns of one accumulator buffer
    static constexpr int TMEM_COLS = tmem_cols(2 * ACC_COLS);             // two buffers
    static_assert(2 * ACC_COLS <= 512, "two accumulator buffers must fit the 512 TMEM columns");
};

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// 16 consecutive features (first .. first+15) of one token row. v: accumulators (for SWIGLU the gate), u: the up values.
template <int EPI>
__device__ __forceinline__ void emit_row16(void* __restrict__ out, const float (&v)[16], const float (&u)[16],
                                           const float* __restrict__ bias, size_t row_off, int first, int n_out, bool vec_ok) {
    float x[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) x[j] = v[j];
    if (bias != nullptr) {
        if (first + 16 <= n_out) {          // 16 features start on a 64-byte boundary of the bias
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(bias + first) + j);
                x[4 * j] += b.x; x[4 * j + 1] += b.y; x[4 * j + 2] += b.z; x[4 * j + 3] += b.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (first + j < n_out) x[j] += __ldg(bias + first + j);
        }
    }
    if (EPI == EPI_SWIGLU) {
        // silu(g) * u with the fast exponential and division (2 ulp): the result is rounded to bfloat16
#pragma unroll
        for (int j = 0; j < 16; ++j) x[j] = __fdividef(x[j], 1.0f + __expf(-x[j])) * u[j];
    }
    if (vec_ok && first + 16 <= n_out) {
        if (EPI == EPI_STORE || EPI == EPI_SWIGLU) {
            uint4 p0, p1;
            __nv_bfloat162* h0 = reinterpret_cast<__nv_bfloat162*>(&p0);
            __nv_bfloat162* h1 = reinterpret_cast<__nv_bfloat162*>(&p1);
#pragma unroll
            for (int j = 0; j < 4; ++j) { h0[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]); h1[j] = __floats2bfloat162_rn(x[8 + 2 * j], x[9 + 2 * j]); }
            uint4* dst = reinterpret_cast<uint4*>((__nv_bfloat16*)out + row_off + first);
            dst[0] = p0;
            dst[1] = p1;
        } else if (EPI == EPI_F32) {
            float4* dst = reinterpret_cast<float4*>((float*)out + row_off + first);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_float4(x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
        } else {
            float* dst = (float*)out + row_off + first;
#pragma unroll
            for (int j = 0; j < 4; ++j) red_add_v4(dst + 4 * j, x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (first + j >= n_out) break;
        const size_t o = row_off + first + j;
        if (EPI == EPI_STORE || EPI == EPI_SWIGLU) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(x[j]);
        else if (EPI == EPI_F32) ((float*)out)[o] = x[j];
        else atomicAdd((float*)out + o, x[j]);
    }
}

// ---- the q/k/v projection's epilogue (EPI_QKV), for the kernels whose threads own a TOKEN row of the accumulator
// The product's columns are [q heads | k heads | v heads] of HD features each; a tile of 128 columns holds whole heads.
// Per head: bias, rotation of query and key heads by the token's position (halves paired: d with d + HD/2, the whole
// head is rotated), one rounding to bfloat16, the row into the activation buffer and, for key and value heads, into the
// slot of the token's position in its request's page. Reference: cpp/src/ops.cpp:146-168 (rotation),
// cpp/src/cuda/cuda_backend.cu:354-367 (page write).
struct QkvRows {
    int heads, kv_heads, rotate;           // rotate: 1 = rotate q and k heads (tables of HD/2 values per position)
    const int* positions; const int* req_index; const float* cos_t; const float* sin_t;
    const int* block_table; int bt_stride, page_size, num_pages;
    __nv_bfloat16* k_pages; __nv_bfloat16* v_pages; int writes;
};

// addr: TMEM address of the head's first column in this thread's lane; f: the head's first feature; live: the row exists;
// cos_row, sin_row: the HD/2 table values of the token's position (staged in shared memory by the caller).
// Every thread of the warp calls it (the TMEM loads are warp-wide); only live rows store.
template <int HD>
__device__ __forceinline__ void emit_qkv_head(unsigned addr, int f, const float* __restrict__ bias, __nv_bfloat16* __restrict__ row_out,
                                              const QkvRows& q, int pos, long long page, bool live,
                                              const float* cos_row, const float* sin_row) {
    unsigned r[HD / 16][16];
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) tmem_ld16_async(addr + 16 * i, r[i]);
    tmem_wait_ld();
    if (!live) return;
    float x[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) x[i] = __uint_as_float(r[i >> 4][i & 15]);
    if (bias != nullptr) {
#pragma unroll
        for (int i = 0; i < HD / 4; ++i) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(bias + f) + i);
            x[4 * i] += b.x; x[4 * i + 1] += b.y; x[4 * i + 2] += b.z; x[4 * i + 3] += b.w;
        }
    }
    const int hs = f / HD;
    if (q.rotate && hs < q.heads + q.kv_heads) {
        constexpr int HALF = HD / 2;
#pragma unroll
        for (int d = 0; d < HALF; ++d) {
            const float c = cos_row[d], sn = sin_row[d];
            const float lo = x[d], hi = x[d + HALF];
            x[d] = lo * c - hi * sn;
            x[d + HALF] = hi * c + lo * sn;
        }
    }
    uint4 packed[HD / 8];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(x[8 * i + 2 * j], x[8 * i + 2 * j + 1]);
    }
    uint4* dst = reinterpret_cast<uint4*>(row_out + f);
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) dst[i] = packed[i];
    if (hs >= q.heads && q.writes && page >= 0) {
        const bool is_v = hs >= q.heads + q.kv_heads;
        const int kvh = hs - q.heads - (is_v ? q.kv_heads : 0);
        __nv_bfloat16* pages = is_v ? q.v_pages : q.k_pages;
        uint4* slot = reinterpret_cast<uint4*>(pages + (((size_t)page * q.kv_heads + kvh) * q.page_size + pos % q.page_size) * HD);
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) slot[i] = packed[i];
    }
}

// The epilogue of 16 consecutive tokens (first_token ..) of output feature f: v = accumulator, u = the
// second accumulator of the swiglu form, b = bias.
template <int EPI>
__device__ __forceinline__ void emit16(void* __restrict__ out, const float (&v)[16], const float (&u)[16], float b, int f,
                                       int first_token, int tokens, int ldo) {
    if (EPI == EPI_ADD) {
        // The sum into the residual stream is a reduction in memory (red.global.add.f32): nothing is
        // read back, so the epilogue does not wait a memory round trip per batch of tokens. Each element
        // has one writer here (one add, the same bits as load-add-store); with K split several items add.
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int t = first_token + j;
            if (t < tokens) atomicAdd((float*)out + (size_t)t * ldo + f, v[j] + b);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int t = first_token + j;
            if (t >= tokens) break;
            const size_t o = (size_t)t * ldo + f;
            const float x = v[j] + b;
            if (EPI == EPI_STORE) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(x);
            else if (EPI == EPI_F32) ((float*)out)[o] = x;
            else ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(__fdividef(x, 1.0f + __expf(-x)) * u[j]);
        }
    }
}

// grid: persistent CTAs; tile index -> (feature tile, token tile), feature tiles fastest
//
// SWAP (tiles of 128 tokens): the operands change places, so the TOKENS are the instruction's M side (the TMEM lanes)
// and the 128 features its columns. The loads and the main loop are the same; the epilogue's thread then owns a token
// row and finds consecutive features in its lane: 32-byte stores and 16-byte reductions instead of one element at a
// time, and the q/k/v form (EPI_QKV, heads of HD) can rotate a head and write it to its page from registers.
template <int TOK, int EPI, bool SWAP = false, int HD = 0>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
               const float* __restrict__ bias, void* __restrict__ out, int tokens, int n_out, int k_dim, int ldo,
               int splits, int kb_per_split, float* __restrict__ scratch, int* __restrict__ counters, int vec_ok,
               const QkvRows qe, unsigned long long* trace, int trace_cap) {
    static_assert(!SWAP || (TOK == BLOCK_F && EPI != EPI_SWIGLU), "the swapped form has tiles of 128 tokens and one accumulator");
    static_assert((EPI == EPI_QKV) == (HD != 0) && (EPI != EPI_QKV || SWAP), "the q/k/v epilogue owns token rows");
    constexpr bool DUAL = (EPI == EPI_SWIGLU);
    using C = Cfg<TOK, DUAL, HD>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + C::STAGES * C::STAGE_BYTES);
    unsigned long long* empty_bar = full_bar + C::STAGES;
    unsigned long long* acc_full_bar = empty_bar + C::STAGES;     // [2]
    unsigned long long* acc_empty_bar = acc_full_bar + 2;         // [2]
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty_bar + 2);
    float* tab_cos = reinterpret_cast<float*>(smem + C::OFF_TAB);            // [128][HD/2 + 1] (q/k/v form only)
    float* tab_sin = tab_cos + BLOCK_F * C::TAB_ROW;
    __shared__ volatile int s_failed;

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_GEMM_TC, EPI, 0);
    const int f_tiles = (n_out + BLOCK_F - 1) / BLOCK_F, t_tiles = (tokens + TOK - 1) / TOK;
    const int items = f_tiles * t_tiles * splits;       // work item = (output tile, split of K), splits fastest
    const int k_blocks = (k_dim + BLOCK_K - 1) / BLOCK_K;

    if (threadIdx.x == 0) {
        s_failed = 0;
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_a);
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full_bar[b], 1); mbar_init(&acc_empty_bar[b], 4); }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_wait();         // from here on the kernel reads what earlier kernels wrote (activations, the residual stream)
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_GEMM_TC, EPI, 1);

    if (warp == 0 && lane == 0) {
        // ---------------- producer: TMA loads of W (and the up rows) and A tiles, stage after stage across tiles
        int it = 0, issued = 0;
        for (int item = blockIdx.x; item < items && !s_failed; item += gridDim.x) {
            const int tile = item / splits, split = item - tile * splits;
            const int f0 = (tile % f_tiles) * BLOCK_F, t0 = (tile / f_tiles) * TOK;
            const int kb_end = min(k_blocks, (split + 1) * kb_per_split);
            for (int kb = split * kb_per_split; kb < kb_end; ++kb, ++it) {
                const int s = it % C::STAGES;
                if (!mbar_wait(&empty_bar[s], ((it / C::STAGES) & 1) ^ 1)) {
                    atomicCAS(&g_tc_error, 0, (1 << 16) | (int)blockIdx.x);
                    s_failed = 1;
                    break;
                }
                unsigned char* st = smem + s * C::STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
                tma_load_2d(st, &map_w, &full_bar[s], kb * BLOCK_K, f0);
                if (DUAL) tma_load_2d(st + C::W_BYTES, &map_w, &full_bar[s], kb * BLOCK_K, n_out + f0);
                tma_load_2d(st + (DUAL ? 2 : 1) * C::W_BYTES, &map_a, &full_bar[s], kb * BLOCK_K, t0);
                issued = it + 1;
            }
        }
        if (s_failed) {
            // copies already issued still target this CTA's shared memory: wait for them, bounded
            for (int i = max(0, issued - C::STAGES); i < issued; ++i)
                mbar_wait(&full_bar[i % C::STAGES], (i / C::STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        constexpr unsigned idesc = SWAP ? instr_desc(TOK, BLOCK_F) : instr_desc(BLOCK_F, TOK);
        int it = 0, local = 0;
        for (int item = blockIdx.x; item < items && !s_failed; item += gridDim.x, ++local) {
            const int buf = local & 1;
            const int split = item % splits;
            const int kb_begin = split * kb_per_split, kb_end = min(k_blocks, kb_begin + kb_per_split);
            // the epilogue has drained this buffer (two tiles ago)
            if (!mbar_wait(&acc_empty_bar[buf], ((local >> 1) & 1) ^ 1)) {
                atomicCAS(&g_tc_error, 0, (4 << 16) | (int)blockIdx.x);
                s_failed = 1;
                break;
            }
            tc_fence_after();
            const unsigned acc = tmem_base + buf * C::ACC_COLS;
            for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                const int s = it % C::STAGES;
                if (!mbar_wait(&full_bar[s], (it / C::STAGES) & 1)) {
                    atomicCAS(&g_tc_error, 0, (2 << 16) | (int)blockIdx.x);
                    s_failed = 1;
                    break;
                }
                tc_fence_after();
                const unsigned st = smem_u32(smem + s * C::STAGE_BYTES);
                const unsigned long long w_desc = desc_kmajor(st);
                const unsigned long long u_desc = desc_kmajor(st + C::W_BYTES);
                const unsigned long long a_desc = desc_kmajor(st + (DUAL ? 2 : 1) * C::W_BYTES);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const unsigned long long adv = (unsigned long long)((k * UMMA_K * 2) >> 4);   // 32 bytes per step
                    const bool accumulate = (kb > kb_begin) || (k > 0);
                    if (SWAP) tc_mma(acc, a_desc + adv, w_desc + adv, idesc, accumulate);
                    else tc_mma(acc, w_desc + adv, a_desc + adv, idesc, accumulate);
                    if (DUAL) tc_mma(acc + TOK, u_desc + adv, a_desc + adv, idesc, accumulate);
                }
                tc_commit(&empty_bar[s]);        // the stage is free when these MMAs have read it
            }
            if (s_failed) break;
            tc_commit(&acc_full_bar[buf]);       // the accumulator is complete when all MMAs are done
        }
    } else if (warp >= 2) {
        // ---------------- epilogue: TMEM -> registers -> global, one output feature per thread
        const int quad = warp & 3;                       // the TMEM lanes this warp may read: 32*quad..
        int local = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x, ++local) {
            const int buf = local & 1;
            const int tile = item / splits;
            const int f0 = (tile % f_tiles) * BLOCK_F, t0 = (tile / f_tiles) * TOK;
            const int f = f0 + quad * 32 + lane;
            // q/k/v form: what the epilogue reads besides the accumulator (the token's position and page, its rows of the
            // rotation tables, the tile's bias) is nobody's result: fetched while the tensor core still works on the tile
            int qkv_pos = 0;
            long long qkv_page = -1;
            if constexpr (EPI == EPI_QKV) {
                const int t = t0 + quad * 32 + lane;
                if (t < tokens) {
                    qkv_pos = __ldg(qe.positions + t);
                    if (qe.writes) {
                        qkv_page = __ldg(qe.block_table + (size_t)__ldg(qe.req_index + t) * qe.bt_stride + qkv_pos / qe.page_size);
                        if (qkv_page >= qe.num_pages) qkv_page = -1;      // never write outside the pool
                    }
                }
                if (qe.rotate) {
                    // the tables' rows of this warp's 32 tokens, read with the lanes along a row (coalesced)
                    __syncwarp();
                    const int rows_here = min(32, tokens - (t0 + quad * 32));          // warp-uniform
#pragma unroll 1
                    for (int r0 = 0; r0 < 32; r0 += 16) {
                        // sixteen rows' loads are issued before the first is stored: one wait for memory, not sixteen
                        float vc[16][HD / 64], vs[16][HD / 64];
#pragma unroll
                        for (int r = 0; r < 16; ++r) {
                            const int pos_r = __shfl_sync(0xffffffffu, qkv_pos, r0 + r);
#pragma unroll
                            for (int d = 0; d < HD / 64; ++d) {
                                vc[r][d] = r0 + r < rows_here ? __ldg(qe.cos_t + (size_t)pos_r * (HD / 2) + 32 * d + lane) : 0.f;
                                vs[r][d] = r0 + r < rows_here ? __ldg(qe.sin_t + (size_t)pos_r * (HD / 2) + 32 * d + lane) : 0.f;
                            }
                        }
#pragma unroll
                        for (int r = 0; r < 16; ++r)
#pragma unroll
                            for (int d = 0; d < HD / 64; ++d) {
                                tab_cos[(quad * 32 + r0 + r) * C::TAB_ROW + 32 * d + lane] = vc[r][d];
                                tab_sin[(quad * 32 + r0 + r) * C::TAB_ROW + 32 * d + lane] = vs[r][d];
                            }
                    }
                    __syncwarp();
                }
                if (bias != nullptr && lane < 4 && f0 + lane * 32 < n_out) asm volatile("prefetch.global.L1 [%0];\n" ::"l"(bias + f0 + lane * 32));
            }
            bool ok = !s_failed && mbar_wait(&acc_full_bar[buf], (local >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0 && !s_failed) { atomicCAS(&g_tc_error, 0, (3 << 16) | (int)blockIdx.x); s_failed = 1; }
                break;
            }
            tc_fence_after();
            const unsigned lane_addr = tmem_base + buf * C::ACC_COLS + ((unsigned)(quad * 32) << 16);
            if constexpr (SWAP) {
                // ---- this thread owns token row t; its lane holds the tile's 128 features
                const int t = t0 + quad * 32 + lane;
                const bool live = t < tokens;
                if constexpr (EPI == EPI_QKV) {
#pragma unroll 1
                    for (int c = 0; c < BLOCK_F; c += HD) {
                        if (f0 + c >= n_out) break;
                        emit_qkv_head<HD>(lane_addr + c, f0 + c, bias, (__nv_bfloat16*)out + (size_t)t * ldo, qe, qkv_pos, qkv_page, live,
                                          tab_cos + (quad * 32 + lane) * C::TAB_ROW, tab_sin + (quad * 32 + lane) * C::TAB_ROW);
                    }
                } else {
                    const float* item_bias = (item - tile * splits == 0) ? bias : nullptr;     // the bias is added once
#pragma unroll 1
                    for (int c = 0; c < BLOCK_F; c += 64) {
                        if (f0 + c >= n_out) break;
                        unsigned r[4][16];
#pragma unroll
                        for (int j = 0; j < 4; ++j) tmem_ld16_async(lane_addr + c + 16 * j, r[j]);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float v[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[j][i]);
                            if (live && f0 + c + 16 * j < n_out)
                                emit_row16<EPI>(out, v, v, item_bias, (size_t)t * ldo, f0 + c + 16 * j, n_out, vec_ok != 0);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
            } else {
            // ---- this thread owns output feature f; its lane holds the tile's tokens
            const float b = (bias != nullptr && f < n_out) ? bias[f] : 0.f;
            if (splits == 1) {
#pragma unroll 1
                for (int c = 0; c < TOK; c += 16) {
                    float v[16], u[16];
                    tmem_ld16(lane_addr + c, v);
                    if (DUAL) tmem_ld16(lane_addr + TOK + c, u);
                    if (f < n_out) emit16<EPI>(out, v, u, b, f, t0 + c, tokens, ldo);
                }
                // this warp has read its part of the buffer: hand it back to the MMA warp
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
                continue;
            }
            if (EPI == EPI_ADD) {
                // ---- split K into a 32-bit sum: every item adds its part, the first one the bias too
                const float b0 = (item - tile * splits == 0) ? b : 0.f;
                const int live = min(TOK, tokens - t0);
#pragma unroll 1
                for (int c = 0; c < live; c += 16) {
                    float v[16];
                    tmem_ld16(lane_addr + c, v);
                    if (f < n_out) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c + j < live) atomicAdd((float*)out + (size_t)(t0 + c + j) * ldo + f, v[j] + b0);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
                continue;
            }
            // ---- split K: leave the partial sums, count, and let the last warp of this quadrant finish the tile
            constexpr int ITEM_FLOATS = (DUAL ? 2 : 1) * TOK * BLOCK_F;
            const int live = min(TOK, tokens - t0);             // token rows of this tile that exist
            float* part = scratch + (size_t)item * ITEM_FLOATS + quad * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < live; c += 16) {
                float v[16], u[16];
                tmem_ld16(lane_addr + c, v);
                if (DUAL) tmem_ld16(lane_addr + TOK + c, u);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (c + j < live) {
                        __stcg(part + (size_t)(c + j) * BLOCK_F, v[j]);
                        if (DUAL) __stcg(part + (size_t)(TOK + c + j) * BLOCK_F, u[j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
            __threadfence();                                    // the partials are visible before the count
            __syncwarp();
            int last = 0;
            if (lane == 0) {
                last = (atomicAdd(&counters[tile * 4 + quad], 1) == splits - 1);
                if (last) counters[tile * 4 + quad] = 0;        // ready for the next launch
                __threadfence();
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (!last) continue;
            const float* first = scratch + (size_t)tile * splits * ITEM_FLOATS + quad * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < live; c += 16) {
                float v[16], u[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) { v[j] = 0.f; u[j] = 0.f; }
                for (int sp = 0; sp < splits; ++sp) {
                    const float* src = first + (size_t)sp * ITEM_FLOATS;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c + j < live) {
                            v[j] += __ldcg(src + (size_t)(c + j) * BLOCK_F);
                            if (DUAL) u[j] += __ldcg(src + (size_t)(TOK + c + j) * BLOCK_F);
                        }
                    }
                }
                if (f < n_out) emit16<EPI>(out, v, u, b, f, t0 + c, tokens, ldo);
            }
            }   // !SWAP
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_GEMM_TC, EPI, 2);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------- two SMs on one tile
// The product for many tokens (a prefill) with tcgen05.mma.cta_group::2, in the other orientation: the
// TOKENS are the M side (a cluster of two CTAs owns 256 of them, 128 TMEM lanes in each CTA), the output
// FEATURES are the N side (NT = 128 or 256 per tile). Each CTA loads its own 128 token rows and HALF of
// the weight rows of the tile; the instruction, issued by one thread of the even CTA, reads the weight
// operand from both CTAs' shared memory. Per CTA and step of K that is 16 KB of activations + NT/2 x 128
// bytes of weights for 128 x NT x 64 multiply-adds: half the traffic per flop of the one-CTA kernel, from
// L2 and from shared memory. A thread of the epilogue owns one token row and reads consecutive features
// from its TMEM lane, so it stores 32 contiguous bytes at a time (bfloat16), adds into the residual stream
// with 16-byte reductions, and takes the bias from broadcast loads.
//
// Fused SiLU(gate)*up: the 256 columns of a tile are the gate rows (loaded by the even CTA) and the up
// rows (loaded by the odd CTA) of the same 128 features, so every thread finds both values of a feature in
// its own lane.
//
// Who signals whom: both CTAs' TMA copies complete on the EVEN CTA's full barrier (it expects the bytes of
// both); tcgen05.commit multicasts to the empty barrier of the stage and to the accumulator-full barrier in
// both CTAs; the epilogue warps of both CTAs arrive on the even CTA's accumulator-empty barrier. No TMA
// multicast. The cluster meets at a hardware barrier twice, after the barriers are initialised and before
// tensor memory is freed; every other wait is bounded as above, so every thread reaches those two.
constexpr int PAIR_M = 256;      // tokens per cluster tile
constexpr int PAIR_THREADS = 320; // TMA warp, MMA warp, 8 epilogue warps: two per TMEM lane quadrant, half of the columns each

template <int NT> struct PairCfg {
    static constexpr int M_BYTES = BLOCK_F * BLOCK_K * 2;                 // this CTA's 128 token rows
    static constexpr int N_BYTES = (NT / 2) * BLOCK_K * 2;                // this CTA's half of the weight rows
    static constexpr int STAGE_BYTES = M_BYTES + N_BYTES;
    static constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 8 ? 8 : (200 * 1024 / STAGE_BYTES);
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
    static constexpr int TMEM_COLS = tmem_cols(2 * NT);                   // two accumulator buffers
    static_assert(2 * NT <= 512, "two accumulator buffers must fit the 512 TMEM columns");
};

// map_m: activations [tokens, K], box 64 x 128 rows; map_n: weights [rows, K], box 64 x NT/2 rows.
template <int NT, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_m, const __grid_constant__ CUtensorMap map_n,
                 const float* __restrict__ bias, void* __restrict__ out, int tokens, int n_out, int k_dim, int ldo, int vec_ok,
                 int splits, int kb_per_split, unsigned long long* trace, int trace_cap) {
    constexpr bool GU = (EPI == EPI_SWIGLU);                       // the tile's columns: gate rows | up rows of NT/2 features
    constexpr int FEAT = GU ? NT / 2 : NT;                         // output features per tile
    using C = PairCfg<NT>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + C::STAGES * C::STAGE_BYTES);
    unsigned long long* empty_bar = full_bar + C::STAGES;
    unsigned long long* acc_full_bar = empty_bar + C::STAGES;     // [2]
    unsigned long long* acc_empty_bar = acc_full_bar + 2;         // [2], used in the even CTA
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty_bar + 2);
    __shared__ volatile int s_failed;

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_GEMM_PAIR, EPI, 0);
    const unsigned rank = cluster_rank();                       // 0: issues the MMAs and owns the shared barriers
    const int n_tiles = (n_out + FEAT - 1) / FEAT, m_tiles = (tokens + PAIR_M - 1) / PAIR_M;
    // work item = (tile, split of K); splits fastest, feature tiles next. More than one split only with the
    // ADD epilogue: every item adds its partial sums into the output (reductions in memory).
    const int items = n_tiles * m_tiles * splits;
    const int k_blocks = (k_dim + BLOCK_K - 1) / BLOCK_K;
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        s_failed = 0;
        prefetch_tensormap(&map_m);
        prefetch_tensormap(&map_n);
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full_bar[b], 1); mbar_init(&acc_empty_bar[b], 16); }
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, C::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();            // the peer's barriers exist before anything signals them
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_wait();
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_GEMM_PAIR, EPI, 1);

    if (warp == 0 && lane == 0) {
        // ---------------- producer (in both CTAs): this CTA's 128 token rows and its half of the weight rows
        int it = 0;
        for (int item = cluster_id; item < items && !s_failed; item += n_clusters) {
            const int tile = item / splits, split = item - tile * splits;
            const int f0 = (tile % n_tiles) * FEAT, t0 = (tile / n_tiles) * PAIR_M + (int)rank * BLOCK_F;
            // weight rows: half of the tile's features, or (gate/up) the gate rows here and the up rows in the peer
            const int w0 = GU ? f0 + (int)rank * n_out : f0 + (int)rank * (NT / 2);
            const int kb_end = min(k_blocks, (split + 1) * kb_per_split);
            for (int kb = split * kb_per_split; kb < kb_end; ++kb, ++it) {
                const int s = it % C::STAGES;
                if (!mbar_wait(&empty_bar[s], ((it / C::STAGES) & 1) ^ 1)) {
                    atomicCAS(&g_tc_error, 0, (5 << 16) | (int)blockIdx.x);
                    s_failed = 1;
                    break;
                }
                unsigned char* st = smem + s * C::STAGE_BYTES;
                const unsigned bar0 = peer_smem(&full_bar[s], 0);
                if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);
                tma_load_2d_pair(st, &map_m, bar0, kb * BLOCK_K, t0);
                tma_load_2d_pair(st + C::M_BYTES, &map_n, bar0, kb * BLOCK_K, w0);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---------------- MMA issuer: one thread of the even CTA, for both
        constexpr unsigned idesc = instr_desc(PAIR_M, NT);
        int it = 0, local = 0;
        for (int item = cluster_id; item < items && !s_failed; item += n_clusters, ++local) {
            const int buf = local & 1;
            const int split = item % splits;
            const int kb_begin = split * kb_per_split, kb_end = min(k_blocks, kb_begin + kb_per_split);
            if (!mbar_wait(&acc_empty_bar[buf], ((local >> 1) & 1) ^ 1)) {
                atomicCAS(&g_tc_error, 0, (6 << 16) | (int)blockIdx.x);
                s_failed = 1;
                break;
            }
            tc_fence_after();
            const unsigned acc = tmem_base + buf * NT;
            for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                const int s = it % C::STAGES;
                if (!mbar_wait(&full_bar[s], (it / C::STAGES) & 1)) {
                    atomicCAS(&g_tc_error, 0, (7 << 16) | (int)blockIdx.x);
                    s_failed = 1;
                    break;
                }
                tc_fence_after();
                const unsigned st = smem_u32(smem + s * C::STAGE_BYTES);
                const unsigned long long m_desc = desc_kmajor(st);
                const unsigned long long n_desc = desc_kmajor(st + C::M_BYTES);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const unsigned long long adv = (unsigned long long)((k * UMMA_K * 2) >> 4);
                    tc_mma_pair(acc, m_desc + adv, n_desc + adv, idesc, (kb > kb_begin) || (k > 0));
                }
                tc_commit_pair(&empty_bar[s]);       // frees the stage in both CTAs
            }
            if (s_failed) break;
            tc_commit_pair(&acc_full_bar[buf]);      // the accumulators of both CTAs are complete
        }
    } else if (warp >= 2) {
        // ---------------- epilogue (in both CTAs): one token row per thread, half of the tile's features per warp
        const int quad = warp & 3;
        const int c_begin = ((warp - 2) >> 2) * (FEAT / 2), c_end = c_begin + FEAT / 2;
        const unsigned acc_empty0 = peer_smem(&acc_empty_bar[0], 0);
        int local = 0;
        for (int item = cluster_id; item < items; item += n_clusters, ++local) {
            const int buf = local & 1;
            const int tile = item / splits;
            const float* item_bias = (item - tile * splits == 0) ? bias : nullptr;     // the bias is added once
            const int f0 = (tile % n_tiles) * FEAT;
            const int t = (tile / n_tiles) * PAIR_M + (int)rank * BLOCK_F + quad * 32 + lane;
            bool ok = !s_failed && mbar_wait(&acc_full_bar[buf], (local >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0 && !s_failed) { atomicCAS(&g_tc_error, 0, (8 << 16) | (int)blockIdx.x); s_failed = 1; }
                break;
            }
            tc_fence_after();
            const unsigned lane_addr = tmem_base + buf * NT + ((unsigned)(quad * 32) << 16);
            const size_t row_off = (size_t)t * ldo;
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 16) {
                if (f0 + c >= n_out) break;
                float v[16], u[16];
                tmem_ld16(lane_addr + c, v);
                if (GU) tmem_ld16(lane_addr + FEAT + c, u);
                if (t < tokens) emit_row16<EPI>(out, v, u, item_bias, row_off, f0 + c, n_out, vec_ok != 0);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_peer(acc_empty0 + buf * 8);    // to the even CTA, from both
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_GEMM_PAIR, EPI, 2);
    cluster_sync();            // the peer no longer reads this CTA's shared memory or signals its barriers
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------- host side
// Map of a row-major bfloat16 matrix [rows, k] with row stride ld elements; box = 64 x box_rows, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, long long rows, long long k, long long ld, int box_rows) {
    NibEncodeTiledFn enc = nib_tensor_map_encoder();
    NIB_REQUIRE(enc != nullptr, "gemm (tensor cores): cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NIB_REQUIRE(r == CUDA_SUCCESS, "gemm (tensor cores): cuTensorMapEncodeTiled failed with code %d (rows=%lld k=%lld ld=%lld)", (int)r, rows, k, ld);
    return 0;
}

struct MapKey {
    const void* p; long long rows, k; int box;
    bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && k == o.k && box == o.box; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& x) const {
        return std::hash<const void*>()(x.p) ^ (std::hash<long long>()(x.rows) * 31) ^ (std::hash<long long>()(x.k) * 131) ^ (size_t)x.box;
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_weight_maps;   // weights live as long as the model
std::mutex g_map_mutex;

struct SplitK {
    int splits = 1;          // work items per output tile
    float* scratch = nullptr;
    int* counters = nullptr;
    long long scratch_floats = 0, counter_ints = 0;
};

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            sms = 1;
    }
    return sms;
}

template <int TOK, int EPI, bool SWAP = false, int HD = 0>
int launch_tc(const CUtensorMap& mw, const CUtensorMap& ma, const float* bias, void* out, int tokens, int n_out,
              int k, int ldo, const SplitK& sk, cudaStream_t stream, int vec_ok = 0, const QkvRows& qe = QkvRows{}) {
    using C = Cfg<TOK, EPI == EPI_SWIGLU, HD>;
    static bool configured = false;
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<TOK, EPI, SWAP, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured = true;
    }
    const int sms = sm_count();
    const int tiles = ceil_div(n_out, BLOCK_F) * ceil_div(tokens, TOK);
    const int k_blocks = ceil_div(k, BLOCK_K);
    int splits = sk.splits < 1 ? 1 : sk.splits;
    if (splits > k_blocks) splits = k_blocks;
    int kb_per_split = ceil_div(k_blocks, splits);
    splits = ceil_div(k_blocks, kb_per_split);               // no split without work
    NIB_REQUIRE(!SWAP || splits == 1 || EPI == EPI_ADD, "gemm (tensor cores): token-row tiles split K only for the sum into the output");
    if (splits > 1 && EPI != EPI_ADD) {
        const long long need = (long long)tiles * splits * (EPI == EPI_SWIGLU ? 2 : 1) * TOK * BLOCK_F;
        NIB_REQUIRE(sk.scratch != nullptr && sk.counters != nullptr && need <= sk.scratch_floats && 4LL * tiles <= sk.counter_ints,
                    "gemm (tensor cores): %d splits of %d tiles need %lld floats of scratch and %d counters (have %lld, %lld)",
                    splits, tiles, need, 4 * tiles, sk.scratch_floats, sk.counter_ints);
    }
    const int items = tiles * splits;
    NIB_CUDA(launch_pdl(gemm_tc_kernel<TOK, EPI, SWAP, HD>, dim3(items < sms ? items : sms), dim3(THREADS), (size_t)C::SMEM, stream,
                        mw, ma, bias, out, tokens, n_out, k, ldo, splits, kb_per_split, sk.scratch, sk.counters, vec_ok, qe,
                        nib_trace_buffer(), nib_trace_capacity()));
    return 0;
}

template <int TOK>
int launch_tc_epi(int epi, const CUtensorMap& mw, const CUtensorMap& ma, const float* bias, void* out, int tokens,
                  int n_out, int k, int ldo, const SplitK& sk, cudaStream_t stream) {
    switch (epi) {
        case EPI_STORE: return launch_tc<TOK, EPI_STORE>(mw, ma, bias, out, tokens, n_out, k, ldo, sk, stream);
        case EPI_ADD: return launch_tc<TOK, EPI_ADD>(mw, ma, bias, out, tokens, n_out, k, ldo, sk, stream);
        case EPI_F32: return launch_tc<TOK, EPI_F32>(mw, ma, bias, out, tokens, n_out, k, ldo, sk, stream);
        case EPI_SWIGLU:
            if constexpr (TOK <= 128) return launch_tc<TOK, EPI_SWIGLU>(mw, ma, bias, out, tokens, n_out, k, ldo, sk, stream);
            break;
    }
    nib_set_error("gemm (tensor cores): unknown epilogue %d", epi);
    return 1;
}

template <int NT, int EPI>
int launch_pair(const CUtensorMap& mm, const CUtensorMap& mn, const float* bias, void* out, int tokens, int n_out,
                int k, int ldo, int vec_ok, int splits, cudaStream_t stream) {
    using C = PairCfg<NT>;
    static bool configured = false;
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(gemm_pair_kernel<NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured = true;
    }
    const int feat = EPI == EPI_SWIGLU ? NT / 2 : NT;
    const int tiles = ceil_div(n_out, feat) * ceil_div(tokens, PAIR_M);
    const int k_blocks = ceil_div(k, BLOCK_K);
    if (EPI != EPI_ADD || splits < 1) splits = 1;
    if (splits > k_blocks) splits = k_blocks;
    const int kb_per_split = ceil_div(k_blocks, splits);
    splits = ceil_div(k_blocks, kb_per_split);
    int ctas = 2 * tiles * splits, most = sm_count() & ~1;
    if (ctas > most) ctas = most;
    NIB_CUDA(launch_pdl(gemm_pair_kernel<NT, EPI>, dim3(ctas), dim3(PAIR_THREADS), (size_t)C::SMEM, stream, mm, mn, bias, out,
                        tokens, n_out, k, ldo, vec_ok, splits, kb_per_split, nib_trace_buffer(), nib_trace_capacity()));
    return 0;
}

template <int NT>
int launch_pair_epi(int epi, const CUtensorMap& mm, const CUtensorMap& mn, const float* bias, void* out, int tokens,
                    int n_out, int k, int ldo, int vec_ok, int splits, cudaStream_t stream) {
    switch (epi) {
        case EPI_STORE: return launch_pair<NT, EPI_STORE>(mm, mn, bias, out, tokens, n_out, k, ldo, vec_ok, splits, stream);
        case EPI_ADD: return launch_pair<NT, EPI_ADD>(mm, mn, bias, out, tokens, n_out, k, ldo, vec_ok, splits, stream);
        case EPI_F32: return launch_pair<NT, EPI_F32>(mm, mn, bias, out, tokens, n_out, k, ldo, vec_ok, splits, stream);
        case EPI_SWIGLU: return launch_pair<NT, EPI_SWIGLU>(mm, mn, bias, out, tokens, n_out, k, ldo, vec_ok, splits, stream);
    }
    nib_set_error("gemm (tensor cores, two SMs per tile): unknown epilogue %d", epi);
    return 1;
}

}  // namespace

// 1 if the tensor-core kernel takes these operands: K a multiple of 8 (16-byte rows) and 16-byte aligned bases.
NIB_API int nib_gemm_tc_supported(const void* A, const void* W, int K, int lda) {
    if (K <= 0 || K % 8 || lda % 8) return 0;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return 0;
    return nib_tensor_map_encoder() != nullptr;
}

// The error word of the kernels' bounded waits: 0, or (role << 16 | block) of the first wait that ran
// out (role 1 producer, 2 MMA issuer, 3 epilogue). Reading it synchronises with the device; it is cleared.
NIB_API int nib_gemm_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    return v;
}

// A [tokens, K] bfloat16 with row stride lda; W [N, K] (SWIGLU: [2N, K]); out [tokens, N] with row
// stride ldo. epi: 0 store bf16, 1 add into float, 2 store float, 3 swiglu. tok_tile: 0 = chosen here.
// splits: work items per output tile along K; 0 = chosen here (more than one only when the tiles alone
// leave SMs idle and the scratch holds the partial sums), 1 = none. scratch/counters: a float buffer and
// a zeroed int buffer that the kernels of one stream share (the counters are left zeroed).
NIB_API int nib_gemm_tc_splitk(const void* A, const void* W, const float* bias, void* out, int tokens, int N, int K,
                               int lda, int ldo, int epi, int tok_tile, int splits, float* scratch, int* counters,
                               long long scratch_floats, long long counter_ints, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && N > 0 && K > 0 && lda >= K && ldo >= N, "gemm (tensor cores): bad sizes tokens=%d N=%d K=%d", tokens, N, K);
    NIB_REQUIRE(nib_gemm_tc_supported(A, W, K, lda), "gemm (tensor cores): K=%d / lda=%d must be multiples of 8 and bases 16-byte aligned", K, lda);
    NIB_REQUIRE(epi != EPI_SWIGLU || bias == nullptr, "gemm (tensor cores): the swiglu epilogue takes no bias");
    NIB_REQUIRE(splits >= 0, "gemm (tensor cores): splits=%d", splits);
    if (tokens == 0) return 0;
    const int f_tiles = ceil_div(N, BLOCK_F);
    if (tok_tile == 0) {
        tok_tile = tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64 : 128;
        // 256 tokens per tile halves the shared-memory traffic per flop; take it when the grid still fills the GPU
        if (tokens >= 512 && (long long)f_tiles * ceil_div(tokens, 256) >= 148 && epi != EPI_SWIGLU) tok_tile = 256;
        // 33..64 tokens with few feature tiles (a decode step of 64 requests): two tiles of 32 tokens put twice the
        // SMs on the weights, which are what the step has to stream (measured: 3.4 us a layer at the 0.5B widths).
        // The sum into the output can split K over CTAs instead, which reads large weights once (measured better from
        // about 16 MB of weights on: +8 % at the 7B widths, -2 % at the 0.5B widths).
        if (tok_tile == 64 && 2LL * f_tiles <= sm_count() && (epi != EPI_ADD || 2LL * N * K <= (16LL << 20))) tok_tile = 32;
    }
    NIB_REQUIRE(ceil_div(tokens, tok_tile) <= 65535, "gemm (tensor cores): too many token tiles");
    SplitK sk;
    sk.scratch = scratch; sk.counters = counters; sk.scratch_floats = scratch_floats; sk.counter_ints = counter_ints;
    sk.splits = splits;
    if (splits == 0) {
        // Fill the SMs: as many items as SMs, but at least 4 blocks of K (256 elements) per item, and only
        // what the scratch holds. The partial sums cost traffic of their own, so wide token tiles stay whole.
        const long long tiles = (long long)f_tiles * ceil_div(tokens, tok_tile);
        const int sms = sm_count(), k_blocks = ceil_div(K, BLOCK_K);
        int want = 1;
        if (tiles * 2 <= sms) {
            want = (int)(sms / tiles);
            if (want > k_blocks / 4) want = k_blocks / 4;
            if (epi != EPI_ADD) {
                // partial sums through the scratch: one warp adds them up, which pays for few tokens only
                const long long per_split = tiles * (epi == EPI_SWIGLU ? 2 : 1) * tok_tile * BLOCK_F;
                if (scratch == nullptr || counters == nullptr || tok_tile > 16 || 4 * tiles > counter_ints) want = 1;
                else if ((long long)want * per_split > scratch_floats) want = (int)(scratch_floats / per_split);
            }
            if (want < 1) want = 1;
        }
        sk.splits = want;
    }
    const long long w_rows = (epi == EPI_SWIGLU) ? 2LL * N : N;
    CUtensorMap mw, ma;
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        MapKey key{W, w_rows, K, BLOCK_F};
        auto it = g_weight_maps.find(key);
        if (it == g_weight_maps.end()) {
            if (make_map(&mw, W, w_rows, K, K, BLOCK_F)) return 1;
            if (g_weight_maps.size() > 4096) g_weight_maps.clear();
            g_weight_maps.emplace(key, mw);
        } else {
            mw = it->second;
        }
    }
    if (make_map(&ma, A, tokens, K, lda, tok_tile)) return 1;
    if (tok_tile == BLOCK_F && epi != EPI_SWIGLU && ((uintptr_t)bias & 15) == 0) {
        // tiles of 128 tokens: the token-row form (its epilogue writes rows, not columns). It splits K only for the sum.
        int splits_now = sk.splits < 1 ? 1 : sk.splits;
        if (epi == EPI_ADD || splits_now == 1) {
            const int elem = epi == EPI_STORE ? 2 : 4;
            const int vec_ok = (((uintptr_t)out & 15) == 0 && ((long long)ldo * elem) % 16 == 0) ? 1 : 0;
            switch (epi) {
                case EPI_STORE: return launch_tc<BLOCK_F, EPI_STORE, true>(mw, ma, bias, out, tokens, N, K, ldo, sk, stream, vec_ok);
                case EPI_ADD: return launch_tc<BLOCK_F, EPI_ADD, true>(mw, ma, bias, out, tokens, N, K, ldo, sk, stream, vec_ok);
                case EPI_F32: return launch_tc<BLOCK_F, EPI_F32, true>(mw, ma, bias, out, tokens, N, K, ldo, sk, stream, vec_ok);
            }
        }
    }
    switch (tok_tile) {
        case 16: return launch_tc_epi<16>(epi, mw, ma, bias, out, tokens, N, K, ldo, sk, stream);
        case 32: return launch_tc_epi<32>(epi, mw, ma, bias, out, tokens, N, K, ldo, sk, stream);
        case 64: return launch_tc_epi<64>(epi, mw, ma, bias, out, tokens, N, K, ldo, sk, stream);
        case 128: return launch_tc_epi<128>(epi, mw, ma, bias, out, tokens, N, K, ldo, sk, stream);
        case 256:
            NIB_REQUIRE(epi != EPI_SWIGLU, "gemm (tensor cores): the swiglu epilogue takes token tiles up to 128 (two accumulators, double buffered)");
            return launch_tc_epi<256>(epi, mw, ma, bias, out, tokens, N, K, ldo, sk, stream);
    }
    NIB_REQUIRE(false, "gemm (tensor cores): token tile %d is not one of 16, 32, 64, 128, 256", tok_tile);
}

// The same without split K (no scratch).
NIB_API int nib_gemm_tc(const void* A, const void* W, const float* bias, void* out, int tokens, int N, int K,
                        int lda, int ldo, int epi, int tok_tile, cudaStream_t stream) {
    return nib_gemm_tc_splitk(A, W, bias, out, tokens, N, K, lda, ldo, epi, tok_tile, 1, nullptr, nullptr, 0, 0, stream);
}

// 1 if nib_gemm_tc_qkv takes these sizes: heads of 64 or 128 that are rotated whole (rot == head_dim) or not at all,
// 16-byte aligned rows and bias.
NIB_API int nib_gemm_tc_qkv_supported(const void* A, const void* W, const void* bias, const void* qkv, int K, int lda,
                                      int ldq, int head_dim, int rot) {
    if (head_dim != 64 && head_dim != 128) return 0;
    if (rot != 0 && rot != head_dim) return 0;
    if (((uintptr_t)bias & 15) || ((uintptr_t)qkv & 15) || ldq % 8) return 0;
    return nib_gemm_tc_supported(A, W, K, lda);
}

// The q/k/v projection of a prompt portion with what follows it, in one kernel: qkv[tokens, (heads + 2 kv_heads) *
// head_dim] = A . W^T + bias; query and key heads rotated by positions[token] (tables of head_dim/2 values per
// position, halves paired) when rot == head_dim; the row stored to ``qkv``; with ``writes`` the rotated key and the
// value also into the slot of the token's position in its request's page (block_table[req_index[token]][position /
// page_size]; a negative entry is skipped). Tiles of 128 tokens x 128 features on one SM.
NIB_API int nib_gemm_tc_qkv(const void* A, const void* W, const float* bias, void* qkv, int tokens, int heads, int kv_heads,
                            int head_dim, int K, int lda, int ldq, const int* positions, const int* req_index,
                            const float* cos_t, const float* sin_t, int rot, const int* block_table, int bt_stride,
                            int page_size, void* k_pages, void* v_pages, int num_pages, int writes, cudaStream_t stream) {
    const int N = (heads + 2 * kv_heads) * head_dim;
    NIB_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && K > 0 && lda >= K && ldq >= N, "gemm (tensor cores, q/k/v): bad sizes");
    NIB_REQUIRE(nib_gemm_tc_qkv_supported(A, W, bias, qkv, K, lda, ldq, head_dim, rot),
                "gemm (tensor cores, q/k/v): needs heads of 64 or 128 rotated whole or not at all, K %% 8 == 0 and 16-byte aligned rows (head_dim=%d rot=%d K=%d)", head_dim, rot, K);
    NIB_REQUIRE(rot == 0 || (cos_t && sin_t), "gemm (tensor cores, q/k/v): rotation needs the tables");
    NIB_REQUIRE(positions && req_index, "gemm (tensor cores, q/k/v): positions and request rows are needed");
    NIB_REQUIRE(!writes || (block_table && k_pages && v_pages && page_size > 0 && num_pages > 0), "gemm (tensor cores, q/k/v): writing needs pages and a block table");
    if (tokens == 0) return 0;
    CUtensorMap mw, ma;
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        MapKey key{W, N, K, BLOCK_F};
        auto it = g_weight_maps.find(key);
        if (it == g_weight_maps.end()) {
            if (make_map(&mw, W, N, K, K, BLOCK_F)) return 1;
            if (g_weight_maps.size() > 4096) g_weight_maps.clear();
            g_weight_maps.emplace(key, mw);
        } else {
            mw = it->second;
        }
    }
    if (make_map(&ma, A, tokens, K, lda, BLOCK_F)) return 1;
    SplitK sk;
    QkvRows qe{heads, kv_heads, rot != 0 ? 1 : 0, positions, req_index, cos_t, sin_t, block_table, bt_stride, page_size,
               num_pages, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, writes};
    if (head_dim == 64) return launch_tc<BLOCK_F, EPI_QKV, true, 64>(mw, ma, bias, qkv, tokens, N, K, ldq, sk, stream, 1, qe);
    return launch_tc<BLOCK_F, EPI_QKV, true, 128>(mw, ma, bias, qkv, tokens, N, K, ldq, sk, stream, 1, qe);
}

// The product for many tokens by pairs of SMs (tcgen05.mma.cta_group::2): tiles of 256 tokens x n_tile
// output features (128 or 256; 0 = 256). splits: work items along K per tile, for the ADD epilogue only
// (0 = chosen here: enough to give every pair of SMs an item, at least 8 blocks of K each; 1 = none).
NIB_API int nib_gemm_tc_pair(const void* A, const void* W, const float* bias, void* out, int tokens, int N, int K,
                             int lda, int ldo, int epi, int n_tile, int splits, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && N > 0 && K > 0 && lda >= K && ldo >= N, "gemm (two SMs per tile): bad sizes tokens=%d N=%d K=%d", tokens, N, K);
    NIB_REQUIRE(nib_gemm_tc_supported(A, W, K, lda), "gemm (two SMs per tile): K=%d / lda=%d must be multiples of 8 and bases 16-byte aligned", K, lda);
    NIB_REQUIRE(epi != EPI_SWIGLU || bias == nullptr, "gemm (two SMs per tile): the swiglu epilogue takes no bias");
    NIB_REQUIRE(epi >= EPI_STORE && epi <= EPI_SWIGLU, "gemm (two SMs per tile): unknown epilogue %d", epi);
    NIB_REQUIRE(((uintptr_t)bias & 15) == 0, "gemm (two SMs per tile): the bias must be 16-byte aligned");
    if (tokens == 0) return 0;
    if (n_tile == 0) n_tile = 256;      // measured: the instruction of 128 columns runs at about half the rate, whatever the grid
    NIB_REQUIRE(n_tile == 128 || n_tile == 256, "gemm (two SMs per tile): feature tile %d is not 128 or 256", n_tile);
    // 16-byte stores and reductions need rows of the output that start on 16 bytes
    const int elem = (epi == EPI_STORE || epi == EPI_SWIGLU) ? 2 : 4;
    const int vec_ok = (((uintptr_t)out & 15) == 0 && ((long long)ldo * elem) % 16 == 0) ? 1 : 0;
    const long long w_rows = (epi == EPI_SWIGLU) ? 2LL * N : N;
    CUtensorMap mm, mn;
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        MapKey key{W, w_rows, K, n_tile / 2};
        auto it = g_weight_maps.find(key);
        if (it == g_weight_maps.end()) {
            if (make_map(&mn, W, w_rows, K, K, n_tile / 2)) return 1;
            if (g_weight_maps.size() > 4096) g_weight_maps.clear();
            g_weight_maps.emplace(key, mn);
        } else {
            mn = it->second;
        }
    }
    if (make_map(&mm, A, tokens, K, lda, BLOCK_F)) return 1;
    NIB_REQUIRE(splits >= 0, "gemm (two SMs per tile): splits=%d", splits);
    if (splits == 0) {
        const int tiles = ceil_div(N, n_tile) * ceil_div(tokens, PAIR_M), clusters = sm_count() / 2;
        splits = 1;
        if (epi == EPI_ADD && tiles < clusters) {
            splits = clusters / tiles;
            const int most = ceil_div(K, BLOCK_K) / 8;
            if (splits > most) splits = most;
            if (splits < 1) splits = 1;
        }
    }
    if (n_tile == 128) return launch_pair_epi<128>(epi, mm, mn, bias, out, tokens, N, K, ldo, vec_ok, splits, stream);
    return launch_pair_epi<256>(epi, mm, mn, bias, out, tokens, N, K, ldo, vec_ok, splits, stream);
}
