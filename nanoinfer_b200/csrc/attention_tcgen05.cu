// Paged causal attention for prompt portions on the 5th-generation tensor cores (tcgen05 + TMEM), for
// bfloat16 and head sizes 64 and 128.
//
// A CTA owns a tile of up to 128 rows, where a row is one (token, query head of the kv group): the keys
// and values of a kv head are read once for all the query heads that share it. For every block of 128
// keys:   S = Q . K^T      (tcgen05.mma, accumulator S in TMEM)
//         P = exp2(S*scale - max), row sums       (two threads per row: no shuffles, one exchange of maxima)
//         O_blk = P . V    (tcgen05.mma, P from shared memory, V as the MN-major operand)
//         O = O * corr + O_blk                     (registers, 32-bit)
// S and O_blk are double buffered in TMEM: the scores of block j+1 are computed while the softmax of
// block j runs.
// Q, K and V tiles arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle): Q through a 3-D map over
// (head dim, heads of the group, tokens), K and V through a 3-D map over the page pool, one box per
// page of the block table; a page the request does not hold is fetched from an out-of-range coordinate
// and arrives as zeros. Roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2..5 =
// softmax and output (eight warps: the 128 keys of a block and the head dim are split between two threads
// per row, so that every scheduler has two warps to alternate between). Every wait is bounded; a wait that runs out records an error word, the CTA stops,
// drains its copies, frees its TMEM and returns.
//
// Formula as in attention_generic.cu (cpp/src/ops.cpp:206-270); the reference's prefill attention is a
// SIMT kernel with 32-key shared-memory slabs (cpp/src/cuda/cuda_backend.cu:489-575).
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace {

constexpr int ROWS = 128;        // rows of a tile (UMMA M): TMEM lanes
constexpr int KEYS = 128;        // keys per block (UMMA N of S, K of P.V)
constexpr int THREADS = 320;     // TMA warp, MMA warp, eight softmax warps (two threads per row)
constexpr unsigned WAIT_LIMIT = 1u << 22;
constexpr float LOG2E = 1.4426950408889634f;

__device__ int g_attn_error = 0;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    // hand-overs between the roles are short: spin first, back off only when a wait drags on
    for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (i > 4096) __nanosleep(100);
    }
    return false;
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, unsigned long long* bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tmem_alloc(unsigned* dst_smem, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(unsigned addr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                       unsigned idesc, bool accumulate) {
    const unsigned acc = accumulate ? 1u : 0u;
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// 32 columns of this thread's TMEM lane; the values may be used only after tmem_wait_ld().
__device__ __forceinline__ void tmem_ld32_async(unsigned addr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
}
// K-major operand tile with the 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ unsigned long long desc_kmajor(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// MN-major operand with the 128-byte swizzle (cute/atom/mma_traits_sm100.hpp, canonical layout
// ((8,n),(8,k)):((1,LBO),(8,SBO)) in 16-byte units): 64 elements of MN are contiguous in a 128-byte row,
// 8 rows of K form a 1024-byte group (SBO), the next 64 elements of MN start `lbo_bytes` further on.
__device__ __forceinline__ unsigned long long desc_mnmajor(unsigned smem_addr, unsigned lbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// D float, A and B bfloat16, M = 128, N = n; b_mn: the B operand is MN-major.
__host__ __device__ constexpr unsigned instr_desc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) | ((unsigned)(ROWS >> 4) << 24);
}

template <int HD> struct Cfg {
    static constexpr int SUB = HD / 64;                       // sub-tiles of 64 elements (128 bytes) along the head dim
    static constexpr int SUBTILE = 128 * 128;                 // bytes of a [128 rows x 64 elements] sub-tile
    static constexpr int Q_BYTES = SUB * SUBTILE;
    static constexpr int KV_BYTES = SUB * SUBTILE;            // one block of 128 keys (or values)
    static constexpr int P_BYTES = 2 * SUBTILE;               // [128 rows x 128 keys]
    static constexpr int OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_P = OFF_V + 2 * KV_BYTES;
    static constexpr int OFF_BAR = OFF_P + P_BYTES;
    static constexpr int OFF_XCH = OFF_BAR + 256;                // [2][2][128] floats: partial row maxima (and sums)
    static constexpr int SMEM = OFF_XCH + 2 * 2 * 128 * 4 + 1024;
    static constexpr int TMEM_COLS = 512;                     // S x2 (256 columns) + O block x2 (2 x HD)
    static constexpr int COL_S = 0, COL_O = 256;
    static constexpr int CTAS_PER_SM = 1;
};

// grid: (row tiles, requests, kv heads)
template <int HD>
__global__ void __launch_bounds__(THREADS, Cfg<HD>::CTAS_PER_SM)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
                            const int* __restrict__ block_table, int bt_stride, int page_size, int num_pages,
                            int heads, int kv_heads, float scale, int window) {
    using C = Cfg<HD>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + C::OFF_BAR);
    unsigned long long* q_full = bars;            // 1
    unsigned long long* k_full = bars + 1;        // 2
    unsigned long long* k_empty = bars + 3;       // 2
    unsigned long long* v_full = bars + 5;        // 2
    unsigned long long* v_empty = bars + 7;       // 2
    unsigned long long* s_full = bars + 9;        // 2
    unsigned long long* p_full = bars + 11;       // 2, 128 arrivals each
    unsigned long long* o_full = bars + 13;       // 2
    unsigned long long* xch_bar = bars + 15;      // 2, 256 arrivals each: the two halves of a row have exchanged their maxima
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 17);
    float* xch = reinterpret_cast<float*>(smem + C::OFF_XCH);
    __shared__ volatile int s_failed;

    pdl_launch_dependents();
    const int req = blockIdx.y, kvh = blockIdx.z;
    const int n_rep = heads / kv_heads;
    const int tpt = ROWS / n_rep;                         // tokens per tile
    const int rows_tile = tpt * n_rep;
    const int row_begin = q_start[req], q_len = q_start[req + 1] - row_begin;
    // tiles late in the portion see the most keys: they start first
    const int tok0 = (gridDim.x - 1 - blockIdx.x) * tpt;  // first token of this tile within the request's portion
    if (tok0 >= q_len) return;
    const int n_tok = min(tpt, q_len - tok0);
    const int ctx = ctx_lens[req];
    const int pos0 = ctx - q_len + tok0;                  // position of the tile's first token
    const int hi_cta = pos0 + n_tok - 1;
    const int lo_cta = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int b_begin = lo_cta / KEYS, b_end = hi_cta / KEYS, n_blk = b_end - b_begin + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* bt = block_table + (size_t)req * bt_stride;

    if (threadIdx.x == 0) {
        s_failed = 0;
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 256);
            mbar_init(&xch_bar[i], 256);
            mbar_init(&o_full[i], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_wait();

    if (warp == 0) {
        // ---------------- producer: lane 0 fetches Q and arms the barriers; lane i fetches page i of every
        // block of 128 keys (its block-table entry is read one block ahead, so that the look-up of a page
        // never stands between two copies)
        if (lane == 0) {
            mbar_expect_tx(q_full, (unsigned)(rows_tile * 128 * C::SUB));
#pragma unroll
            for (int s = 0; s < C::SUB; ++s)
                tma_load_3d(smem + C::OFF_Q + s * C::SUBTILE, &map_q, q_full, s * 64, kvh * n_rep, row_begin + tok0);
        }
        const int pages_per_block = KEYS / page_size;
        const int oob = num_pages * kv_heads;             // a coordinate outside the pool: the box arrives as zeros
        auto plane_of = [&](int j) -> int {               // third coordinate of this lane's page in block j
            const int key = (b_begin + j) * KEYS + lane * page_size;
            if (lane >= pages_per_block || key > hi_cta || key + page_size <= lo_cta) return oob;
            const int page = __ldg(bt + key / page_size);
            return (page >= 0 && page < num_pages) ? page * kv_heads + kvh : oob;
        };
        int z_next = plane_of(0);
        int issued = 0;
        for (int j = 0; j < n_blk; ++j) {
            const int st = j & 1;
            const int z = z_next;
            if (j + 1 < n_blk) z_next = plane_of(j + 1);
            int ok = 1;
            if (lane == 0) {
                const unsigned par = ((j >> 1) & 1) ^ 1;
                ok = !s_failed && mbar_wait(&k_empty[st], par) && mbar_wait(&v_empty[st], par);
                if (ok) {
                    mbar_expect_tx(&k_full[st], C::KV_BYTES);
                    mbar_expect_tx(&v_full[st], C::KV_BYTES);
                } else if (!s_failed) {
                    atomicCAS(&g_attn_error, 0, (1 << 16) | (int)blockIdx.x);
                    s_failed = 1;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < pages_per_block) {
#pragma unroll
                for (int s = 0; s < C::SUB; ++s) {
                    tma_load_3d(smem + C::OFF_K + st * C::KV_BYTES + s * C::SUBTILE + lane * page_size * 128, &map_k, &k_full[st], s * 64, 0, z);
                    tma_load_3d(smem + C::OFF_V + st * C::KV_BYTES + s * C::SUBTILE + lane * page_size * 128, &map_v, &v_full[st], s * 64, 0, z);
                }
            }
            issued = j + 1;
        }
        if (s_failed && lane == 0) {
            // copies already issued still target this CTA's shared memory: wait for them, bounded
            mbar_wait(q_full, 0);
            for (int j = max(0, issued - 2); j < issued; ++j) {
                mbar_wait(&k_full[j & 1], (j >> 1) & 1);
                mbar_wait(&v_full[j & 1], (j >> 1) & 1);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer: QK(0), QK(1), PV(0), QK(2), PV(1), ...
        constexpr unsigned idesc_s = instr_desc(KEYS, false);
        constexpr unsigned idesc_o = instr_desc(HD, true);
        const unsigned q_addr = smem_u32(smem + C::OFF_Q), p_addr = smem_u32(smem + C::OFF_P);
        bool ok = mbar_wait(q_full, 0);
        if (!ok) { atomicCAS(&g_attn_error, 0, (2 << 16) | (int)blockIdx.x); s_failed = 1; }
        auto issue_pv = [&](int j) -> bool {
            const int st = j & 1;
            if (!mbar_wait(&p_full[st], (j >> 1) & 1) || !mbar_wait(&v_full[st], (j >> 1) & 1)) return false;
            tc_fence_after();
            const unsigned v_addr = smem_u32(smem + C::OFF_V + st * C::KV_BYTES);
            const unsigned pj_addr = p_addr;      // one P tile: the softmax of block j+1 starts after P_j . V_j was collected
#pragma unroll
            for (int kk = 0; kk < KEYS / 16; ++kk) {
                // P: sub-tile kk/4 (64 keys each), 32 bytes per step inside it; V: 16 keys = 2048 bytes further down
                const unsigned long long a = desc_kmajor(pj_addr + (kk >> 2) * C::SUBTILE) + (unsigned long long)(((kk & 3) * 32) >> 4);
                const unsigned long long b = desc_mnmajor(v_addr + kk * 16 * 128, C::SUBTILE);
                tc_mma(tmem_base + C::COL_O + st * HD, a, b, idesc_o, kk > 0);
            }
            tc_commit(&o_full[st]);
            tc_commit(&v_empty[st]);
            return true;
        };
        auto issue_qk = [&](int j) -> bool {
            const int st = j & 1;
            if (!mbar_wait(&k_full[st], (j >> 1) & 1)) return false;
            tc_fence_after();
            const unsigned k_addr = smem_u32(smem + C::OFF_K + st * C::KV_BYTES);
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const unsigned sub = (kk >> 2) * C::SUBTILE;
                const unsigned long long adv = (unsigned long long)(((kk & 3) * 32) >> 4);
                tc_mma(tmem_base + C::COL_S + st * KEYS, desc_kmajor(q_addr + sub) + adv, desc_kmajor(k_addr + sub) + adv, idesc_s, kk > 0);
            }
            tc_commit(&s_full[st]);
            tc_commit(&k_empty[st]);
            return true;
        };
        // QK(0), QK(1), PV(0), QK(2), PV(1), ...: S[b] is free for QK(j+2) once P_j is complete (PV(j) waited for it)
        if (ok) ok = issue_qk(0);
        for (int j = 0; j < n_blk && ok; ++j) {
            if (j + 1 < n_blk) ok = issue_qk(j + 1);
            if (ok) ok = issue_pv(j);
        }
        if (!ok && !s_failed) { atomicCAS(&g_attn_error, 0, (3 << 16) | (int)blockIdx.x); s_failed = 1; }
    } else if (warp >= 2) {
        // ---------------- softmax and output: two threads per row. `half` 0 takes keys 0..63 of every block
        // and output columns 0..HD/2-1, `half` 1 the rest; a warp may read the TMEM lanes 32*(warp%4)...
        constexpr int HK = KEYS / 2, HO = HD / 2;
        const int half = (warp - 2) >> 2, quad = warp & 3, row = quad * 32 + lane;
        const unsigned lane_addr = tmem_base + ((unsigned)(quad * 32) << 16);
        const bool live = row < n_tok * n_rep;
        const int ti = row / n_rep, head = kvh * n_rep + (row - ti * n_rep);
        const int hi = live ? pos0 + ti : -1;
        const int lo = window > 0 ? max(0, hi - window + 1) : 0;
        const float scale2 = scale * LOG2E;
        float m_run = -INFINITY, l_run = 0.f;       // l_run: the sum over this thread's half of the keys
        float o[HO];
#pragma unroll
        for (int d = 0; d < HO; ++d) o[d] = 0.f;
        // this thread's half of the row in P: sub-tile `half` (64 keys), row `row`
        unsigned char* p_row = smem + C::OFF_P + half * C::SUBTILE + (row >> 3) * 1024 + (row & 7) * 128;
        bool ok = true;
        unsigned raw[2][32];                      // this thread's 64 scores of the block in work
        float m_use = 0.f, corr = 0.f;            // of the block in work

        // First half of a block's softmax: scores from TMEM, mask, the row's maximum (exchanged with the
        // thread that holds the other 64 keys), running max and the factor for the running output.
        auto scores_and_max = [&](int j) -> bool {
            const int sb = j & 1;
            bool good = !s_failed && mbar_wait(&s_full[sb], (j >> 1) & 1);
            good = __all_sync(0xffffffffu, good);
            if (!good) return false;
            tc_fence_after();
            const int key0 = (b_begin + j) * KEYS + half * HK;
            const unsigned s_addr = lane_addr + C::COL_S + sb * KEYS + half * HK;
            const bool all_visible = key0 >= lo && key0 + HK - 1 <= hi;       // no mask needed for this thread's keys
            tmem_ld32_async(s_addr, raw[0]);
            tmem_ld32_async(s_addr + 32, raw[1]);
            tmem_wait_ld();
            float mx = -INFINITY;
            if (all_visible) {
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(raw[c][i]));
            } else {
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = key0 + c * 32 + i;
                        if (!(key >= lo && key <= hi)) raw[c][i] = 0xff800000u;      // -inf
                        mx = fmaxf(mx, __uint_as_float(raw[c][i]));
                    }
            }
            xch[(sb * 2 + half) * 128 + row] = mx;
            mbar_arrive(&xch_bar[sb]);
            good = mbar_wait(&xch_bar[sb], (j >> 1) & 1);
            good = __all_sync(0xffffffffu, good);
            if (!good) return false;
            mx = fmaxf(mx, xch[(sb * 2 + (half ^ 1)) * 128 + row]) * scale2;   // scale2 > 0
            const float m_new = fmaxf(m_run, mx);
            m_use = (m_new == -INFINITY) ? 0.f : m_new;
            corr = (m_run == -INFINITY) ? 0.f : ex2(m_run - m_use);
            m_run = m_new;
            return true;
        };

        ok = scores_and_max(0);
        for (int j = 0; j < n_blk && ok; ++j) {
            const int sb = j & 1;
            // second half: probabilities of block j into P, their sum
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                unsigned pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = ex2(fmaf(__uint_as_float(raw[c][i]), scale2, -m_use));       // ex2(-inf) = 0
                    const float p1 = ex2(fmaf(__uint_as_float(raw[c][i + 1]), scale2, -m_use));
                    sum += p0 + p1;
                    __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    pk[i >> 1] = *reinterpret_cast<unsigned*>(&h);
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = (c << 2) + q4;                         // 16-byte chunk within the 128-byte row
                    *reinterpret_cast<uint4*>(p_row + ((chunk ^ (row & 7)) << 4)) =
                        make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
                }
            }
            l_run = l_run * corr + sum;
            const float corr_j = corr;
            // P is read by the tensor core through the async proxy
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            tc_fence_before();
            mbar_arrive(&p_full[sb]);
            // while the tensor core multiplies P_j by V_j: the scores and the maximum of block j+1
            if (j + 1 < n_blk) { ok = scores_and_max(j + 1); if (!ok) break; }
            // O = O * corr_j + P_j . V_j, this thread's half of the columns
            ok = mbar_wait(&o_full[sb], (j >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            {
                unsigned ov[HO / 32][32];
#pragma unroll
                for (int c = 0; c < HO / 32; ++c) tmem_ld32_async(lane_addr + C::COL_O + sb * HD + half * HO + c * 32, ov[c]);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < HO / 32; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], corr_j, __uint_as_float(ov[c][i]));
            }
            tc_fence_before();
        }
        // the row's sum: both halves. The exchange buffers alternate with the blocks; use the next one.
        if (ok) {
            const int sb = n_blk & 1;
            xch[(sb * 2 + half) * 128 + row] = l_run;
            mbar_arrive(&xch_bar[sb]);
            ok = mbar_wait(&xch_bar[sb], (n_blk >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) l_run += xch[(sb * 2 + (half ^ 1)) * 128 + row];
        }
        if (!ok) {
            if (lane == 0 && !s_failed) { atomicCAS(&g_attn_error, 0, (4 << 16) | (int)blockIdx.x); s_failed = 1; }
        } else if (live) {
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            __nv_bfloat16* orow = out + ((size_t)(row_begin + tok0 + ti) * heads + head) * HD + half * HO;
#pragma unroll
            for (int d = 0; d < HO; d += 8) {
                uint4 w;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(o[d] * inv, o[d + 1] * inv), h1 = __floats2bfloat162_rn(o[d + 2] * inv, o[d + 3] * inv);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(o[d + 4] * inv, o[d + 5] * inv), h3 = __floats2bfloat162_rn(o[d + 6] * inv, o[d + 7] * inv);
                w.x = *reinterpret_cast<unsigned*>(&h0); w.y = *reinterpret_cast<unsigned*>(&h1);
                w.z = *reinterpret_cast<unsigned*>(&h2); w.w = *reinterpret_cast<unsigned*>(&h3);
                *reinterpret_cast<uint4*>(orow + d) = w;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 3-D map over bfloat16 data: dims (d0 innermost), strides in elements for d1 and d2, box (64, b1, b2).
int make_map3(CUtensorMap* map, const void* ptr, long long d0, long long d1, long long d2, long long s1, long long s2,
              int b1, int b2) {
    EncodeTiledFn enc = get_encode();
    NIB_REQUIRE(enc != nullptr, "attention (tcgen05): cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2};
    cuuint64_t strides[2] = {(cuuint64_t)s1 * 2, (cuuint64_t)s2 * 2};
    cuuint32_t box[3] = {64u, (cuuint32_t)b1, (cuuint32_t)b2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NIB_REQUIRE(r == CUDA_SUCCESS, "attention (tcgen05): cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, const int* q_start,
           const int* ctx_lens, const int* block_table, int bt_stride, int page_size, int num_pages, int n_req,
           int max_q_len, int heads, int kv_heads, float scale, int window, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<HD>::SMEM));
        configured = true;
    }
    const int tpt = ROWS / (heads / kv_heads);
    dim3 grid(ceil_div(max_q_len, tpt), n_req, kv_heads);
    NIB_CUDA(launch_pdl(attention_prefill_tc_kernel<HD>, grid, dim3(THREADS), (size_t)Cfg<HD>::SMEM, stream, mq, mk, mv,
                        (__nv_bfloat16*)out, q_start, ctx_lens, block_table, bt_stride, page_size, num_pages, heads,
                        kv_heads, scale, window));
    return 0;
}

}  // namespace

// 1 if the tcgen05 kernel takes this shape: head size 64 or 128, at most 128 query heads per kv head,
// pages of 8..128 tokens that divide 128, 16-byte aligned rows.
NIB_API int nib_attention_prefill_tc_supported(int heads, int kv_heads, int head_dim, int page_size, int q_stride) {
    if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > ROWS) return 0;
    if (head_dim != 64 && head_dim != 128) return 0;
    if (page_size < 8 || page_size > KEYS || KEYS % page_size) return 0;
    if (q_stride % 8) return 0;
    return get_encode() != nullptr;
}

// The error word of the kernel's bounded waits (0 = none); synchronises with the device and clears it.
NIB_API int nib_attention_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
    return v;
}

// Same arguments as nib_attention_prefill_mma plus the number of rows of qkv (m_tokens, for the map's extent).
NIB_API int nib_attention_prefill_tc(const void* qkv, int q_stride, void* out, const int* q_start, const int* ctx_lens,
                                     const int* block_table, int bt_stride, int page_size, const void* k_pages,
                                     const void* v_pages, int num_pages, int n_req, int max_q_len, int m_tokens,
                                     int heads, int kv_heads, int head_dim, float scale, int window,
                                     cudaStream_t stream) {
    NIB_REQUIRE(nib_attention_prefill_tc_supported(heads, kv_heads, head_dim, page_size, q_stride),
                "attention (tcgen05): head_dim %d, %d/%d heads, page size %d are not supported", head_dim, heads, kv_heads, page_size);
    NIB_REQUIRE(n_req >= 0 && max_q_len > 0 && num_pages > 0 && window >= 0 && m_tokens > 0, "attention (tcgen05): bad sizes");
    NIB_REQUIRE((((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)out) & 15) == 0, "attention (tcgen05): bases must be 16-byte aligned");
    NIB_REQUIRE(n_req <= 65535 && kv_heads <= 65535, "attention (tcgen05): too many requests or kv heads for one launch");
    if (n_req == 0) return 0;
    const int n_rep = heads / kv_heads, tpt = ROWS / n_rep;
    CUtensorMap mq, mk, mv;
    // queries: (head dim, heads, tokens); a box is 64 x n_rep heads x tpt tokens
    if (make_map3(&mq, qkv, head_dim, heads, m_tokens, head_dim, q_stride, n_rep, tpt)) return 1;
    // pool: (head dim, slot in page, page * kv_heads + kv head); a box is one page of one kv head
    const long long planes = (long long)num_pages * kv_heads;
    if (make_map3(&mk, k_pages, head_dim, page_size, planes, head_dim, (long long)page_size * head_dim, page_size, 1)) return 1;
    if (make_map3(&mv, v_pages, head_dim, page_size, planes, head_dim, (long long)page_size * head_dim, page_size, 1)) return 1;
    if (head_dim == 64)
        return launch<64>(mq, mk, mv, out, q_start, ctx_lens, block_table, bt_stride, page_size, num_pages, n_req, max_q_len,
                          heads, kv_heads, scale, window, stream);
    return launch<128>(mq, mk, mv, out, q_start, ctx_lens, block_table, bt_stride, page_size, num_pages, n_req, max_q_len,
                       heads, kv_heads, scale, window, stream);
}
