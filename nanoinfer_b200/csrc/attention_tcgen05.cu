// Paged causal attention for prompt portions on the 5th-generation tensor cores (tcgen05 + TMEM), for
// bfloat16 and head sizes 64 and 128.
//
// A CTA owns a tile of up to 128 rows, where a row is one (token, query head of the kv group): the keys and
// values of a kv head are read once for all the query heads that share it. For every block of 128 (heads of
// 128: 64) keys:
//         S = Q . K^T         (tcgen05.mma, accumulator S in tensor memory, two buffers)
//         P = exp2(S*scale - max), row sums       (a thread per row: no exchange between threads)
//         O += P . V          (tcgen05.mma, P from shared memory (two buffers), V as the MN-major operand; O
//                              stays in tensor memory over all blocks)
// The scores of block j+1 are multiplied while the softmax of block j runs, and P.V of block j while the softmax
// of block j+1 runs: the softmax warps, which bound the kernel (exponentials), never wait for the tensor core.
// The running maximum that the exponents refer to is only replaced when the row's maximum grew by more than
// 2^8; only then is the row of O rescaled (read from tensor memory, multiplied, written back). At the end O is
// read once and divided by the sum.
// Q, K and V tiles arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle): Q through a 3-D map over
// (head dim, heads of the group, tokens), K and V through a 3-D map over the page pool, one box per
// page of the block table; a page the request does not hold is fetched from an out-of-range coordinate
// and arrives as zeros. Roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 4..7 =
// softmax and output. Every wait is bounded; a wait that runs out records an error word, the CTA stops,
// drains its copies, frees its TMEM and returns.
//
// Formula as in attention_generic.cu (cpp/src/ops.cpp:206-270); the reference's prefill attention is a
// SIMT kernel with 32-key shared-memory slabs (cpp/src/cuda/cuda_backend.cu:489-575).
#include "tcgen05.cuh"

using namespace nibp;
using namespace nibt;

namespace {

constexpr int ROWS = 128;        // rows of a tile (UMMA M): TMEM lanes
constexpr int THREADS = 384;     // TMA warp, MMA warp, two idle warps; eight softmax warps (two threads per row, half of a block's keys each)
constexpr float LOG2E = 1.4426950408889634f;

__device__ int g_attn_error = 0;

// The hand-overs between the roles of this kernel are short and on the critical path of every block of keys: poll
// without sleeping for a long while (the limit still holds).
__device__ __forceinline__ bool mbar_spin(unsigned long long* bar, unsigned parity) {
#pragma unroll 1      // (unrolled, each of the kernel's thirty waits would be several copies of this loop: instruction cache)
    for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (i > (1u << 16)) __nanosleep(100);
    }
    return false;
}
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Keys per block: 128 for heads of 64; 64 for heads of 128, where two query tiles, the key and value stages and two
// tiles of probabilities of 128 keys would not fit the shared memory of an SM.
template <int HD> constexpr int keys_of() { return HD == 64 ? 128 : 64; }

template <int HD> struct Cfg {
    static constexpr int KEYS = keys_of<HD>();                // keys per block (UMMA N of S, K of P.V)
    static constexpr int SUB = HD / 64;                       // sub-tiles of 64 elements (128 bytes) along the head dim
    static constexpr int PSUB = KEYS / 64;                    // sub-tiles of 64 keys of a tile of probabilities
    static constexpr int SUBTILE = 128 * 128;                 // bytes of a [128 rows x 64 elements] sub-tile
    static constexpr int Q_BYTES = SUB * SUBTILE;             // the tile of queries
    static constexpr int KV_BYTES = KEYS * HD * 2;            // one block of keys (or values)
    static constexpr int P_BYTES = PSUB * SUBTILE;            // [128 rows x KEYS]
    static constexpr int STAGES = 2;
    static constexpr int OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = OFF_K + STAGES * KV_BYTES, OFF_P = OFF_V + STAGES * KV_BYTES;
    static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
    static constexpr int OFF_XCH = OFF_BAR + 256;             // what the two threads of a row tell each other: [3][2][128] floats
    static constexpr int SMEM = OFF_XCH + 3 * 2 * 128 * 4 + 1024;
    static constexpr int COL_S = 0, COL_O = 2 * KEYS;         // two buffers of scores, then the output
    static constexpr int TMEM_COLS = (2 * KEYS + HD) <= 256 ? 256 : 512;
};

// The running maximum of a row is replaced by a larger one only when it grew by more than this (in log2 units):
// the output accumulator in tensor memory then has to be rescaled, which costs a read and a write of the row.
// Meanwhile probabilities are at most 2^8, harmless in bfloat16 and in the 32-bit sums.
constexpr float RESCALE_ABOVE = 8.0f;

// grid: (row tiles, requests, kv heads)
template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
                            const int* __restrict__ block_table, int bt_stride, int page_size, int num_pages,
                            int heads, int kv_heads, float scale, int window, unsigned long long* trace, int trace_cap) {
    using C = Cfg<HD>;
    constexpr int KEYS = C::KEYS, STAGES = C::STAGES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + C::OFF_BAR);
    unsigned long long* q_full = bars;            // 1
    unsigned long long* k_full = bars + 1;        // [STAGES]
    unsigned long long* k_empty = bars + 3;
    unsigned long long* v_full = bars + 5;
    unsigned long long* v_empty = bars + 7;
    // One barrier per BUFFER (of scores in tensor memory, of probabilities in shared memory): a buffer's next phase
    // cannot complete before its last one was seen, which a single barrier shared by both buffers would not ensure.
    unsigned long long* s_full = bars + 9;        // [2] the scores of a block are in buffer b
    unsigned long long* p_full = bars + 11;       // [2] 256 arrivals: the probabilities of a block are in buffer b
    unsigned long long* o_done = bars + 13;       // [2] P.V of the block whose probabilities were in buffer b has been added
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 15);
    unsigned long long* pair_bar = bars + 16;     // [4] the two softmax warps of a lane quadrant meet here (one arrival each)
    __shared__ volatile int s_failed;

    pdl_launch_dependents();
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_ATTN_PREFILL, 0, 0);
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
    const int b_begin = lo_cta / KEYS, n_blk = hi_cta / KEYS - b_begin + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* bt = block_table + (size_t)req * bt_stride;

    if (threadIdx.x == 0) {
        s_failed = 0;
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 256);
            mbar_init(&o_done[i], 1);
        }
        for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 2);
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
    pdl_wait();
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_ATTN_PREFILL, 0, 1);

    if (warp == 0) {
        // ---------------- producer: lane 0 fetches Q and arms the barriers; lane i fetches page i of every block of
        // keys (its block-table entry is read one block ahead, so that the look-up of a page never stands between
        // two copies)
        if (lane == 0) {
            mbar_expect_tx(q_full, (unsigned)(rows_tile * 128 * C::SUB));
#pragma unroll
            for (int s = 0; s < C::SUB; ++s)
                tma_load_3d(smem + C::OFF_Q + s * C::SUBTILE, &map_q, q_full, s * 64, kvh * n_rep, row_begin + tok0);
        }
        const int pages_per_block = KEYS / page_size;
        const int oob = num_pages * kv_heads;             // a coordinate outside the pool: the box arrives as zeros
        // This lane's block-table entry of block j, or -1 where it has no page to fetch there. The entry of block j+1 is
        // asked for while block j is being sent for and is looked at only a block later: the look-up's latency (more
        // than half a microsecond) must not stand between two blocks' copies.
        auto entry_of = [&](int j) -> int {
            const int key = (b_begin + j) * KEYS + lane * page_size;
            if (lane >= pages_per_block || key > hi_cta || key + page_size <= lo_cta) return -1;
            return __ldg(bt + key / page_size);
        };
        int entry_next = entry_of(0);
        int issued = 0;
        for (int j = 0; j < n_blk; ++j) {
            const int st = j % STAGES;
            const int entry = entry_next;
            if (j + 1 < n_blk) entry_next = entry_of(j + 1);
            const int z = (entry >= 0 && entry < num_pages) ? entry * kv_heads + kvh : oob;      // third coordinate of the page
            // keys first (the scores of this block are wanted a whole block ahead), values when their stage is free
            const unsigned par = ((j / STAGES) & 1) ^ 1;
            int ok = 1;
#pragma unroll
            for (int kv = 0; kv < 2; ++kv) {
                unsigned long long* empty = kv ? &v_empty[st] : &k_empty[st];
                unsigned long long* full = kv ? &v_full[st] : &k_full[st];
                if (lane == 0) {
                    ok = !s_failed && mbar_wait(empty, par);
                    if (ok) mbar_expect_tx(full, C::KV_BYTES);
                    else if (!s_failed) { atomicCAS(&g_attn_error, 0, (1 << 16) | (int)(blockIdx.x & 0xffff)); s_failed = 1; }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane < pages_per_block) {
#pragma unroll
                    for (int s = 0; s < C::SUB; ++s)
                        tma_load_3d(smem + (kv ? C::OFF_V : C::OFF_K) + st * C::KV_BYTES + s * (KEYS * 128) + lane * page_size * 128,
                                    kv ? &map_v : &map_k, full, s * 64, 0, z);
                }
            }
            if (!ok) break;
            issued = j + 1;
        }
        if (s_failed && lane == 0) {
            // copies already issued still target this CTA's shared memory: wait for them, bounded
            mbar_wait(q_full, 0);
            for (int j = max(0, issued - STAGES); j < issued; ++j) {
                mbar_wait(&k_full[j % STAGES], (j / STAGES) & 1);
                mbar_wait(&v_full[j % STAGES], (j / STAGES) & 1);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer: S(0); then for every block j: S(j+1) into the other buffer of scores at once (so
        // the softmax of block j+1 never waits for the tensor core), and O += P(j) . V(j) when P(j) is there.
        constexpr unsigned idesc_s = instr_desc(ROWS, KEYS, false);
        constexpr unsigned idesc_o = instr_desc(ROWS, HD, true);
        const unsigned q_addr = smem_u32(smem + C::OFF_Q);
        auto issue_qk = [&](int j) {
            const unsigned k_addr = smem_u32(smem + C::OFF_K + (j % STAGES) * C::KV_BYTES);
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const unsigned long long adv = (unsigned long long)(((kk & 3) * 32) >> 4);
                tc_mma(tmem_base + C::COL_S + (j & 1) * KEYS, desc_kmajor(q_addr + (kk >> 2) * C::SUBTILE) + adv,
                       desc_kmajor(k_addr + (kk >> 2) * (KEYS * 128)) + adv, idesc_s, kk > 0);
            }
            tc_commit(&s_full[j & 1]);
            tc_commit(&k_empty[j % STAGES]);
        };
        auto issue_pv = [&](int j) {
            const unsigned p_addr = smem_u32(smem + C::OFF_P + (j & 1) * C::P_BYTES);
            const unsigned v_addr = smem_u32(smem + C::OFF_V + (j % STAGES) * C::KV_BYTES);
#pragma unroll
            for (int kk = 0; kk < KEYS / 16; ++kk) {
                // P: sub-tile kk/4 (64 keys each), 32 bytes per step inside it; V: 16 keys = 2048 bytes further down,
                // the second 64 elements of the head dim KEYS*128 bytes further on
                const unsigned long long a = desc_kmajor(p_addr + (kk >> 2) * C::SUBTILE) + (unsigned long long)(((kk & 3) * 32) >> 4);
                const unsigned long long b = desc_mnmajor(v_addr + kk * 16 * 128, KEYS * 128);
                tc_mma(tmem_base + C::COL_O, a, b, idesc_o, j > 0 || kk > 0);
            }
            tc_commit(&o_done[j & 1]);
            tc_commit(&v_empty[j % STAGES]);
        };
        bool ok = mbar_spin(q_full, 0) && mbar_spin(&k_full[0], 0);
        if (!ok) { atomicCAS(&g_attn_error, 0, (2 << 16) | (int)(blockIdx.x & 0xffff)); s_failed = 1; }
        if (ok) { tc_fence_after(); issue_qk(0); }
        for (int j = 0; j < n_blk && ok; ++j) {
            if (j + 1 < n_blk) {
                // the other buffer of scores is free: the probabilities of block j-1 were complete before its P.V
                ok = mbar_spin(&k_full[(j + 1) % STAGES], ((j + 1) / STAGES) & 1);
                if (!ok) break;
                tc_fence_after();
                issue_qk(j + 1);
            }
            ok = mbar_spin(&p_full[j & 1], (j >> 1) & 1) && mbar_spin(&v_full[j % STAGES], (j / STAGES) & 1);
            if (!ok) break;
            tc_fence_after();
            issue_pv(j);
        }
        if (!ok && !s_failed) { atomicCAS(&g_attn_error, 0, (3 << 16) | (int)(blockIdx.x & 0xffff)); s_failed = 1; }
    } else if (warp >= 4) {
        // ---------------- softmax and output: two threads own a row, in warps that may read the same TMEM lanes
        // (32*(warp%4)...): each takes half of a block's keys and half of the output row's columns. They tell each other
        // the maximum of their halves (and at the end the sum) through shared memory, meeting at a barrier of their two
        // warps. Rows past the tile's last (the tile holds a whole number of tokens) see what the last row sees; nothing
        // of them is stored.
        constexpr int HK = KEYS / 2;                      // keys of a block per thread
        const int quad = warp & 3, half = (warp - 4) >> 2, row = quad * 32 + lane;
        const unsigned lane_addr = tmem_base + ((unsigned)(quad * 32) << 16);
        const unsigned o_addr = lane_addr + C::COL_O + half * (HD / 2);
        float* xch = reinterpret_cast<float*>(smem + C::OFF_XCH);        // [3][2][128]
        // the meeting of the two warps of a quadrant: an mbarrier, so that the wait is bounded like every other (a warp
        // that has given up never arrives, and its partner then gives up too instead of waiting for ever)
        unsigned pair_phase = 0;
        auto pair_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(&pair_bar[quad]);
            const bool met = mbar_spin(&pair_bar[quad], pair_phase & 1);
            ++pair_phase;
            return __all_sync(0xffffffffu, met);
        };
        const bool live = row < n_tok * n_rep;
        const int ti = min(row / n_rep, n_tok - 1), head = kvh * n_rep + (row % n_rep);
        const int hi = pos0 + ti;
        const int lo = window > 0 ? max(0, hi - window + 1) : 0;
        const float scale2 = scale * LOG2E;
        float m_cur = -INFINITY, l_run = 0.f;       // the maximum that the exponents refer to, and this thread's part of the sum
        bool ok = true;
        for (int j = 0; j < n_blk && ok; ++j) {
            const int b = j & 1;
            ok = !s_failed && mbar_spin(&s_full[b], (j >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int key0 = (b_begin + j) * KEYS;
            // the same branch for the whole warp: a warp that took both would do the work twice
            const bool all_visible = __all_sync(0xffffffffu, key0 >= lo && key0 + KEYS - 1 <= hi);
            // this thread's scores of the block: all loads are issued, then waited for once (a load from tensor memory
            // takes hundreds of cycles). Four maxima side by side, so that no instruction waits for the one before it.
            const unsigned s_addr = lane_addr + C::COL_S + b * KEYS + half * HK;
            unsigned raw[HK / 32][32];
#pragma unroll
            for (int c = 0; c < HK / 32; ++c) tmem_ld32_async(s_addr + c * 32, raw[c]);
            tmem_wait_ld();
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < HK / 32; ++c) {
                if (all_visible) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(raw[c][i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = key0 + half * HK + c * 32 + i;
                        if (!(key >= lo && key <= hi)) raw[c][i] = 0xff800000u;      // -inf: its probability will be 0
                        mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(raw[c][i]));
                    }
                }
            }
            // the row's maximum over both halves (the slot of block j is written again at block j + 2, after the barrier
            // of block j + 1, which the other thread reaches only when it has read this one)
            float mine = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            xch[(b * 2 + half) * 128 + row] = mine;
            ok = pair_sync();
            if (!ok) break;
            const float mx = fmaxf(mine, xch[(b * 2 + (half ^ 1)) * 128 + row]) * scale2;      // scale2 > 0
            float corr = 1.f;
            bool grow = false;
            if (m_cur == -INFINITY) {
                m_cur = mx;                                 // nothing summed yet: sum and output row are zero
            } else if (mx > m_cur + RESCALE_ABOVE) {
                corr = ex2(m_cur - mx);
                l_run *= corr;
                m_cur = mx;
                grow = true;
            }
            const float m_use = (m_cur == -INFINITY) ? 0.f : m_cur;
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                // rare: the output row is rescaled in tensor memory (each thread its half of the columns), once P.V of
                // the block before has been added. Both threads of a row decide alike: they see the same maxima.
                ok = mbar_spin(&o_done[(j - 1) & 1], ((j - 1) >> 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 64; ++c) {
                    unsigned ov[32];
                    tmem_ld32_async(o_addr + c * 32, ov);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    tmem_st32(o_addr + c * 32, ov);
                }
                tmem_wait_st();
            }
            if (j >= 2) {
                // this buffer of probabilities was read by P.V of block j-2
                ok = mbar_spin(&o_done[b], ((j - 2) >> 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            // the probabilities into shared memory, their sum (four partial sums)
            unsigned char* p_row = smem + C::OFF_P + b * C::P_BYTES + (row >> 3) * 1024 + (row & 7) * 128;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < HK / 32; ++c) {
                unsigned pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = ex2(fmaf(__uint_as_float(raw[c][i]), scale2, -m_use));         // ex2(-inf) = 0
                    const float p1 = ex2(fmaf(__uint_as_float(raw[c][i + 1]), scale2, -m_use));
                    sum4[(i >> 1) & 3] += p0 + p1;
                    pk[i >> 1] = pack2(p0, p1);
                }
                const int cg = half * (HK / 32) + c;                        // the chunk of 32 keys within the block
                unsigned char* sub = p_row + (cg >> 1) * C::SUBTILE;       // 64 keys per sub-tile
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = ((cg & 1) << 2) + q4;                 // 16-byte chunk within the 128-byte row
                    *reinterpret_cast<uint4*>(sub + ((chunk ^ (row & 7)) << 4)) =
                        make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
                }
            }
            l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // P is read by the tensor core through the async proxy
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            tc_fence_before();
            mbar_arrive(&p_full[b]);
        }
        if (ok) {
            ok = mbar_spin(&o_done[(n_blk - 1) & 1], ((n_blk - 1) >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            // the row's sum: both parts, added in the same order by both threads
            xch[(4 + half) * 128 + row] = l_run;
            ok = pair_sync();
        }
        if (!ok) {
            if (lane == 0 && !s_failed) { atomicCAS(&g_attn_error, 0, (4 << 16) | (int)(blockIdx.x & 0xffff)); s_failed = 1; }
        } else {
            tc_fence_after();
            const float l_all = xch[4 * 128 + row] + xch[5 * 128 + row];
            const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
            __nv_bfloat16* orow = out + ((size_t)(row_begin + tok0 + ti) * heads + head) * HD + half * (HD / 2);
#pragma unroll
            for (int c = 0; c < HD / 64; ++c) {
                unsigned ov[32];
                tmem_ld32_async(o_addr + c * 32, ov);
                tmem_wait_ld();
                if (live) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 w;
                        w.x = pack2(__uint_as_float(ov[d]) * inv, __uint_as_float(ov[d + 1]) * inv);
                        w.y = pack2(__uint_as_float(ov[d + 2]) * inv, __uint_as_float(ov[d + 3]) * inv);
                        w.z = pack2(__uint_as_float(ov[d + 4]) * inv, __uint_as_float(ov[d + 5]) * inv);
                        w.w = pack2(__uint_as_float(ov[d + 6]) * inv, __uint_as_float(ov[d + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + d) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_ATTN_PREFILL, 0, 2);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------- host side
// 3-D map over bfloat16 data: dims (d0 innermost), strides in elements for d1 and d2, box (64, b1, b2).
int make_map3(CUtensorMap* map, const void* ptr, long long d0, long long d1, long long d2, long long s1, long long s2,
              int b1, int b2) {
    NibEncodeTiledFn enc = nib_tensor_map_encoder();
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
                        kv_heads, scale, window, nib_trace_buffer(), nib_trace_capacity()));
    return 0;
}

}  // namespace

// 1 if the tcgen05 kernel takes this shape: head size 64 or 128, at most 128 query heads per kv head,
// pages of 8..128 tokens that divide 128, 16-byte aligned rows.
NIB_API int nib_attention_prefill_tc_supported(int heads, int kv_heads, int head_dim, int page_size, int q_stride) {
    if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > ROWS) return 0;
    if (head_dim != 64 && head_dim != 128) return 0;
    const int keys = head_dim == 64 ? keys_of<64>() : keys_of<128>();
    if (page_size < 8 || page_size > keys || keys % page_size) return 0;
    if (q_stride % 8) return 0;
    return nib_tensor_map_encoder() != nullptr;
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
