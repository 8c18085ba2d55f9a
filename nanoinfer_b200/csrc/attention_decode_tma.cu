// Decode attention (one new token per request) with the key/value pages brought in by TMA.
//
// A page of one kv head is a dense block of page_size x head_dim bfloat16 in the pool, so one
// cp.async.bulk.tensor instruction of one lane fetches it whole, with the 128-byte swizzle that makes
// the ldmatrix reads conflict free; nobody computes addresses chunk by chunk. A page that the request
// does not hold (freed by a window, beyond the context, a padding row) is fetched at a coordinate
// outside the pool and arrives as zeros. Slots of a held page beyond the context hold finite values
// (the pool starts zeroed and only finite values are written), and their scores are masked.
//
// grid (splits, tokens, kv heads). A CTA walks over its tiles of 64 or 128 keys (aligned to absolute
// multiples of the tile) with a few tiles in flight: a producer warp issues the copies and runs ahead, a
// full and an empty mbarrier per stage hand the tiles back and forth, and no barrier of the whole CTA
// stands in the loop. The consumer warps take 16 keys of every tile each, keep their own running
// (max, sum, output) and merge at the end. The 16 keys are the ROWS of the tensor-core tile and the
// query heads of the kv group (at most 16, usually fewer than 8) its columns: S^T = K Q^T, the
// probabilities are transposed inside the warp (movmatrix) and O^T = V^T P^T. With the heads as the rows
// a group of 7 heads would fill 7 of 16 rows and the instruction count, which bounds a decode step's
// warps, would double.
//
// The CTAs that split one (token, kv head) form a thread-block cluster of up to eight. Each leaves its
// partial (max, sum, output) in its own shared memory; after a cluster barrier every CTA of the cluster
// merges a slice of the output columns from all its peers' shared memory (distributed shared memory, in
// rank order) and stores the finished bfloat16 values: no scratch in global memory, no second kernel, no
// extra round trip in a decode layer's chain. Only a context so long that eight CTAs per (token, kv head)
// are too few is cut further: then each cluster writes one partial triple to scratch and
// nib_attention_combine merges the clusters' triples in order.
//
// Every wait has an iteration limit; a wait that runs out sets an error word, the CTA stops, waits
// (bounded) for its copies in flight and returns.
//
// Formula as in attention_generic.cu (cpp/src/ops.cpp:206-270). The reference's decode attention is a
// SIMT split-KV kernel with a combine pass (cpp/src/cuda/cuda_backend.cu:578-640, :331-352).
#include "attention_common.cuh"
#include "pipeline.cuh"

using namespace nibp;

extern "C" int nib_attention_combine(const float* part_o, const float* part_ml, void* out, int rows, int splits,
                                     int head_dim, cudaStream_t stream);

namespace {

// Keys per tile: 128 for heads of 64 (a tile of 64 keys is only 16 KB there, and the fixed work per tile,
// barrier waits and the softmax's shuffles, bounded the kernel at large batches), 64 for heads of 128.
template <int HD> constexpr int keys_of() { return HD == 64 ? 128 : 64; }
// Consumer warps: 16 keys of every tile each, so eight for tiles of 128 keys and four for tiles of 64; one more
// warp fetches. A warp's instructions depend on one another (tensor-core results, shuffles, exponentials), and a
// warp alone on its scheduler waits out every one of those latencies: two warps per scheduler measured faster than
// one with twice the keys.
template <int HD> constexpr int warps_of() { return keys_of<HD>() / 16; }

int g_dec_stages = 3;             // tiles in flight per CTA (2..4): 32 KB each
__device__ int g_dec_error = 0;   // 0, or (code << 16 | blockIdx.x) of the first wait that ran out

template <int HD> struct Cfg {
    static constexpr int KEYS = keys_of<HD>();
    static constexpr int WARPS = warps_of<HD>();
    static constexpr int THREADS = (WARPS + 1) * 32;
    static constexpr int WKEYS = 16;                          // keys of a tile per consumer warp
    static constexpr int SUB = HD / 64;                       // 64-element column blocks of a head
    static constexpr int SUBTILE = KEYS * 128;                // KEYS rows of 128 bytes (64 elements of a head), swizzled
    static constexpr int TILE = SUB * SUBTILE;                // K (or V) of one tile
    static constexpr int STAGE = 2 * TILE;
    static constexpr int MAX_STAGES = 4;
    static constexpr int MERGE = WARPS * 16 * (HD + 4 + 2) * 4 + WARPS * 16 * 4 + 16 * HD * 4 + 16 * 2 * 4;
    static constexpr int data_bytes(int stages) { return stages * STAGE > MERGE ? stages * STAGE : MERGE; }
    static constexpr int smem_bytes(int stages) { return data_bytes(stages) + 1024 /* alignment */ + 64 /* barriers */; }
};

template <int HD, int NH>
__global__ void __launch_bounds__(Cfg<HD>::THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __nv_bfloat16* __restrict__ qkv, int q_stride, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ ctx_lens, const int* __restrict__ block_table, int bt_stride,
                            int page_size, int page_shift, int num_pages, int heads, int kv_heads, int n_rep, float scale,
                            int window, int splits, int csize, int stages, int data_bytes, int own_kv, float* __restrict__ part_o, float* __restrict__ part_ml,
                            unsigned long long* trace, int trace_cap) {
    using C = Cfg<HD>;
    constexpr int KEYS = C::KEYS, SUBTILE = C::SUBTILE, WKEYS = C::WKEYS, MT = WKEYS / 16, WARPS = C::WARPS, THREADS = C::THREADS;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(smem + data_bytes);
    unsigned long long* empty = full + stages;
    __shared__ volatile int s_failed;

    pdl_launch_dependents();
    const int split = blockIdx.x, token = blockIdx.y, kvh = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    if (tid == 0) nib_trace_mark(trace, trace_cap, NIB_TK_ATTN_DECODE, 0, 0);
    const int p = ctx_lens[token] - 1;                     // the token's own position; -1: a padding row
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int* bt = block_table + (size_t)token * bt_stride;

    // key tiles of this split
    const int t_first = lo / KEYS, t_last = p >= 0 ? p / KEYS : -1;
    const int n_tiles = t_last - t_first + 1;
    const int per = (n_tiles + splits - 1) / splits;
    const int t_begin = t_first + split * per;
    const int t_end = min(t_last, t_begin + per - 1);
    const int n_mine = max(0, t_end - t_begin + 1);

    if (tid == 0) {
        s_failed = 0;
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], WARPS); }
        mbar_fence_init();
    }
    __syncthreads();

    // O^T of this warp's keys: [16 dims of a head][8 query heads of the group] tiles; the running maximum of the
    // thread's two heads of every tile (the same in the eight lanes that share them) and ITS OWN part of their sums
    float o[HD / 16][NH][4];
    float m_run[NH][2], l_part[NH][2];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) { m_run[nh][0] = m_run[nh][1] = -INFINITY; l_part[nh][0] = l_part[nh][1] = 0.f; }
    if (warp == WARPS) {
        // ---------------- producer warp: lane i fetches page i of every tile (K and V), lane 0 arms the
        // stage's barrier. The block-table entry of the next tile is read while this one waits for its
        // stage. Keys and values of earlier positions were written by earlier steps, so their tiles are
        // fetched at once, before the step's earlier kernels have finished. The tile that holds p holds this
        // step's own key and value, written by the kernel before this one: with own_kv the consumers take
        // them from the activation buffer instead (below) and no fetch waits; without, that tile's does.
        const int pages_per_tile = KEYS >> page_shift;
        const int oob = num_pages * kv_heads;
        auto plane_of = [&](int j) -> int {
            const int key = (t_begin + j) * KEYS + (lane << page_shift);
            if (lane >= pages_per_tile || j >= n_mine || key > p || key + page_size <= lo) return oob;
            const int page = __ldg(bt + (key >> page_shift));
            return (page >= 0 && page < num_pages) ? page * kv_heads + kvh : oob;
        };
        int z_next = plane_of(0);
        bool waited = false;
        int issued = 0;
        for (int j = 0; j < n_mine; ++j) {
            const int st = j % stages;
            const int z = z_next;
            z_next = plane_of(j + 1);
            if (!own_kv && t_begin + j == t_last && !waited) { pdl_wait(); waited = true; }
            int ok = 1;
            if (lane == 0) {
                if (j >= stages) ok = !s_failed && mbar_wait(&empty[st], ((j / stages) - 1) & 1);
                if (ok) mbar_expect_tx(&full[st], C::STAGE);
                else if (!s_failed) { atomicCAS(&g_dec_error, 0, (2 << 16) | (int)(blockIdx.x & 0xffff)); s_failed = 1; }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < pages_per_tile) {
                unsigned char* kd = smem + st * C::STAGE + ((lane << page_shift) * 128);
#pragma unroll
                for (int s = 0; s < C::SUB; ++s) {
                    tma_load_3d(kd + s * SUBTILE, &map_k, &full[st], s * 64, 0, z);
                    tma_load_3d(kd + C::TILE + s * SUBTILE, &map_v, &full[st], s * 64, 0, z);
                }
            }
            issued = j + 1;
        }
        if (s_failed && lane == 0) {
            // copies already issued still target this CTA's shared memory: wait for them, bounded
            for (int j = max(0, issued - stages); j < issued; ++j) mbar_wait(&full[j % stages], (j / stages) & 1);
        }
    } else {
        // ---------------- the consumer warps: 16 keys of every tile each
        const int wg = warp;
        pdl_wait();
        if (tid == 0) nib_trace_mark(trace, trace_cap, NIB_TK_ATTN_DECODE, 0, 1);
        // The keys are the 16-row operand of the tensor-core instruction and the (at most 8) query heads of the group
        // its 8 columns: S^T = K Q^T and O^T = V^T P^T. With the heads as the rows, 16 rows would hold 7 heads of a
        // typical group and the instruction count would double; the warps of a decode step are bound by that count.
        // Q^T as the column operand: thread (g, t) holds head g, dims 2t, 2t+1 and 2t+8, 2t+9 of every block of 16.
        unsigned qb[HD / 16][NH][2];
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) {
            const int head = nh * 8 + g;
            const __nv_bfloat16* qp = qkv + (size_t)token * q_stride + (size_t)(kvh * n_rep + head) * HD;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                qb[kk][nh][0] = head < n_rep ? *reinterpret_cast<const unsigned*>(qp + kk * 16 + 2 * t) : 0u;
                qb[kk][nh][1] = head < n_rep ? *reinterpret_cast<const unsigned*>(qp + kk * 16 + 8 + 2 * t) : 0u;
            }
        }
#pragma unroll
        for (int d = 0; d < HD / 16; ++d)
#pragma unroll
            for (int nh = 0; nh < NH; ++nh) o[d][nh][0] = o[d][nh][1] = o[d][nh][2] = o[d][nh][3] = 0.f;
        const float scale2 = scale * LOG2E;

        // ldmatrix addresses inside a swizzled tile: row r (128 bytes), 16-byte chunk c at ((c ^ (r & 7)) << 4).
        // K as the row operand: matrices (keys 0-7, dims 0-7), (keys 8-15, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15,
        // dims 8-15). V^T as the row operand, read transposed: (keys 0-7, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, ...).
        const int mat = lane >> 3, rr = lane & 7;
        const unsigned k_row = (unsigned)(wg * WKEYS + (mat & 1) * 8 + rr) * 128u;
        const unsigned k_half = mat >> 1;
        const unsigned v_row = (unsigned)(wg * WKEYS + (mat >> 1) * 8 + rr) * 128u;
        const unsigned v_half = mat & 1;

        for (int j = 0; j < n_mine; ++j) {
            const int st = j % stages;
            bool ok = !s_failed && mbar_wait(&full[st], (j / stages) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0 && !s_failed) { atomicCAS(&g_dec_error, 0, (1 << 16) | (int)(blockIdx.x & 0xffff)); s_failed = 1; }
                break;
            }
            const unsigned kt = smem_u32(smem + st * C::STAGE), vt = kt + C::TILE;
            if (own_kv && t_begin + j == t_last && p >= 0 && (p & (KEYS - 1)) / WKEYS == wg) {
                // this step's own key (rotated) and value, from the token's row of the activation buffer into this
                // warp's rows of the tile: the copy of the page may have been taken before they were written there
                const __nv_bfloat16* k_new = qkv + (size_t)token * q_stride + (size_t)(heads + kvh) * HD;
                const __nv_bfloat16* v_new = qkv + (size_t)token * q_stride + (size_t)(heads + kv_heads + kvh) * HD;
                const int r = p & (KEYS - 1);
                unsigned char* k_tile = smem + st * C::STAGE;
                for (int d = 2 * lane; d < HD; d += 64) {
                    // element d of row r in a swizzled tile: column block d/64, 16-byte chunk (d%64)/8 at ((chunk ^ (r&7)) << 4)
                    const unsigned byte = (unsigned)(d >> 6) * SUBTILE + (unsigned)r * 128u +
                                          (((unsigned)((d & 63) >> 3) ^ (unsigned)(r & 7)) << 4) + (unsigned)(d & 7) * 2u;
                    *reinterpret_cast<unsigned*>(k_tile + byte) = *reinterpret_cast<const unsigned*>(k_new + d);
                    *reinterpret_cast<unsigned*>(k_tile + C::TILE + byte) = *reinterpret_cast<const unsigned*>(v_new + d);
                }
                __syncwarp();
            }
            float s[MT][NH][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nh = 0; nh < NH; ++nh) s[mt][nh][0] = s[mt][nh][1] = s[mt][nh][2] = s[mt][nh][3] = 0.f;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    unsigned a[4];
                    const unsigned chunk = (unsigned)((kk & 3) * 2) + k_half;
                    ldmatrix_x4_addr(a, kt + (kk >> 2) * SUBTILE + k_row + mt * 16 * 128 + ((chunk ^ (unsigned)rr) << 4));
#pragma unroll
                    for (int nh = 0; nh < NH; ++nh) mma_bf16(s[mt][nh], a, qb[kk][nh][0], qb[kk][nh][1]);
                }
            }
            // element e of a tile: key g + 8*(e/2) of the 16, head 2t + (e&1) of the 8. Scores in log2 units; a key outside
            // lo..p counts as -inf. The maximum of a head goes over the thread's keys and then over the eight lanes that
            // hold the head's other keys.
            const int key0 = (t_begin + j) * KEYS + wg * WKEYS + g;
            float corr[NH][2], m_use[NH][2];
#pragma unroll
            for (int nh = 0; nh < NH; ++nh) {
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + mt * 16 + 8 * (e >> 1);
                        const float v = (key >= lo && key <= p) ? s[mt][nh][e] * scale2 : -INFINITY;
                        s[mt][nh][e] = v;
                        mx[e & 1] = fmaxf(mx[e & 1], v);
                    }
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    mx[q] = fmaxf(mx[q], __shfl_xor_sync(0xffffffffu, mx[q], 4));
                    mx[q] = fmaxf(mx[q], __shfl_xor_sync(0xffffffffu, mx[q], 8));
                    mx[q] = fmaxf(mx[q], __shfl_xor_sync(0xffffffffu, mx[q], 16));
                    const float m_new = fmaxf(m_run[nh][q], mx[q]);
                    m_use[nh][q] = (m_new == -INFINITY) ? 0.f : m_new;           // nothing visible yet: exp2(-inf - 0) = 0
                    corr[nh][q] = (m_run[nh][q] == -INFINITY) ? 0.f : exp2f(m_run[nh][q] - m_use[nh][q]);
                    m_run[nh][q] = m_new;
                    l_part[nh][q] *= corr[nh][q];
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float pv = exp2f(s[mt][nh][e] - m_use[nh][e & 1]);
                        s[mt][nh][e] = pv;
                        l_part[nh][e & 1] += pv;
                    }
#pragma unroll
                for (int d = 0; d < HD / 16; ++d) {
                    o[d][nh][0] *= corr[nh][0]; o[d][nh][1] *= corr[nh][1];
                    o[d][nh][2] *= corr[nh][0]; o[d][nh][3] *= corr[nh][1];
                }
            }
            // O^T += V^T P^T: P^T (keys x heads, what the first product left in the accumulators) becomes the column
            // operand by transposing its two 8 x 8 blocks inside the warp
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                unsigned pb[NH][2];
#pragma unroll
                for (int nh = 0; nh < NH; ++nh) {
                    pb[nh][0] = movmatrix_trans(pack_bf16(s[mt][nh][0], s[mt][nh][1]));
                    pb[nh][1] = movmatrix_trans(pack_bf16(s[mt][nh][2], s[mt][nh][3]));
                }
#pragma unroll
                for (int d = 0; d < HD / 16; ++d) {
                    unsigned a[4];
                    const unsigned chunk = (unsigned)((d & 3) * 2) + v_half;
                    ldmatrix_x4_trans_addr(a, vt + (d >> 2) * SUBTILE + v_row + mt * 16 * 128 + ((chunk ^ (unsigned)rr) << 4));
#pragma unroll
                    for (int nh = 0; nh < NH; ++nh) mma_bf16(o[d][nh], a, pb[nh][0], pb[nh][1]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);            // this warp has read the stage
        }
    }
    __syncthreads();        // every tile is consumed (or the CTA failed): no copy is in flight any more

    // ---- merge the consumer warps through shared memory. A CTA that failed, and the rows of a padding token,
    // contribute (max -inf, sum 0); every thread goes on to the cluster's barriers.
    constexpr int MS = HD + 4;                                    // padded row: conflict-free float2 stores
    float* sm_o = reinterpret_cast<float*>(smem);                 // [WARPS][16][MS]
    float* sm_ml = sm_o + WARPS * 16 * MS;                        // [WARPS][16][2]
    float* cta_o = sm_ml + WARPS * 16 * 2;                            // [16][HD]  this CTA's output, relative to its own maximum
    float* cta_ml = cta_o + 16 * HD;                              // [16][2]   its (max, sum)
    const bool failed = s_failed != 0;
    if (warp < WARPS) {
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int head = nh * 8 + 2 * t + q;
                float l = l_part[nh][q];            // the sum over the keys of the lanes that share the head
                l += __shfl_xor_sync(0xffffffffu, l, 4);
                l += __shfl_xor_sync(0xffffffffu, l, 8);
                l += __shfl_xor_sync(0xffffffffu, l, 16);
#pragma unroll
                for (int d = 0; d < HD / 16; ++d) {
                    sm_o[(warp * 16 + head) * MS + d * 16 + g] = o[d][nh][q];
                    sm_o[(warp * 16 + head) * MS + d * 16 + g + 8] = o[d][nh][2 + q];
                }
                if (g == 0) {
                    sm_ml[(warp * 16 + head) * 2] = failed ? -INFINITY : m_run[nh][q];
                    sm_ml[(warp * 16 + head) * 2 + 1] = failed ? 0.f : l;
                }
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < n_rep * HD; i += THREADS) {
        const int row = i / HD, d = i - row * HD;
        float mw[WARPS], m_row = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) { mw[w] = sm_ml[(w * 16 + row) * 2]; m_row = fmaxf(m_row, mw[w]); }
        float acc = 0.f, l_row = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - m_row);
            acc += sm_o[(w * 16 + row) * MS + d] * f;
            l_row += sm_ml[(w * 16 + row) * 2 + 1] * f;
        }
        cta_o[row * HD + d] = acc;
        if (d == 0) {
            cta_ml[row * 2] = m_row;
            cta_ml[row * 2 + 1] = l_row;
        }
    }
    if (csize > 1) cluster_sync(); else __syncthreads();

    // ---- merge the CTAs of the cluster: this CTA finishes its slice of the group's n_rep x HD outputs from
    // every peer's (max, sum, output), in rank order
    const int rank = csize > 1 ? (int)cluster_rank() : 0;
    const int outer = splits / csize, oidx = split / csize;
    const int total = n_rep * HD;
    const int slice = (total + csize - 1) / csize;
    const int i_end = min(total, (rank + 1) * slice);
    for (int i = rank * slice + tid; i < i_end; i += THREADS) {
        const int row = i / HD, d = i - row * HD;
        float m_all = -INFINITY, l_all = 0.f, acc = 0.f;
        if (csize > 1) {
            // every peer's (max, sum, output) of this element is asked for before the first is used: one round trip
            float mr[8], lr[8], orr[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                mr[r] = -INFINITY; lr[r] = 0.f; orr[r] = 0.f;
                if (r < csize) {
                    mr[r] = ld_peer_f32(peer_smem(&cta_ml[row * 2], r));
                    lr[r] = ld_peer_f32(peer_smem(&cta_ml[row * 2 + 1], r));
                    orr[r] = ld_peer_f32(peer_smem(&cta_o[row * HD + d], r));
                }
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) m_all = fmaxf(m_all, mr[r]);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float f = (mr[r] == -INFINITY) ? 0.f : exp2f(mr[r] - m_all);
                l_all += lr[r] * f;
                acc += orr[r] * f;
            }
        } else {
            m_all = cta_ml[row * 2];
            l_all = cta_ml[row * 2 + 1];
            acc = cta_o[row * HD + d];
        }
        const size_t th = (size_t)token * heads + kvh * n_rep + row;
        if (outer == 1) {
            out[th * HD + d] = __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
        } else {
            part_o[(th * outer + oidx) * HD + d] = acc;
            if (d == 0) {
                part_ml[(th * outer + oidx) * 2] = m_all;
                part_ml[(th * outer + oidx) * 2 + 1] = l_all;
            }
        }
    }
    if (tid == 0) nib_trace_mark(trace, trace_cap, NIB_TK_ATTN_DECODE, 0, 2);
    if (csize > 1) cluster_sync();      // nobody leaves while a peer may still read its shared memory
}

// ---------------------------------------------------------------------------------- host side

// Map over the pool: (head dim, slot in page, page * kv_heads + kv head); a box is 64 elements of one page of one kv head.
int make_pool_map(CUtensorMap* map, const void* ptr, int head_dim, int page_size, long long planes) {
    NibEncodeTiledFn enc = nib_tensor_map_encoder();
    NIB_REQUIRE(enc != nullptr, "attention decode (TMA): cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)page_size * head_dim * 2};
    cuuint32_t box[3] = {64u, (cuuint32_t)page_size, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NIB_REQUIRE(r == CUDA_SUCCESS, "attention decode (TMA): cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int HD, int NH>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const void* qkv, int q_stride, void* out, const int* ctx_lens,
           const int* block_table, int bt_stride, int page_size, int num_pages, int n_tokens, int heads, int kv_heads,
           float scale, int window, int splits, int csize, int own_kv, float* part_o, float* part_ml, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(attention_decode_tma_kernel<HD, NH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg<HD>::smem_bytes(Cfg<HD>::MAX_STAGES)));
        configured = true;
    }
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, n_tokens, kv_heads);
    cfg.blockDim = dim3(Cfg<HD>::THREADS);
    const int stages = g_dec_stages;
    cfg.dynamicSmemBytes = (size_t)Cfg<HD>::smem_bytes(stages);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (csize > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = csize;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    if (nib_pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    NIB_CUDA(cudaLaunchKernelEx(&cfg, attention_decode_tma_kernel<HD, NH>, mk, mv, (const __nv_bfloat16*)qkv, q_stride,
                                (__nv_bfloat16*)out, ctx_lens, block_table, bt_stride, page_size, shift, num_pages, heads,
                                kv_heads, heads / kv_heads, scale, window, splits, csize, stages, Cfg<HD>::data_bytes(stages), own_kv, part_o, part_ml,
                                nib_trace_buffer(), nib_trace_capacity()));
    const int outer = splits / csize;
    if (outer > 1) return nib_attention_combine(part_o, part_ml, out, n_tokens * heads, outer, HD, stream);
    return 0;
}

}  // namespace

// 1 if the TMA decode kernel takes this shape: head size 64 or 128, at most 16 query heads per kv head,
// pages of 8, 16, 32 or 64 tokens.
NIB_API int nib_attention_decode_tma_supported(int heads, int kv_heads, int head_dim, int page_size) {
    if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > 16) return 0;
    if (head_dim != 64 && head_dim != 128) return 0;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return 0;
    return nib_tensor_map_encoder() != nullptr;
}

// Tiles in flight per CTA (2..4, 32 KB of shared memory each); for measurements.
NIB_API void nib_attention_decode_tma_stages(int stages) { g_dec_stages = stages < 2 ? 2 : (stages > 4 ? 4 : stages); }

// The error word of the kernel's bounded waits (0 = none); synchronises with the device and clears it.
NIB_API int nib_attention_decode_tma_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_dec_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_dec_error, &zero, sizeof(int));
    return v;
}

// Attention of n_tokens single decoded tokens (token i is request i) over their cached keys; ``qkv`` holds the
// rotated queries, and the token's own key and value are in its page already; with ``own_kv`` the row also holds the
// token's rotated key and its value behind the queries ([q heads | k heads | v heads]) and they are taken from there, so
// that no page has to be read after the kernel that wrote them. ``splits`` CTAs share the keys
// of a (token, kv head): 1, 2, 4 or 8 (one cluster merges them in shared memory), or a multiple of 8 (clusters
// of eight, whose partial results go to ``part_o`` [tokens*heads*splits/8*head_dim] and ``part_ml``
// [tokens*heads*splits/8*2] floats and are merged by a second kernel).
NIB_API int nib_attention_decode_tma(const void* qkv, int q_stride, void* out, const int* ctx_lens,
                                     const int* block_table, int bt_stride, int page_size, const void* k_pages,
                                     const void* v_pages, int num_pages, int n_tokens, int heads, int kv_heads,
                                     int head_dim, float scale, int window, int splits, int own_kv, float* part_o,
                                     float* part_ml, cudaStream_t stream) {
    NIB_REQUIRE(nib_attention_decode_tma_supported(heads, kv_heads, head_dim, page_size),
                "attention decode (TMA): head_dim %d, %d/%d heads, page size %d are not supported", head_dim, heads, kv_heads, page_size);
    NIB_REQUIRE(n_tokens >= 0 && num_pages > 0 && window >= 0 && splits >= 1 && splits <= 64, "attention decode (TMA): bad sizes (1..64 splits)");
    const int csize = splits >= 8 ? 8 : splits;
    NIB_REQUIRE((csize & (csize - 1)) == 0 && splits % csize == 0,
                "attention decode (TMA): %d splits; 1, 2, 4, 8 or a multiple of 8 are possible", splits);
    NIB_REQUIRE(splits == csize || (part_o && part_ml), "attention decode (TMA): more than 8 splits need scratch memory");
    NIB_REQUIRE(n_tokens <= 65535 && kv_heads <= 65535, "attention decode (TMA): too many tokens or kv heads for one launch");
    NIB_REQUIRE((((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0 && q_stride % 2 == 0, "attention decode (TMA): the pools must be 16-byte aligned, rows 4-byte aligned");
    NIB_REQUIRE((long long)num_pages * kv_heads < (1LL << 31) - 1, "attention decode (TMA): too many pages");
    if (n_tokens == 0) return 0;
    CUtensorMap mk, mv;
    const long long planes = (long long)num_pages * kv_heads;
    if (make_pool_map(&mk, k_pages, head_dim, page_size, planes)) return 1;
    if (make_pool_map(&mv, v_pages, head_dim, page_size, planes)) return 1;
#define CALL(HD, NH) launch<HD, NH>(mk, mv, qkv, q_stride, out, ctx_lens, block_table, bt_stride, page_size, num_pages, n_tokens, heads, \
                                    kv_heads, scale, window, splits, csize, own_kv, part_o, part_ml, stream)
    if (heads / kv_heads <= 8) return head_dim == 64 ? CALL(64, 1) : CALL(128, 1);
    return head_dim == 64 ? CALL(64, 2) : CALL(128, 2);
#undef CALL
}
