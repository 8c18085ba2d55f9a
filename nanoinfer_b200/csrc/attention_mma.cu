// Paged attention on the tensor cores (bfloat16 operands, 32-bit accumulation and softmax), for head
// sizes 16..128 in steps of 16. Two kernels share their building blocks:
//
//  * prefill: a tile of 64 rows per CTA, where a row is one (token, query head of the kv group), so
//    the keys and values of a kv head are read once for all the query heads that share it; key tiles of
//    64 through the block table, online softmax, causal and window masks by absolute position.
//  * decode: the rows are the query heads of ONE token's kv group (at most 16); the four warps of a CTA
//    each take a quarter of every key tile, several CTAs split the keys of a long context, and a
//    combine kernel merges the partial (max, sum, output) triples in a fixed order.
//
// Formula as in attention_generic.cu (cpp/src/ops.cpp:206-270): score = dot * scale, keys lo..p, softmax
// with the max subtracted, weighted sum of values. The reference's counterparts are SIMT:
// cpp/src/cuda/cuda_backend.cu:489-575 (tiled prefill), :578-640 and :331-352 (split-KV and combine).
//
// Tensor-core path: mma.sync m16n8k16 with ldmatrix from padded shared-memory tiles filled by cp.async.
#include "attention_common.cuh"

namespace {

constexpr int BLOCK_N = 64;     // keys per tile
constexpr int WARPS = 4;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Shared-memory tile of BLOCK_N rows of HD bfloat16, each row padded by 16 bytes: the row stride in
// 32-bit words is 4 mod 8, so the eight rows of an ldmatrix 8x8 block fall into distinct banks.
template <int HD> struct Tile {
    static constexpr int ROW_BYTES = HD * 2 + 16;
    static constexpr int BYTES = BLOCK_N * ROW_BYTES;
    static constexpr int CHUNKS_PER_ROW = HD / 8;            // 16-byte chunks
};

// Copies keys and values key0..key0+63 of one kv head into a K tile and a V tile; rows outside [lo, hi] or
// without a page are zero. A row's page is looked up once for both tensors; for the usual power-of-two page
// sizes the division is a shift (shift >= 0).
template <int HD, int THREADS>
__device__ __forceinline__ void load_tiles(unsigned char* k_tile, unsigned char* v_tile,
                                           const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                                           const int* __restrict__ bt, int page_size, int shift, int num_pages,
                                           int kv_heads, int kvh, int key0, int lo, int hi, int tid) {
    constexpr int CPR = Tile<HD>::CHUNKS_PER_ROW;
    constexpr int TOTAL = BLOCK_N * CPR;
#pragma unroll
    for (int i = tid; i < TOTAL; i += THREADS) {
        const int r = i / CPR, c = i - r * CPR;
        const int j = key0 + r;
        bool valid = (j >= lo) && (j <= hi);
        size_t off = 0;
        if (valid) {
            const int lp = shift >= 0 ? (j >> shift) : (j / page_size);
            const int slot = shift >= 0 ? (j & (page_size - 1)) : (j - lp * page_size);
            const int page = bt[lp];
            valid = page >= 0 && page < num_pages;
            if (valid) off = (((size_t)page * kv_heads + kvh) * page_size + slot) * HD + c * 8;
        }
        cp_async_16(k_tile + r * Tile<HD>::ROW_BYTES + c * 16, k_pages + off, valid);
        cp_async_16(v_tile + r * Tile<HD>::ROW_BYTES + c * 16, v_pages + off, valid);
    }
}

// S[16 x (8*NT)] += Q[16 x HD] . K^T for the key rows row0.. of a tile. q: A fragments per 16 dims.
template <int HD, int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const unsigned (&q)[HD / 16][4],
                                        const unsigned char* k_tile, int row0, int lane) {
    // ldmatrix.x4 addresses: matrices (keys 0-7, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 0-7), (keys 8-15, dims 8-15)
    const int mat = lane >> 3, rr = lane & 7;
    const int key_off = (mat >> 1) * 8 + rr, dim_off = (mat & 1) * 8;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            unsigned b[4];
            ldmatrix_x4(b, k_tile + (row0 + np * 16 + key_off) * Tile<HD>::ROW_BYTES + (kk * 16 + dim_off) * 2);
            mma_bf16(s[2 * np], q[kk], b[0], b[1]);
            mma_bf16(s[2 * np + 1], q[kk], b[2], b[3]);
        }
    }
}

// O[16 x HD] += P[16 x (16*KB)] . V for the value rows row0.. of a tile. p: A fragments per 16 keys.
template <int HD, int KB>
__device__ __forceinline__ void pv_tile(float (&o)[HD / 8][4], const unsigned (&p)[KB][4],
                                        const unsigned char* v_tile, int row0, int lane) {
    // transposed ldmatrix.x4: matrices (keys 0-7, dims 0-7), (keys 8-15, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 8-15)
    const int mat = lane >> 3, rr = lane & 7;
    const int key_off = (mat & 1) * 8 + rr, dim_off = (mat >> 1) * 8;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
            unsigned b[4];
            ldmatrix_x4_trans(b, v_tile + (row0 + kb * 16 + key_off) * Tile<HD>::ROW_BYTES + (dp * 16 + dim_off) * 2);
            mma_bf16(o[2 * dp], p[kb], b[0], b[1]);
            mma_bf16(o[2 * dp + 1], p[kb], b[2], b[3]);
        }
    }
}

// ------------------------------------------------------------------------------------------ prefill
// grid: (row tiles of 64, requests, kv heads). Rows of a request and kv head: r = token * n_rep + g.
template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ qkv, int q_stride, __nv_bfloat16* __restrict__ out,
                         const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
                         const int* __restrict__ block_table, int bt_stride, int page_size,
                         const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                         int num_pages, int heads, int kv_heads, float scale, int window) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    const int req = blockIdx.y, kvh = blockIdx.z;
    const int n_rep = heads / kv_heads;
    const int row_begin = q_start[req], q_len = q_start[req + 1] - row_begin;
    const int rows_total = q_len * n_rep;
    const int row0 = blockIdx.x * (WARPS * 16);
    if (row0 >= rows_total) return;
    const int ctx = ctx_lens[req];
    const int pos0 = ctx - q_len;                     // position of the request's first token in this step
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2;
    const int* bt = block_table + (size_t)req * bt_stride;
    const int shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    // this thread's two rows
    int vis_lo[2], vis_hi[2];
    const __nv_bfloat16* q_ptr[2];
    int out_off[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + warp * 16 + g + 8 * r;
        if (row < rows_total) {
            const int ti = row / n_rep, head = kvh * n_rep + (row - ti * n_rep);
            const int p = pos0 + ti;
            vis_hi[r] = p;
            vis_lo[r] = window > 0 ? max(0, p - window + 1) : 0;
            q_ptr[r] = qkv + (size_t)(row_begin + ti) * q_stride + (size_t)head * HD;
            out_off[r] = (row_begin + ti) * heads * HD + head * HD;
        } else {
            vis_hi[r] = -1; vis_lo[r] = 0; q_ptr[r] = nullptr; out_off[r] = -1;
        }
    }
    // key range of the whole CTA
    const int last_row = min(rows_total, row0 + WARPS * 16) - 1;
    const int hi_cta = pos0 + last_row / n_rep;
    const int lo_cta = window > 0 ? max(0, pos0 + row0 / n_rep - window + 1) : 0;
    const int t_begin = lo_cta / BLOCK_N, t_end = hi_cta / BLOCK_N;

    pdl_wait();     // queries, and the keys and values of this step's tokens, come from the kernels before
    unsigned q[HD / 16][4];
    load_q<HD>(q, q_ptr, lane);

    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float scale2 = scale * LOG2E;

    unsigned char* k_buf[2] = {smem, smem + 2 * Tile<HD>::BYTES};
    unsigned char* v_buf[2] = {smem + Tile<HD>::BYTES, smem + 3 * Tile<HD>::BYTES};

    load_tiles<HD, WARPS * 32>(k_buf[0], v_buf[0], k_pages, v_pages, bt, page_size, shift, num_pages, kv_heads, kvh, t_begin * BLOCK_N, lo_cta, hi_cta, tid);
    cp_async_commit();

    for (int tile = t_begin; tile <= t_end; ++tile) {
        const int cur = (tile - t_begin) & 1;
        if (tile < t_end) {
            load_tiles<HD, WARPS * 32>(k_buf[cur ^ 1], v_buf[cur ^ 1], k_pages, v_pages, bt, page_size, shift, num_pages, kv_heads, kvh, (tile + 1) * BLOCK_N, lo_cta, hi_cta, tid);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        float s[BLOCK_N / 8][4];
#pragma unroll
        for (int n = 0; n < BLOCK_N / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        qk_tile<HD, BLOCK_N / 8>(s, q, k_buf[cur], 0, lane);
        unsigned p[BLOCK_N / 16][4];
        softmax_block<HD, BLOCK_N / 8>(s, p, o, m_run, l_run, scale2, tile * BLOCK_N, vis_lo, vis_hi, lane);
        pv_tile<HD, BLOCK_N / 16>(o, p, v_buf[cur], 0, lane);
        __syncthreads();    // the tile may be overwritten by the load issued in the next iteration
    }
    cp_async_wait<0>();

    const int t = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (out_off[r] < 0) continue;
        const float inv = l_run[r] > 0.f ? 1.0f / l_run[r] : 0.f;
        __nv_bfloat16* orow = out + out_off[r];
#pragma unroll
        for (int d = 0; d < HD / 8; ++d)
            *reinterpret_cast<unsigned*>(orow + d * 8 + 2 * t) = pack_bf16(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
    }
}

// ------------------------------------------------------------------------------------------ decode
// grid: (splits, tokens, kv heads). Every token has q_len 1; its position is ctx_len - 1.
// part_o: [tokens, heads, splits, HD] float, part_ml: [tokens, heads, splits, 2] (max in log2 units, sum).
template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ qkv, int q_stride, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ ctx_lens, const int* __restrict__ block_table, int bt_stride,
                        int page_size, const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages, int num_pages, int heads, int kv_heads,
                        float scale, int window, int splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ counters) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_last;
    pdl_launch_dependents();
    const int split = blockIdx.x, token = blockIdx.y, kvh = blockIdx.z;
    const int n_rep = heads / kv_heads;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int p = ctx_lens[token] - 1;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int* bt = block_table + (size_t)token * bt_stride;
    const int shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    // key tiles of this split: tiles are aligned to absolute multiples of 64
    const int t_first = lo / BLOCK_N, t_last = p / BLOCK_N;
    const int n_tiles = t_last - t_first + 1;
    const int per = (n_tiles + splits - 1) / splits;
    const int t_begin = t_first + split * per;
    const int t_end = min(t_last, t_begin + per - 1);

    int vis_lo[2] = {lo, lo}, vis_hi[2] = {g < n_rep ? p : -1, -1};      // rows g+8 exist only if n_rep > 8
    const __nv_bfloat16* q_ptr[2] = {nullptr, nullptr};
    if (g < n_rep) q_ptr[0] = qkv + (size_t)token * q_stride + (size_t)(kvh * n_rep + g) * HD;
    if (g + 8 < n_rep) { q_ptr[1] = qkv + (size_t)token * q_stride + (size_t)(kvh * n_rep + g + 8) * HD; vis_hi[1] = p; }

    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float scale2 = scale * LOG2E;

    unsigned char* k_buf[2] = {smem, smem + 2 * Tile<HD>::BYTES};
    unsigned char* v_buf[2] = {smem + Tile<HD>::BYTES, smem + 3 * Tile<HD>::BYTES};
    auto issue = [&](int tile, int buf) {
        load_tiles<HD, WARPS * 32>(k_buf[buf], v_buf[buf], k_pages, v_pages, bt, page_size, shift, num_pages, kv_heads, kvh, tile * BLOCK_N, lo, p, tid);
    };

    // Two tiles are kept in flight. Keys and values of positions before p were written by earlier steps,
    // so tiles that do not hold p may be fetched before the wait for the kernels of this step; the tile
    // that holds p (this step's own key and value) and the queries only after it.
    const int own = t_last;                        // the tile that holds position p
    bool issued0 = false, issued1 = false;
    if (t_begin <= t_end && t_begin < own) { issue(t_begin, 0); issued0 = true; }
    cp_async_commit();
    if (issued0 && t_begin + 1 <= t_end && t_begin + 1 < own) { issue(t_begin + 1, 1); issued1 = true; }
    cp_async_commit();
    pdl_wait();
    unsigned q[HD / 16][4];
    load_q<HD>(q, q_ptr, lane);
    if (!issued0) {
        if (t_begin <= t_end) issue(t_begin, 0);
        cp_async_commit();
    }
    if (!issued1) {
        if (t_begin + 1 <= t_end) issue(t_begin + 1, 1);
        cp_async_commit();
    }
    // groups committed so far, oldest first: tile t_begin, tile t_begin + 1 (possibly with empty groups between)
    for (int tile = t_begin; tile <= t_end; ++tile) {
        const int cur = (tile - t_begin) & 1;
        cp_async_wait<1>();                        // everything but the newest group: tile `tile` has landed
        __syncthreads();
        // each warp takes 16 keys of the tile
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        qk_tile<HD, 2>(s, q, k_buf[cur], warp * 16, lane);
        unsigned pfrag[1][4];
        softmax_block<HD, 2>(s, pfrag, o, m_run, l_run, scale2, tile * BLOCK_N + warp * 16, vis_lo, vis_hi, lane);
        pv_tile<HD, 1>(o, pfrag, v_buf[cur], warp * 16, lane);
        __syncthreads();
        if (tile + 2 <= t_end) issue(tile + 2, cur);
        cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();

    // merge the four warps through shared memory (the tiles are no longer needed)
    constexpr int MS = HD + 4;                                    // row stride of the merge buffer (padded against bank conflicts)
    float* sm_o = reinterpret_cast<float*>(smem);                 // [WARPS][16][MS]
    float* sm_ml = sm_o + WARPS * 16 * MS;                        // [WARPS][16][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
#pragma unroll
        for (int d = 0; d < HD / 8; ++d) {
            *reinterpret_cast<float2*>(&sm_o[(warp * 16 + row) * MS + d * 8 + 2 * t]) = make_float2(o[d][2 * r], o[d][2 * r + 1]);
        }
        if (t == 0) {
            sm_ml[(warp * 16 + row) * 2] = m_run[r];
            sm_ml[(warp * 16 + row) * 2 + 1] = l_run[r];
        }
    }
    __syncthreads();
    for (int i = tid; i < n_rep * HD; i += WARPS * 32) {
        const int row = i / HD, d = i - row * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_ml[(w * 16 + row) * 2]);
        float l = 0.f, acc = 0.f;
        if (m != -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float mw = sm_ml[(w * 16 + row) * 2];
                const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
                l += sm_ml[(w * 16 + row) * 2 + 1] * f;
                acc += sm_o[(w * 16 + row) * MS + d] * f;
            }
        }
        const int head = kvh * n_rep + row;
        if (splits == 1) {
            out[((size_t)token * heads + head) * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else {
            const size_t slot = ((size_t)token * heads + head) * splits + split;
            part_o[slot * HD + d] = acc;
            if (d == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
        }
    }
    if (splits == 1 || counters == nullptr) return;     // without counters a second kernel merges the splits

    // The CTA that arrives last at this (token, kv head)'s counter merges the splits, in split order.
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(&counters[token * kv_heads + kvh], 1) == splits - 1) ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float* c_m = reinterpret_cast<float*>(smem);                 // [n_rep][splits] maxima, then factors
    float* c_l = c_m + 16 * 64;                                  // [n_rep] sums
    const size_t th0 = (size_t)token * heads + (size_t)kvh * n_rep;
    for (int i = tid; i < n_rep * splits; i += WARPS * 32) {
        const int row = i / splits, sp = i - row * splits;
        c_m[row * 64 + sp] = __ldcg(part_ml + ((th0 + row) * splits + sp) * 2);
    }
    __syncthreads();
    if (tid < n_rep) {
        float m = -INFINITY;
        for (int sp = 0; sp < splits; ++sp) m = fmaxf(m, c_m[tid * 64 + sp]);
        float l = 0.f;
        for (int sp = 0; sp < splits; ++sp) {
            const float ms = c_m[tid * 64 + sp];
            const float f = (m == -INFINITY || ms == -INFINITY) ? 0.f : exp2f(ms - m);
            l += __ldcg(part_ml + ((th0 + tid) * splits + sp) * 2 + 1) * f;
            c_m[tid * 64 + sp] = f;
        }
        c_l[tid] = l;
    }
    __syncthreads();
    for (int i = tid; i < n_rep * HD; i += WARPS * 32) {
        const int row = i / HD, d = i - row * HD;
        const float* po = part_o + (th0 + row) * splits * HD + d;
        const float* f = c_m + row * 64;
        float acc = 0.f;
        int sp = 0;
        for (; sp + 8 <= splits; sp += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(po + (size_t)(sp + u) * HD);
#pragma unroll
            for (int u = 0; u < 8; ++u) acc += v[u] * f[sp + u];
        }
        for (; sp < splits; ++sp) acc += __ldcg(po + (size_t)sp * HD) * f[sp];
        const float l = c_l[row];
        out[(th0 + row) * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
    if (tid == 0) counters[token * kv_heads + kvh] = 0;         // ready for the next launch
}

// Merges the partial results of the splits, in split order. grid: tokens * heads; block: 128 threads.
// The (max, sum) pairs of all splits are fetched at once into shared memory, and the partial outputs are
// read in unrolled batches, so the block waits for memory a few times, not once per split.
__global__ void __launch_bounds__(128)
attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         __nv_bfloat16* __restrict__ out, int splits, int hd) {
    __shared__ float s_m[64], s_f[64];
    __shared__ float s_l;
    pdl_launch_dependents();
    pdl_wait();
    const size_t th = blockIdx.x;
    const int tid = threadIdx.x;
    if (tid < splits) s_m[tid] = __ldcg(part_ml + (th * splits + tid) * 2);
    if (tid >= 64 && tid - 64 < splits) s_f[tid - 64] = __ldcg(part_ml + (th * splits + (tid - 64)) * 2 + 1);   // sums, for now
    __syncthreads();
    if (tid == 0) {
        float m = -INFINITY;
        for (int s = 0; s < splits; ++s) m = fmaxf(m, s_m[s]);
        float l = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float f = (m == -INFINITY || s_m[s] == -INFINITY) ? 0.f : exp2f(s_m[s] - m);
            l += s_f[s] * f;
            s_f[s] = f;                                   // from here on: the factor of split s
        }
        s_l = l;
    }
    __syncthreads();
    if (tid >= hd) return;
    const float* po = part_o + th * splits * hd + tid;
    float acc = 0.f;
    int s = 0;
    for (; s + 8 <= splits; s += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldcg(po + (size_t)(s + u) * hd);
#pragma unroll
        for (int u = 0; u < 8; ++u) acc += v[u] * s_f[s + u];
    }
    for (; s < splits; ++s) acc += __ldcg(po + (size_t)s * hd) * s_f[s];
    out[th * hd + tid] = __float2bfloat16_rn(s_l > 0.f ? acc / s_l : 0.f);
}

template <int HD> int prefill_smem() { return 4 * Tile<HD>::BYTES; }
template <int HD> int decode_smem() {
    const int tiles = 4 * Tile<HD>::BYTES, merge = WARPS * 16 * (HD + 4 + 2) * 4, combine = (16 * 64 + 16) * 4;
    const int a = tiles > merge ? tiles : merge;
    return a > combine ? a : combine;
}

template <int HD>
int launch_prefill(const void* qkv, int q_stride, void* out, const int* q_start, const int* ctx_lens,
                   const int* block_table, int bt_stride, int page_size, const void* k_pages, const void* v_pages,
                   int num_pages, int n_req, int max_q_len, int heads, int kv_heads, float scale, int window,
                   cudaStream_t stream) {
    static bool configured = false;
    const int smem = prefill_smem<HD>();
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    const int n_rep = heads / kv_heads;
    dim3 grid(ceil_div((long long)max_q_len * n_rep, WARPS * 16), n_req, kv_heads);
    NIB_CUDA(launch_pdl(attention_prefill_kernel<HD>, grid, dim3(WARPS * 32), (size_t)smem, stream,
                        (const __nv_bfloat16*)qkv, q_stride, (__nv_bfloat16*)out, q_start, ctx_lens, block_table, bt_stride,
                        page_size, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, num_pages, heads, kv_heads,
                        scale, window));
    return 0;
}

template <int HD>
int launch_decode(const void* qkv, int q_stride, void* out, const int* ctx_lens, const int* block_table,
                  int bt_stride, int page_size, const void* k_pages, const void* v_pages, int num_pages,
                  int n_tokens, int heads, int kv_heads, float scale, int window, int splits, float* part_o,
                  float* part_ml, int* counters, cudaStream_t stream) {
    static bool configured = false;
    const int smem = decode_smem<HD>();
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    dim3 grid(splits, n_tokens, kv_heads);
    NIB_CUDA(launch_pdl(attention_decode_kernel<HD>, grid, dim3(WARPS * 32), (size_t)smem, stream,
                        (const __nv_bfloat16*)qkv, q_stride, (__nv_bfloat16*)out, ctx_lens, block_table, bt_stride, page_size,
                        (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, num_pages, heads, kv_heads, scale,
                        window, splits, part_o, part_ml, counters));
    if (splits > 1 && counters == nullptr)
        NIB_CUDA(launch_pdl(attention_combine_kernel, dim3(n_tokens * heads), dim3(128), (size_t)0, stream,
                            (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, splits, HD));
    return 0;
}

}  // namespace

#define NIB_HD_SWITCH(hd, CALL)                      \
    switch (hd) {                                    \
        case 16: return CALL(16);                    \
        case 32: return CALL(32);                    \
        case 48: return CALL(48);                    \
        case 64: return CALL(64);                    \
        case 80: return CALL(80);                    \
        case 96: return CALL(96);                    \
        case 112: return CALL(112);                  \
        case 128: return CALL(128);                  \
        default: break;                              \
    }

// Merges the partial (max, sum, output) triples of `splits` key ranges, in split order: part_o [rows, splits,
// head_dim], part_ml [rows, splits, 2] (max in log2 units, sum) -> out [rows, head_dim] bfloat16.
NIB_API int nib_attention_combine(const float* part_o, const float* part_ml, void* out, int rows, int splits,
                                  int head_dim, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && splits >= 1 && splits <= 64 && head_dim >= 1 && head_dim <= 128, "attention combine: bad sizes");
    if (rows == 0) return 0;
    NIB_CUDA(launch_pdl(attention_combine_kernel, dim3(rows), dim3(128), (size_t)0, stream, part_o, part_ml,
                        (__nv_bfloat16*)out, splits, head_dim));
    return 0;
}

// 1 if the tensor-core kernels take this head size and grouping, else 0 (the caller then uses the general kernel).
NIB_API int nib_attention_mma_supported(int heads, int kv_heads, int head_dim) {
    if (kv_heads <= 0 || heads % kv_heads) return 0;
    return head_dim >= 16 && head_dim <= 128 && head_dim % 16 == 0;
}

// Requests q_start[0..n_req], rows of every request contiguous; bfloat16 only.
NIB_API int nib_attention_prefill_mma(const void* qkv, int q_stride, void* out, const int* q_start, const int* ctx_lens,
                                      const int* block_table, int bt_stride, int page_size, const void* k_pages,
                                      const void* v_pages, int num_pages, int n_req, int max_q_len, int heads,
                                      int kv_heads, int head_dim, float scale, int window, cudaStream_t stream) {
    NIB_REQUIRE(nib_attention_mma_supported(heads, kv_heads, head_dim), "attention (tensor cores): head_dim %d with %d/%d heads is not supported", head_dim, heads, kv_heads);
    NIB_REQUIRE(n_req >= 0 && max_q_len > 0 && page_size > 0 && num_pages > 0 && window >= 0, "attention prefill: bad sizes");
    NIB_REQUIRE(q_stride % 2 == 0 && head_dim % 8 == 0, "attention prefill: rows must be 4-byte aligned");
    NIB_REQUIRE(n_req <= 65535 && kv_heads <= 65535, "attention prefill: too many requests or kv heads for one launch");
    if (n_req == 0) return 0;
#define CALL(HD) launch_prefill<HD>(qkv, q_stride, out, q_start, ctx_lens, block_table, bt_stride, page_size, k_pages, v_pages, num_pages, n_req, max_q_len, heads, kv_heads, scale, window, stream)
    NIB_HD_SWITCH(head_dim, CALL)
#undef CALL
    NIB_REQUIRE(false, "attention prefill: unreachable head_dim %d", head_dim);
}

// One token per request (q_len 1). part_o: [n_tokens, heads, splits, head_dim] float and part_ml:
// [n_tokens, heads, splits, 2] float are scratch, needed only when splits > 1. counters: n_tokens *
// kv_heads ints that are zero between launches (the kernel leaves them zero); with them the CTA that
// finishes last merges the splits, without them (nullptr) a second kernel does.
NIB_API int nib_attention_decode_mma(const void* qkv, int q_stride, void* out, const int* ctx_lens,
                                     const int* block_table, int bt_stride, int page_size, const void* k_pages,
                                     const void* v_pages, int num_pages, int n_tokens, int heads, int kv_heads,
                                     int head_dim, float scale, int window, int splits, float* part_o, float* part_ml,
                                     int* counters, cudaStream_t stream) {
    NIB_REQUIRE(nib_attention_mma_supported(heads, kv_heads, head_dim), "attention (tensor cores): head_dim %d with %d/%d heads is not supported", head_dim, heads, kv_heads);
    NIB_REQUIRE(heads / kv_heads <= 16, "attention decode: at most 16 query heads per kv head, got %d", heads / kv_heads);
    NIB_REQUIRE(n_tokens >= 0 && page_size > 0 && num_pages > 0 && window >= 0 && splits >= 1 && splits <= 64, "attention decode: bad sizes (1..64 splits)");
    NIB_REQUIRE(splits == 1 || (part_o && part_ml), "attention decode: splits > 1 need scratch memory");
    NIB_REQUIRE(n_tokens <= 65535 && kv_heads <= 65535, "attention decode: too many tokens or kv heads for one launch");
    if (n_tokens == 0) return 0;
#define CALL(HD) launch_decode<HD>(qkv, q_stride, out, ctx_lens, block_table, bt_stride, page_size, k_pages, v_pages, num_pages, n_tokens, heads, kv_heads, scale, window, splits, part_o, part_ml, counters, stream)
    NIB_HD_SWITCH(head_dim, CALL)
#undef CALL
    NIB_REQUIRE(false, "attention decode: unreachable head_dim %d", head_dim);
}

// ------------------------------------------------------------------------------------------ no allocation
// The split decode attention for callers that cannot allocate (see no_alloc.h). Its scratch is this
// file-scope device array. In host code the name `g_noalloc_scratch` is only a handle for the runtime,
// not a device address: the address a kernel can use comes from cudaGetSymbolAddress, once per device.
#include "no_alloc.h"

static __device__ __align__(256) unsigned char g_noalloc_scratch[NIB_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
}

NIB_API int nib_attention_decode_noalloc(const void* qkv, int q_stride, void* out, const int* ctx_lens,
                                         const int* block_table, int bt_stride, int page_size, const void* k_pages,
                                         const void* v_pages, int num_pages, int n_tokens, int heads, int kv_heads,
                                         int head_dim, float scale, int window, int splits, cudaStream_t stream) {
    NIB_REQUIRE(n_tokens >= 0 && heads > 0 && head_dim > 0 && splits >= 1, "attention decode (no allocation): bad sizes");
    const unsigned long long need = (unsigned long long)n_tokens * heads * splits * (head_dim + 2) * sizeof(float);
    NIB_REQUIRE(need <= NIB_NOALLOC_SCRATCH_BYTES,
                "attention decode (no allocation): %d tokens x %d heads x %d splits x head_dim %d need %llu bytes of scratch, "
                "the built-in array has %u; use fewer splits or tokens, or nib_attention_decode_mma with your own scratch",
                n_tokens, heads, splits, head_dim, need, (unsigned)NIB_NOALLOC_SCRATCH_BYTES);
    int dev = -1;
    NIB_CUDA(cudaGetDevice(&dev));
    NIB_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, "attention decode (no allocation): device index %d is out of range", dev);
    if (g_noalloc_ptr[dev] == nullptr) {          // set-up: first call on this device
        void* p = nullptr;
        NIB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        NIB_REQUIRE(p != nullptr, "attention decode (no allocation): the scratch array has no address on device %d", dev);
        g_noalloc_ptr[dev] = static_cast<float*>(p);
    }
    float* part_o = g_noalloc_ptr[dev];
    float* part_ml = part_o + (size_t)n_tokens * heads * splits * head_dim;
    return nib_attention_decode_mma(qkv, q_stride, out, ctx_lens, block_table, bt_stride, page_size, k_pages, v_pages,
                                    num_pages, n_tokens, heads, kv_heads, head_dim, scale, window, splits, part_o,
                                    part_ml, nullptr, stream);
}
