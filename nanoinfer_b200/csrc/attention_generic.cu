// The general attention kernel over the paged cache: one warp per (token, query head), any mix of
// prompt portions and decoded tokens, any head size up to 256, any page size, grouped kv heads,
// optional window. All arithmetic is 32-bit whatever the storage type. It is the attention of the
// true 32-bit path and the fallback of the bfloat16 path.
//
// A query at position p sees the keys at positions lo..p of its own request (lo = 0, or
// p - window + 1 with a window), read from the cache through the request's block table; the keys
// of this step were written there before. Keys are taken in blocks of 32 that start at absolute
// multiples of 32, with a running max and sum (online softmax), so the result for a position does
// not depend on how the request was cut into steps, nor on what else is in the batch.
//
// Formula: cpp/src/ops.cpp:206-270 (score = dot * scale, scale after the dot; max-subtracted exp;
// sum of p_j v_j / sum p_j); kv head = head / (heads / kv_heads): cpp/src/paged.cpp:171. Warp-level
// online softmax in the reference: cpp/src/cuda/cuda_backend.cu:113-178, 419-487.
#include "common.cuh"

constexpr int GEN_MAX_D = 256;
constexpr int GEN_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(GEN_WARPS * 32)
attention_generic_kernel(const T* __restrict__ qkv, int q_stride, T* __restrict__ out,
                         const int* __restrict__ positions, const int* __restrict__ req_index,
                         const int* __restrict__ block_table, int bt_stride, int page_size,
                         const T* __restrict__ k_pages, const T* __restrict__ v_pages, int num_pages,
                         int m_tokens, int heads, int kv_heads, int head_dim, float scale, int window) {
    __shared__ float q_s[GEN_WARPS][GEN_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * GEN_WARPS + warp;
    if (w >= (long long)m_tokens * heads) return;
    const int token = (int)(w / heads), head = (int)(w % heads);
    const int kvh = head / (heads / kv_heads);
    const int pos = positions[token];
    const int* bt = block_table + (size_t)req_index[token] * bt_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    const T* q = qkv + (size_t)token * q_stride + (size_t)head * head_dim;
    for (int d = lane; d < head_dim; d += 32) q_s[warp][d] = Elem<T>::load(q + d);
    __syncwarp();

    float m_run = -INFINITY, l_run = 0.f;
    float acc[GEN_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < GEN_MAX_D / 32; ++i) acc[i] = 0.f;

    for (int kb = (lo / 32) * 32; kb <= pos; kb += 32) {
        const int j = kb + lane;
        const bool valid = (j >= lo) && (j <= pos);
        float s = -INFINITY;
        long long row = -1;  // element offset of this lane's key row in the pages
        if (valid) {
            const int page = bt[j / page_size];
            if (page >= 0 && page < num_pages) {
                row = (((long long)page * kv_heads + kvh) * page_size + (j % page_size)) * head_dim;
                const T* kr = k_pages + row;
                float dot = 0.f;
                for (int d = 0; d < head_dim; ++d) dot = fmaf(q_s[warp][d], Elem<T>::load(kr + d), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m_run, warp_max(s));
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        l_run = l_run * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < GEN_MAX_D / 32; ++i) acc[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long rj = __shfl_sync(0xffffffffu, row, jj);
            if (pj == 0.f || rj < 0) continue;  // uniform over the warp
            const T* vr = v_pages + rj;
#pragma unroll
            for (int i = 0; i < GEN_MAX_D / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, Elem<T>::load(vr + d), acc[i]);
            }
        }
        m_run = m_new;
    }
    T* o = out + (size_t)token * heads * head_dim + (size_t)head * head_dim;
    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
    for (int i = 0; i < GEN_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) Elem<T>::store(o + d, acc[i] * inv);
    }
}

// qkv: rows of q_stride elements whose first heads*head_dim are the (rotated) queries.
// out: [m_tokens, heads*head_dim]. Pages: [num_pages, kv_heads, page_size, head_dim].
NIB_API int nib_attention_generic(const void* qkv, int q_stride, void* out, const int* positions,
                                  const int* req_index, const int* block_table, int bt_stride, int page_size,
                                  const void* k_pages, const void* v_pages, int num_pages, int m_tokens,
                                  int heads, int kv_heads, int head_dim, float scale, int window, int dtype,
                                  cudaStream_t stream) {
    NIB_REQUIRE(m_tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "attention: bad head counts %d / %d", heads, kv_heads);
    NIB_REQUIRE(head_dim > 0 && head_dim <= GEN_MAX_D, "attention: head_dim %d is outside 1..%d", head_dim, GEN_MAX_D);
    NIB_REQUIRE(page_size > 0 && num_pages > 0 && window >= 0, "attention: bad page_size/num_pages/window");
    if (m_tokens == 0) return 0;
    const long long warps = (long long)m_tokens * heads;
    const int blocks = ceil_div(warps, GEN_WARPS);
    if (dtype == NIB_F32)
        attention_generic_kernel<float><<<blocks, GEN_WARPS * 32, 0, stream>>>((const float*)qkv, q_stride, (float*)out, positions,
            req_index, block_table, bt_stride, page_size, (const float*)k_pages, (const float*)v_pages, num_pages,
            m_tokens, heads, kv_heads, head_dim, scale, window);
    else if (dtype == NIB_BF16)
        attention_generic_kernel<__nv_bfloat16><<<blocks, GEN_WARPS * 32, 0, stream>>>((const __nv_bfloat16*)qkv, q_stride,
            (__nv_bfloat16*)out, positions, req_index, block_table, bt_stride, page_size, (const __nv_bfloat16*)k_pages,
            (const __nv_bfloat16*)v_pages, num_pages, m_tokens, heads, kv_heads, head_dim, scale, window);
    else
        NIB_REQUIRE(false, "attention: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}
