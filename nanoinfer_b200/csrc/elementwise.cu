// Embedding gather, RMSNorm, and rotation of queries and keys fused with the write of keys and
// values into the cache pages. All arithmetic is 32-bit; T is the storage type of activations,
// tables and cache (float or bfloat16).
//
// Reference formulas: cpp/src/ops.cpp:71-84 (embedding), :272-292 (rmsnorm: eps inside the root),
// :146-168 (half-split rotation), cpp/src/cuda/cuda_backend.cu:354-367 (page write through the
// block table). The reference runs these as separate one-thread-per-element kernels
// (cpp/src/cuda/cuda_elementwise.cu:26-135) with one thread per ROW for the norm.
#include "common.cuh"

// ---------------------------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ out, int hidden, int vocab, unsigned long long* trace, int trace_cap) {
    const int m = blockIdx.x;
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_EMBED, 0, 1);
    const int id = ids[m];
    float* o = out + (size_t)m * hidden;
    if (id < 0 || id >= vocab) {  // the engine checks ids on the host; never read outside the table
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = Elem<T>::load(src + c);
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_EMBED, 0, 2);
}

NIB_API int nib_embed(const int* ids, const void* table, float* out, int m, int hidden, int vocab,
                      int dtype, cudaStream_t stream) {
    NIB_REQUIRE(m >= 0 && hidden > 0 && vocab > 0, "embed: bad sizes m=%d hidden=%d vocab=%d", m, hidden, vocab);
    if (m == 0) return 0;
    const int threads = hidden >= 256 ? 256 : 64;
    if (dtype == NIB_F32)
        embed_kernel<float><<<m, threads, 0, stream>>>(ids, (const float*)table, out, hidden, vocab, nib_trace_buffer(), nib_trace_capacity());
    else if (dtype == NIB_BF16)
        embed_kernel<__nv_bfloat16><<<m, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, out, hidden, vocab, nib_trace_buffer(), nib_trace_capacity());
    else
        NIB_REQUIRE(false, "embed: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- RMSNorm
// One block per output row. The sum of squares is reduced in a fixed order (thread-strided partial
// sums, warp butterflies, then warp 0 over the warps), so a row's result does not depend on which
// other rows are in the batch.
template <typename T, int THREADS>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                               const int* __restrict__ rows, T* __restrict__ out, int hidden, float eps) {
    __shared__ float warp_part[THREADS / 32];
    __shared__ float s_scale;
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += THREADS) {
        const float v = xr[c];
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < THREADS / 32 ? warp_part[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) s_scale = 1.0f / sqrtf(v / (float)hidden + eps);
    }
    __syncthreads();
    const float scale = s_scale;
    T* o = out + (size_t)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += THREADS) Elem<T>::store(o + c, xr[c] * scale * gain[c]);
}

// One WARP per output row, for widths that are multiples of 4 up to 128 * NV: the row stays in registers
// (NV float4 per lane) between the sum of squares and the scaling, so it is read once, with 16-byte
// loads; no shared memory, no block barrier. Which kernel runs depends on the width alone, so a row's
// result still does not depend on the batch.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ gain, const int* __restrict__ rows,
                    T* __restrict__ out, int n_rows, int hidden, float eps, int late_dependents, unsigned long long* trace, int trace_cap) {
    // late_dependents: the kernel behind this one starts only when this kernel's loads are out (see nib_rmsnorm)
    if (!late_dependents) pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_RMSNORM, 0, 0);
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int n4 = hidden >> 2;
    float4 g[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {       // the gains are weights: fetched before the wait
        const int c = lane + 32 * i;
        g[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(gain) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_RMSNORM, 0, 1);
    if (r >= n_rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * hidden);
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = warp_sum(ss);
    if (late_dependents) pdl_launch_dependents();
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    T* o = out + (size_t)r * hidden;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < n4) {
            const float a = v[i].x * scale * g[i].x, b = v[i].y * scale * g[i].y;
            const float cc = v[i].z * scale * g[i].z, d = v[i].w * scale * g[i].w;
            if constexpr (sizeof(T) == 4) {
                reinterpret_cast<float4*>(o)[c] = make_float4(a, b, cc, d);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(cc, d);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned*>(&lo);
                pk.y = *reinterpret_cast<unsigned*>(&hi);
                reinterpret_cast<uint2*>(o)[c] = pk;
            }
        }
    }
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_RMSNORM, 0, 2);
}

template <typename T>
int launch_rmsnorm_rows(const float* x, const float* gain, const int* rows, T* out, int n_rows, int hidden, float eps,
                        int late_dependents, cudaStream_t stream) {
    const int warps = n_rows >= 8 ? 8 : n_rows;           // rows per block
    const dim3 grid(ceil_div(n_rows, warps)), block(32 * warps);
    if (hidden <= 128 * 8)
        NIB_CUDA(launch_pdl(rmsnorm_rows_kernel<T, 8>, grid, block, (size_t)0, stream, x, gain, rows, out, n_rows, hidden, eps, late_dependents, nib_trace_buffer(), nib_trace_capacity()));
    else if (hidden <= 128 * 16)
        NIB_CUDA(launch_pdl(rmsnorm_rows_kernel<T, 16>, grid, block, (size_t)0, stream, x, gain, rows, out, n_rows, hidden, eps, late_dependents, nib_trace_buffer(), nib_trace_capacity()));
    else
        NIB_CUDA(launch_pdl(rmsnorm_rows_kernel<T, 32>, grid, block, (size_t)0, stream, x, gain, rows, out, n_rows, hidden, eps, late_dependents, nib_trace_buffer(), nib_trace_capacity()));
    return 0;
}

// late_dependents: the kernel launched behind this one (programmatic dependent launch) may start only when this kernel's
// loads are out, instead of at once. Right when that kernel has next to no set-up of its own and would only take issue
// slots and bandwidth meanwhile (the small-M product); wrong when it has a long set-up to hide (the tcgen05 products).
NIB_API int nib_rmsnorm(const float* x, const float* gain, const int* rows, void* out, int n_rows,
                        int hidden, float eps, int dtype, int late_dependents, cudaStream_t stream) {
    NIB_REQUIRE(n_rows >= 0 && hidden > 0, "rmsnorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    if (n_rows == 0) return 0;
    // rows of 16-byte multiples up to 4096 wide: a warp per row
    if (hidden % 4 == 0 && hidden <= 4096 && (((uintptr_t)x | (uintptr_t)gain | (uintptr_t)out) & 15) == 0 &&
        (dtype == NIB_F32 || dtype == NIB_BF16)) {
        const int rc = dtype == NIB_F32 ? launch_rmsnorm_rows<float>(x, gain, rows, (float*)out, n_rows, hidden, eps, late_dependents, stream)
                                        : launch_rmsnorm_rows<__nv_bfloat16>(x, gain, rows, (__nv_bfloat16*)out, n_rows, hidden, eps, late_dependents, stream);
        if (rc) return rc;
        NIB_LAUNCH_CHECK();
        return 0;
    }
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(rmsnorm_kernel<float, 256>, dim3(n_rows), dim3(256), (size_t)0, stream, x, gain, rows, (float*)out, hidden, eps));
    else if (dtype == NIB_BF16)
        NIB_CUDA(launch_pdl(rmsnorm_kernel<__nv_bfloat16, 256>, dim3(n_rows), dim3(256), (size_t)0, stream, x, gain, rows,
                            (__nv_bfloat16*)out, hidden, eps));
    else
        NIB_REQUIRE(false, "rmsnorm: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- rotation + page write
// qkv row layout: [heads | kv_heads | kv_heads] x head_dim. Queries and keys are rotated in place
// (pairs d, d + rot/2 for d < rot/2; elements >= rot are left as they are); rotated keys and the
// values are also written to the page of the token's position, if write_kv.
// Pages: [num_pages, kv_heads, page_size, head_dim].
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const int* __restrict__ req_index, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, int rot, const int* __restrict__ block_table,
                                  int bt_stride, int page_size, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                  int heads, int kv_heads, int head_dim, int num_pages, int write_kv) {
    pdl_launch_dependents();
    const int m = blockIdx.x;
    const int pos = positions[m];
    T* row = qkv + (size_t)m * (heads + 2 * kv_heads) * head_dim;
    const int half = rot / 2;
    long long page = -1;
    int off = 0;
    if (write_kv) {
        page = block_table[(size_t)req_index[m] * bt_stride + pos / page_size];
        off = pos % page_size;
        if (page < 0 || page >= num_pages) page = -1;  // never write outside the pool
    }
    pdl_wait();     // positions and block tables are the step's inputs; qkv is the previous kernel's output
    // rotated pairs of queries and keys
    const int pairs = (heads + kv_heads) * half;
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int h = i / half, d = i - h * half;
        const float c = cos_t[(size_t)pos * half + d], s = sin_t[(size_t)pos * half + d];
        T* p = row + (size_t)h * head_dim;
        const float x1 = Elem<T>::load(p + d), x2 = Elem<T>::load(p + d + half);
        const float o1 = x1 * c - x2 * s, o2 = x2 * c + x1 * s;
        Elem<T>::store(p + d, o1);
        Elem<T>::store(p + d + half, o2);
        if (h >= heads && page >= 0) {
            T* dst = k_pages + (((size_t)page * kv_heads + (h - heads)) * page_size + off) * head_dim;
            Elem<T>::store(dst + d, o1);
            Elem<T>::store(dst + d + half, o2);
        }
    }
    if (page < 0) return;
    // keys beyond the rotated width
    const int tail = head_dim - rot;
    for (int i = threadIdx.x; i < kv_heads * tail; i += blockDim.x) {
        const int h = i / tail, d = rot + (i - h * tail);
        k_pages[(((size_t)page * kv_heads + h) * page_size + off) * head_dim + d] =
            row[(size_t)(heads + h) * head_dim + d];
    }
    // values
    for (int i = threadIdx.x; i < kv_heads * head_dim; i += blockDim.x) {
        const int h = i / head_dim, d = i - h * head_dim;
        v_pages[(((size_t)page * kv_heads + h) * page_size + off) * head_dim + d] =
            row[(size_t)(heads + kv_heads + h) * head_dim + d];
    }
}

// The same for bfloat16 with 16-byte accesses: one thread per chunk of 8 elements. A token has
// (heads + kv_heads) * rot/16 rotation items (8 pairs each: two loads, two stores, and two more into the
// page for a key), kv_heads * (head_dim - rot)/8 items of keys beyond the rotated width and kv_heads *
// head_dim/8 items of values. The arithmetic per element is that of the kernel above, so are the bits.
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(h[i]); f[2 * i + 1] = __high2float(h[i]); }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return u;
}

__global__ void __launch_bounds__(256)
rope_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ req_index,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                      const int* __restrict__ block_table, int bt_stride, int page_size, __nv_bfloat16* __restrict__ k_pages,
                      __nv_bfloat16* __restrict__ v_pages, int m_tokens, int heads, int kv_heads, int head_dim, int num_pages,
                      int write_kv, unsigned long long* trace, int trace_cap) {
    pdl_launch_dependents();
    const int half = rot >> 1;
    const int rot_items = (heads + kv_heads) * (half >> 3);
    const int tail_items = write_kv ? kv_heads * ((head_dim - rot) >> 3) : 0;
    const int v_items = write_kv ? kv_heads * (head_dim >> 3) : 0;
    const int per_token = rot_items + tail_items + v_items;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (per_token == 0 || idx >= (long long)m_tokens * per_token) return;
    const int m = (int)(idx / per_token);
    int item = (int)(idx - (long long)m * per_token);
    const int pos = positions[m];
    long long page = -1;
    int off = 0;
    if (write_kv) {
        page = block_table[(size_t)req_index[m] * bt_stride + pos / page_size];
        off = pos % page_size;
        if (page < 0 || page >= num_pages) page = -1;  // never write outside the pool
    }
    __nv_bfloat16* row = qkv + (size_t)m * (heads + 2 * kv_heads) * head_dim;
    pdl_wait();     // positions and block tables are the step's inputs; qkv is the previous kernel's output
    if (idx == 0) nib_trace_mark(trace, trace_cap, NIB_TK_ROPE, 0, 1);
    if (item < rot_items) {
        const int per_head = half >> 3;
        const int h = item / per_head, d = (item - h * per_head) << 3;
        __nv_bfloat16* p = row + (size_t)h * head_dim;
        float x1[8], x2[8], c[8], sn[8], o1[8], o2[8];
        unpack8(*reinterpret_cast<const uint4*>(p + d), x1);
        unpack8(*reinterpret_cast<const uint4*>(p + d + half), x2);
        const float4* cp = reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + d);
        const float4* sp = reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + d);
        *reinterpret_cast<float4*>(&c[0]) = __ldg(cp); *reinterpret_cast<float4*>(&c[4]) = __ldg(cp + 1);
        *reinterpret_cast<float4*>(&sn[0]) = __ldg(sp); *reinterpret_cast<float4*>(&sn[4]) = __ldg(sp + 1);
#pragma unroll
        for (int i = 0; i < 8; ++i) { o1[i] = x1[i] * c[i] - x2[i] * sn[i]; o2[i] = x2[i] * c[i] + x1[i] * sn[i]; }
        const uint4 u1 = pack8(o1), u2 = pack8(o2);
        *reinterpret_cast<uint4*>(p + d) = u1;
        *reinterpret_cast<uint4*>(p + d + half) = u2;
        if (h >= heads && page >= 0) {
            __nv_bfloat16* dst = k_pages + (((size_t)page * kv_heads + (h - heads)) * page_size + off) * head_dim;
            *reinterpret_cast<uint4*>(dst + d) = u1;
            *reinterpret_cast<uint4*>(dst + d + half) = u2;
        }
        return;
    }
    if (page < 0) return;
    item -= rot_items;
    if (item < tail_items) {
        const int per_head = (head_dim - rot) >> 3;
        const int h = item / per_head, d = rot + ((item - h * per_head) << 3);
        *reinterpret_cast<uint4*>(k_pages + (((size_t)page * kv_heads + h) * page_size + off) * head_dim + d) =
            *reinterpret_cast<const uint4*>(row + (size_t)(heads + h) * head_dim + d);
        return;
    }
    item -= tail_items;
    const int per_head = head_dim >> 3;
    const int h = item / per_head, d = (item - h * per_head) << 3;
    *reinterpret_cast<uint4*>(v_pages + (((size_t)page * kv_heads + h) * page_size + off) * head_dim + d) =
        *reinterpret_cast<const uint4*>(row + (size_t)(heads + kv_heads + h) * head_dim + d);
}

NIB_API int nib_rope_store(void* qkv, const int* positions, const int* req_index, const float* cos_t,
                           const float* sin_t, int rot, const int* block_table, int bt_stride, int page_size,
                           void* k_pages, void* v_pages, int m, int heads, int kv_heads, int head_dim,
                           int num_pages, int write_kv, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(m >= 0 && heads > 0 && kv_heads > 0 && head_dim > 0, "rope_store: bad sizes");
    NIB_REQUIRE(rot >= 0 && rot <= head_dim && rot % 2 == 0, "rope_store: rotated width %d must be even and <= head_dim %d", rot, head_dim);
    NIB_REQUIRE(!write_kv || (block_table && k_pages && v_pages && page_size > 0 && num_pages > 0),
                "rope_store: write asked for without pages");
    if (m == 0) return 0;
    const int threads = 128;
    const bool aligned = ((((uintptr_t)qkv | (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) == 0) &&
                         (!write_kv || (((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0);
    if (dtype == NIB_BF16 && head_dim % 8 == 0 && rot % 16 == 0 && aligned) {
        const int half = rot / 2;
        const long long per_token = (long long)(heads + kv_heads) * (half / 8) +
                                    (write_kv ? (long long)kv_heads * ((head_dim - rot) / 8 + head_dim / 8) : 0);
        if (per_token == 0) return 0;
        const long long total = per_token * m;
        NIB_REQUIRE(total < (1LL << 31) * 256, "rope_store: too many elements for one launch");
        NIB_CUDA(launch_pdl(rope_store_vec_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), (size_t)0, stream,
                            (__nv_bfloat16*)qkv, positions, req_index, cos_t, sin_t, rot, block_table, bt_stride, page_size,
                            (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, m, heads, kv_heads, head_dim, num_pages, write_kv,
                            nib_trace_buffer(), nib_trace_capacity()));
        NIB_LAUNCH_CHECK();
        return 0;
    }
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(rope_store_kernel<float>, dim3(m), dim3(threads), (size_t)0, stream, (float*)qkv, positions, req_index,
                            cos_t, sin_t, rot, block_table, bt_stride, page_size, (float*)k_pages, (float*)v_pages, heads,
                            kv_heads, head_dim, num_pages, write_kv));
    else if (dtype == NIB_BF16)
        NIB_CUDA(launch_pdl(rope_store_kernel<__nv_bfloat16>, dim3(m), dim3(threads), (size_t)0, stream, (__nv_bfloat16*)qkv,
                            positions, req_index, cos_t, sin_t, rot, block_table, bt_stride, page_size, (__nv_bfloat16*)k_pages,
                            (__nv_bfloat16*)v_pages, heads, kv_heads, head_dim, num_pages, write_kv));
    else
        NIB_REQUIRE(false, "rope_store: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}
