// Decode attention (one new token per request) with the key/value pages brought in by TMA.
//
// A page of one kv head is a dense block of page_size x head_dim bfloat16 in the pool, so one
// cp.async.bulk.tensor instruction of one lane fetches it whole, with the 128-byte swizzle that makes
// the ldmatrix reads conflict free; nobody computes addresses chunk by chunk. A page that the request
// does not hold (freed by a window, beyond the context, a padding row) is fetched at a coordinate
// outside the pool and arrives as zeros. Slots of a held page beyond the context hold finite values
// (the pool starts zeroed and only finite values are written), and their scores are masked.
//
// grid (splits, tokens, kv heads), 160 threads. A CTA walks over its tiles of 64 or 128 keys (aligned to
// absolute multiples of the tile) with STAGES tiles in flight: a producer warp issues the copies and runs
// ahead, a full and an empty mbarrier per stage hand the tiles back and forth, and no barrier of the
// whole CTA stands in the loop. Four consumer warps take 16 keys of every tile each, keep their own
// running (max, sum, output) and merge at the end. The rows of the mma tile are the query heads of
// the kv group (at most 16). With more than one split the partial triples go to scratch and a second kernel merges them in split order
// (nib_attention_combine).
//
// Every wait has an iteration limit; a wait that runs out sets an error word, the CTA stops, waits
// (bounded) for its copies in flight and returns.
//
// Formula as in attention_generic.cu (cpp/src/ops.cpp:206-270). The reference's decode attention is a
// SIMT split-KV kernel with a combine pass (cpp/src/cuda/cuda_backend.cu:578-640, :331-352).
#include "attention_common.cuh"
#include <cuda.h>

extern "C" int nib_attention_combine(const float* part_o, const float* part_ml, void* out, int rows, int splits,
                                     int head_dim, cudaStream_t stream);

namespace {

constexpr int WARPS = 4;          // consumer warps: 16 keys of every tile each; one more warp fetches
constexpr int THREADS = (WARPS + 1) * 32;
// Keys per tile: 128 for heads of 64 (a tile of 64 keys is only 16 KB there, and the fixed work per tile,
// barrier waits and the softmax's shuffles, bounded the kernel at large batches), 64 for heads of 128.
template <int HD> constexpr int keys_of() { return HD == 64 ? 128 : 64; }
constexpr unsigned WAIT_LIMIT = 1u << 22;

__device__ int g_dec_error = 0;   // 0, or (code << 16 | blockIdx.x) of the first wait that ran out

template <int HD> struct Cfg {
    static constexpr int KEYS = keys_of<HD>();
    static constexpr int WKEYS = KEYS / WARPS;                // keys of a tile per consumer warp: 32 or 16
    static constexpr int SUB = HD / 64;                       // 64-element column blocks of a head
    static constexpr int SUBTILE = KEYS * 128;                // KEYS rows of 128 bytes (64 elements of a head), swizzled
    static constexpr int TILE = SUB * SUBTILE;                // K (or V) of one tile
    static constexpr int STAGE = 2 * TILE;
    static constexpr int STAGES = 3;                          // 96 KB in flight, two CTAs per SM
    static constexpr int MERGE = WARPS * 16 * (HD + 4 + 2) * 4 + WARPS * 16 * 4;
    static constexpr int DATA = STAGES * STAGE > MERGE ? STAGES * STAGE : MERGE;
    static constexpr int SMEM = DATA + 1024 /* alignment */ + 64 /* barriers */;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (i > 256) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, unsigned long long* bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// FUSED: qkv is the raw projection. The queries are rotated as they are loaded; the warp whose 16 keys
// include the token's own position rotates the new key, puts key and value into its rows of the tile (the
// page's slot still holds old data there) and into the page for the steps to come. Nothing of this step is
// read from the pages then, so every tile may be fetched before the wait for the step's earlier kernels.
template <int HD, bool FUSED>
__global__ void __launch_bounds__(THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __nv_bfloat16* __restrict__ qkv, int q_stride, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ ctx_lens, const int* __restrict__ block_table, int bt_stride,
                            int page_size, int page_shift, int num_pages, int heads, int kv_heads, int n_rep, float scale,
                            int window, int splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                            __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot) {
    using C = Cfg<HD>;
    constexpr int KEYS = C::KEYS, SUBTILE = C::SUBTILE, WKEYS = C::WKEYS, NT = WKEYS / 8;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(smem + C::DATA);
    unsigned long long* empty = full + C::STAGES;
    __shared__ volatile int s_failed;

    pdl_launch_dependents();
    const int split = blockIdx.x, token = blockIdx.y, kvh = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
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
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();

    float o[HD / 8][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    if (warp == WARPS) {
        // ---------------- producer warp: lane i fetches page i of every tile (K and V), lane 0 arms the
        // stage's barrier. The block-table entry of the next tile is read while this one waits for its
        // stage. Keys and values of earlier positions were written by earlier steps, so their tiles are
        // fetched at once; the tile that holds p (this step's own key and value) waits for this step's
        // kernels.
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
            const int st = j % C::STAGES;
            const int z = z_next;
            z_next = plane_of(j + 1);
            if (!FUSED && t_begin + j == t_last && !waited) { pdl_wait(); waited = true; }
            int ok = 1;
            if (lane == 0) {
                if (j >= C::STAGES) ok = !s_failed && mbar_wait(&empty[st], ((j / C::STAGES) - 1) & 1);
                if (ok) mbar_expect_tx(&full[st], C::STAGE);
                else if (!s_failed) { atomicCAS(&g_dec_error, 0, (2 << 16) | (int)blockIdx.x); s_failed = 1; }
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
            for (int j = max(0, issued - C::STAGES); j < issued; ++j) mbar_wait(&full[j % C::STAGES], (j / C::STAGES) & 1);
        }
    } else {
        // ---------------- four consumer warps: 16 keys of every tile each
        pdl_wait();
        int vis_lo[2] = {lo, lo}, vis_hi[2] = {g < n_rep ? p : -1, -1};      // rows g+8 exist only if n_rep > 8
        const __nv_bfloat16* q_ptr[2] = {nullptr, nullptr};
        if (g < n_rep) q_ptr[0] = qkv + (size_t)token * q_stride + (size_t)(kvh * n_rep + g) * HD;
        if (g + 8 < n_rep) { q_ptr[1] = qkv + (size_t)token * q_stride + (size_t)(kvh * n_rep + g + 8) * HD; vis_hi[1] = p; }
        unsigned q[HD / 16][4];
        const float* cos_row = FUSED ? cos_t + (size_t)max(p, 0) * (rot >> 1) : nullptr;      // p < 0: a padding row
        const float* sin_row = FUSED ? sin_t + (size_t)max(p, 0) * (rot >> 1) : nullptr;
        if (FUSED) load_q_rotated<HD>(q, q_ptr, lane, cos_row, sin_row, rot);
        else load_q<HD>(q, q_ptr, lane);
#pragma unroll
        for (int d = 0; d < HD / 8; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
        const float scale2 = scale * LOG2E;

        // ldmatrix addresses inside a swizzled tile: row r (128 bytes), 16-byte chunk c at ((c ^ (r & 7)) << 4)
        const int mat = lane >> 3, rr = lane & 7;
        const unsigned k_row = (unsigned)(warp * WKEYS + (mat >> 1) * 8 + rr) * 128u;   // keys 0-7 / 8-15, dims 0-7 / 8-15
        const unsigned k_half = mat & 1;
        const unsigned v_row = (unsigned)(warp * WKEYS + (mat & 1) * 8 + rr) * 128u;    // transposed: keys 0-7 / 8-15 first
        const unsigned v_half = mat >> 1;

        for (int j = 0; j < n_mine; ++j) {
            const int st = j % C::STAGES;
            bool ok = !s_failed && mbar_wait(&full[st], (j / C::STAGES) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0 && !s_failed) { atomicCAS(&g_dec_error, 0, (1 << 16) | (int)blockIdx.x); s_failed = 1; }
                break;
            }
            const unsigned kt = smem_u32(smem + st * C::STAGE), vt = kt + C::TILE;
            if (FUSED && t_begin + j == t_last && p >= 0 && (p & (KEYS - 1)) / WKEYS == warp) {
                // this step's own key (rotated) and value: into this warp's rows of the tile and into the page
                const __nv_bfloat16* k_new = qkv + (size_t)token * q_stride + (size_t)(heads + kvh) * HD;
                const __nv_bfloat16* v_new = qkv + (size_t)token * q_stride + (size_t)(heads + kv_heads + kvh) * HD;
                const int r = p & (KEYS - 1);
                const int page = __ldg(bt + (p >> page_shift));
                const int slot = p & (page_size - 1);
                const bool has_page = page >= 0 && page < num_pages;
                const size_t off = has_page ? (((size_t)page * kv_heads + kvh) * page_size + slot) * HD : 0;
                unsigned char* k_tile = smem + st * C::STAGE;
                for (int d = 2 * lane; d < HD; d += 64) {
                    const unsigned kr = rotated_pair(k_new, d, cos_row, sin_row, rot);
                    const unsigned vr = *reinterpret_cast<const unsigned*>(v_new + d);
                    // element d of row r in a swizzled tile: column block d/64, 16-byte chunk (d%64)/8 at ((chunk ^ (r&7)) << 4)
                    const unsigned byte = (unsigned)(d >> 6) * SUBTILE + (unsigned)r * 128u +
                                          (((unsigned)((d & 63) >> 3) ^ (unsigned)(r & 7)) << 4) + (unsigned)(d & 7) * 2u;
                    *reinterpret_cast<unsigned*>(k_tile + byte) = kr;
                    *reinterpret_cast<unsigned*>(k_tile + C::TILE + byte) = vr;
                    if (has_page) {
                        *reinterpret_cast<unsigned*>(k_pages + off + d) = kr;
                        *reinterpret_cast<unsigned*>(v_pages + off + d) = vr;
                    }
                }
                __syncwarp();
            }
            float s[NT][4];
#pragma unroll
            for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const unsigned chunk = (unsigned)((kk & 3) * 2) + k_half;
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {                    // 16 keys per ldmatrix.x4
                    unsigned b[4];
                    ldmatrix_x4_addr(b, kt + (kk >> 2) * SUBTILE + k_row + np * 16 * 128 + ((chunk ^ (unsigned)rr) << 4));
                    mma_bf16(s[2 * np], q[kk], b[0], b[1]);
                    mma_bf16(s[2 * np + 1], q[kk], b[2], b[3]);
                }
            }
            unsigned pfrag[NT / 2][4];
            softmax_block<HD, NT>(s, pfrag, o, m_run, l_run, scale2, (t_begin + j) * KEYS + warp * WKEYS, vis_lo, vis_hi, lane);
#pragma unroll
            for (int kb = 0; kb < NT / 2; ++kb) {
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {
                    unsigned b[4];
                    const unsigned chunk = (unsigned)((dp & 3) * 2) + v_half;
                    ldmatrix_x4_trans_addr(b, vt + (dp >> 2) * SUBTILE + v_row + kb * 16 * 128 + ((chunk ^ (unsigned)rr) << 4));
                    mma_bf16(o[2 * dp], pfrag[kb], b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], pfrag[kb], b[2], b[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);            // this warp has read the stage
        }
    }
    __syncthreads();        // every tile is consumed (or the CTA failed): no copy is in flight any more
    if (s_failed || warp == WARPS) return;

    // merge the four warps through shared memory (no copy is in flight any more)
    constexpr int MS = HD + 4;                                    // padded row: conflict-free float2 stores
    float* sm_o = reinterpret_cast<float*>(smem);                 // [WARPS][16][MS]
    float* sm_ml = sm_o + WARPS * 16 * MS;                        // [WARPS][16][2]
    float* sm_f = sm_ml + WARPS * 16 * 2;                         // [WARPS][16] factors
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
#pragma unroll
        for (int d = 0; d < HD / 8; ++d)
            *reinterpret_cast<float2*>(&sm_o[(warp * 16 + row) * MS + d * 8 + 2 * t]) = make_float2(o[d][2 * r], o[d][2 * r + 1]);
        if (t == 0) {
            sm_ml[(warp * 16 + row) * 2] = m_run[r];
            sm_ml[(warp * 16 + row) * 2 + 1] = l_run[r];
        }
    }
    __syncthreads();
    float m_row = -INFINITY, l_row = 0.f;
    if (tid < n_rep) {
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m_row = fmaxf(m_row, sm_ml[(w * 16 + tid) * 2]);
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float mw = sm_ml[(w * 16 + tid) * 2];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m_row);
            l_row += sm_ml[(w * 16 + tid) * 2 + 1] * f;
            sm_f[w * 16 + tid] = f;
        }
        if (splits > 1) {
            const size_t slot = ((size_t)token * heads + kvh * n_rep + tid) * splits + split;
            part_ml[slot * 2] = m_row;
            part_ml[slot * 2 + 1] = l_row;
        } else {
            sm_ml[tid * 2 + 1] = l_row;                         // warp 0's slot of the row: the total for the division below
        }
    }
    __syncthreads();
    for (int i = tid; i < n_rep * HD; i += WARPS * 32) {
        const int row = i / HD, d = i - row * HD;
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) acc += sm_o[(w * 16 + row) * MS + d] * sm_f[w * 16 + row];
        const size_t th = (size_t)token * heads + kvh * n_rep + row;
        if (splits == 1) {
            const float l = sm_ml[row * 2 + 1];
            out[th * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else {
            part_o[(th * splits + split) * HD + d] = acc;
        }
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

// Map over the pool: (head dim, slot in page, page * kv_heads + kv head); a box is 64 elements of one page of one kv head.
int make_pool_map(CUtensorMap* map, const void* ptr, int head_dim, int page_size, long long planes) {
    EncodeTiledFn enc = get_encode();
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

template <int HD, bool FUSED>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const void* qkv, int q_stride, void* out, const int* ctx_lens,
           const int* block_table, int bt_stride, int page_size, int num_pages, int n_tokens, int heads, int kv_heads,
           float scale, int window, int splits, float* part_o, float* part_ml, void* k_pages, void* v_pages,
           const float* cos_t, const float* sin_t, int rot, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(attention_decode_tma_kernel<HD, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<HD>::SMEM));
        configured = true;
    }
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    NIB_CUDA(launch_pdl(attention_decode_tma_kernel<HD, FUSED>, dim3(splits, n_tokens, kv_heads), dim3(THREADS), (size_t)Cfg<HD>::SMEM,
                        stream, mk, mv, (const __nv_bfloat16*)qkv, q_stride, (__nv_bfloat16*)out, ctx_lens, block_table,
                        bt_stride, page_size, shift, num_pages, heads, kv_heads, heads / kv_heads, scale, window, splits,
                        part_o, part_ml, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, cos_t, sin_t, rot));
    if (splits > 1) return nib_attention_combine(part_o, part_ml, out, n_tokens * heads, splits, HD, stream);
    return 0;
}

}  // namespace

// 1 if the TMA decode kernel takes this shape: head size 64 or 128, at most 16 query heads per kv head,
// pages of 8, 16, 32 or 64 tokens.
NIB_API int nib_attention_decode_tma_supported(int heads, int kv_heads, int head_dim, int page_size) {
    if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > 16) return 0;
    if (head_dim != 64 && head_dim != 128) return 0;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return 0;
    return get_encode() != nullptr;
}

// The error word of the kernel's bounded waits (0 = none); synchronises with the device and clears it.
NIB_API int nib_attention_decode_tma_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_dec_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_dec_error, &zero, sizeof(int));
    return v;
}

namespace {
int decode_tma(const void* qkv, int q_stride, void* out, const int* ctx_lens, const int* block_table, int bt_stride,
               int page_size, void* k_pages, void* v_pages, int num_pages, int n_tokens, int heads, int kv_heads,
               int head_dim, float scale, int window, int splits, float* part_o, float* part_ml, bool fused,
               const float* cos_t, const float* sin_t, int rot, cudaStream_t stream) {
    NIB_REQUIRE(nib_attention_decode_tma_supported(heads, kv_heads, head_dim, page_size),
                "attention decode (TMA): head_dim %d, %d/%d heads, page size %d are not supported", head_dim, heads, kv_heads, page_size);
    NIB_REQUIRE(n_tokens >= 0 && num_pages > 0 && window >= 0 && splits >= 1 && splits <= 64, "attention decode (TMA): bad sizes (1..64 splits)");
    NIB_REQUIRE(splits == 1 || (part_o && part_ml), "attention decode (TMA): splits > 1 need scratch memory");
    NIB_REQUIRE(n_tokens <= 65535 && kv_heads <= 65535, "attention decode (TMA): too many tokens or kv heads for one launch");
    NIB_REQUIRE((((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0 && q_stride % 2 == 0, "attention decode (TMA): the pools must be 16-byte aligned, rows 4-byte aligned");
    NIB_REQUIRE((long long)num_pages * kv_heads < (1LL << 31) - 1, "attention decode (TMA): too many pages");
    NIB_REQUIRE(!fused || (rot >= 0 && rot <= head_dim && rot % 4 == 0 && (rot == 0 || (cos_t && sin_t))),
                "attention decode (TMA, fused): rotated width %d must be a multiple of 4 and at most head_dim", rot);
    if (n_tokens == 0) return 0;
    CUtensorMap mk, mv;
    const long long planes = (long long)num_pages * kv_heads;
    if (make_pool_map(&mk, k_pages, head_dim, page_size, planes)) return 1;
    if (make_pool_map(&mv, v_pages, head_dim, page_size, planes)) return 1;
#define CALL(HD, F) launch<HD, F>(mk, mv, qkv, q_stride, out, ctx_lens, block_table, bt_stride, page_size, num_pages, n_tokens, heads, \
                                  kv_heads, scale, window, splits, part_o, part_ml, k_pages, v_pages, cos_t, sin_t, rot, stream)
    if (fused) return head_dim == 64 ? CALL(64, true) : CALL(128, true);
    return head_dim == 64 ? CALL(64, false) : CALL(128, false);
#undef CALL
}
}  // namespace

// Arguments as nib_attention_decode_mma (without counters: the splits are merged by the combine kernel).
NIB_API int nib_attention_decode_tma(const void* qkv, int q_stride, void* out, const int* ctx_lens,
                                     const int* block_table, int bt_stride, int page_size, const void* k_pages,
                                     const void* v_pages, int num_pages, int n_tokens, int heads, int kv_heads,
                                     int head_dim, float scale, int window, int splits, float* part_o, float* part_ml,
                                     cudaStream_t stream) {
    return decode_tma(qkv, q_stride, out, ctx_lens, block_table, bt_stride, page_size, const_cast<void*>(k_pages),
                      const_cast<void*>(v_pages), num_pages, n_tokens, heads, kv_heads, head_dim, scale, window, splits, part_o,
                      part_ml, false, nullptr, nullptr, 0, stream);
}

// The same fused with what precedes it in a decode step: qkv is the raw projection; queries and the new key
// are rotated with the tables' row of the token's position (ctx_len - 1), the new key and value are written
// into the token's page and used at once. Arguments as nib_attention_decode_fused_mma.
NIB_API int nib_attention_decode_tma_fused(const void* qkv, int q_stride, void* out, const int* ctx_lens,
                                           const int* block_table, int bt_stride, int page_size, void* k_pages,
                                           void* v_pages, int num_pages, int n_tokens, int heads, int kv_heads,
                                           int head_dim, float scale, int window, int splits, float* part_o,
                                           float* part_ml, const float* cos_t, const float* sin_t, int rot,
                                           cudaStream_t stream) {
    return decode_tma(qkv, q_stride, out, ctx_lens, block_table, bt_stride, page_size, k_pages, v_pages, num_pages, n_tokens,
                      heads, kv_heads, head_dim, scale, window, splits, part_o, part_ml, true, cos_t, sin_t, rot, stream);
}
