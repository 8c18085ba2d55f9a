// Building blocks that the mma.sync attention kernels share: fragment loads, the tensor-core
// instruction, and the online-softmax update of a warp's 16 rows (32-bit, base-2 exponentials).
#pragma once
#include "common.cuh"

namespace {

constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// the same with a shared-memory address already in the 32-bit shared window
__device__ __forceinline__ void ldmatrix_x4_addr(unsigned (&r)[4], unsigned s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans_addr(unsigned (&r)[4], unsigned s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Transposes an 8 x 8 matrix of 16-bit elements that a warp holds in the fragment layout (thread (g, t): row g, columns
// 2t and 2t+1): afterwards the thread holds row g, columns 2t and 2t+1 of the transposed matrix.
__device__ __forceinline__ unsigned movmatrix_trans(unsigned v) {
    unsigned r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Online-softmax update of one warp's 16 rows with a block of NT*8 score columns.
// s holds raw dots; scale2 = scale * log2(e). vis_lo/vis_hi: visible key range of the thread's two
// rows (row g -> [0], row g+8 -> [1]); key_base: key of column 0. Produces P as A fragments.
template <int HD, int NT>
__device__ __forceinline__ void softmax_block(float (&s)[NT][4], unsigned (&p)[NT / 2][4], float (&o)[HD / 8][4],
                                              float (&m_run)[2], float (&l_run)[2], float scale2, int key_base,
                                              const int (&vis_lo)[2], const int (&vis_hi)[2], int lane) {
    const int t = lane & 3;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const int key = key_base + n * 8 + 2 * t + (e & 1);
            const bool vis = key >= vis_lo[r] && key <= vis_hi[r];
            s[n][e] = vis ? s[n][e] * scale2 : -INFINITY;
            mx[r] = fmaxf(mx[r], s[n][e]);
        }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;         // nothing visible yet: exp2(-inf - 0) = 0
        corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float pv = exp2f(s[n][e] - m_use[e >> 1]);
            s[n][e] = pv;
            sum[e >> 1] += pv;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        l_run[r] = l_run[r] * corr[r] + sum[r];
    }
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
        o[d][0] *= corr[0]; o[d][1] *= corr[0];
        o[d][2] *= corr[1]; o[d][3] *= corr[1];
    }
#pragma unroll
    for (int kb = 0; kb < NT / 2; ++kb) {
        p[kb][0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
        p[kb][1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
        p[kb][2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
        p[kb][3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
    }
}

// A fragments of 16 query rows straight from global memory. row_ptr[r]: start of the head's HD elements
// for the thread's row g (r=0) and g+8 (r=1), or nullptr for a row that does not exist.
template <int HD>
__device__ __forceinline__ void load_q(unsigned (&q)[HD / 16][4], const __nv_bfloat16* const (&row_ptr)[2], int lane) {
    const int t = lane & 3;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            unsigned lo = 0u, hi = 0u;
            if (row_ptr[r]) {
                lo = *reinterpret_cast<const unsigned*>(row_ptr[r] + kk * 16 + 2 * t);
                hi = *reinterpret_cast<const unsigned*>(row_ptr[r] + kk * 16 + 8 + 2 * t);
            }
            q[kk][r] = lo;        // a0 (row g) / a1 (row g+8): dims 2t, 2t+1
            q[kk][2 + r] = hi;    // a2 / a3: dims 8+2t, 9+2t
        }
    }
}

}  // namespace
