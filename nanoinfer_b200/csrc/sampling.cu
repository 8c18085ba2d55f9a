// Choosing the next token on the device from 32-bit logits [rows, vocab].
//
// Pipeline, in the reference's order (nanoinfer/sampling.py:126-151, cpp/src/sampling.cpp:90-108):
// repetition penalty on the raw logits -> greedy (first index of the maximum) when temperature is 0
// -> logits / temperature -> top-k (ties at the k-th value stay) -> top-p (a token is dropped iff the
// probability of those before it, in descending order, exceeds p; the first stays) -> softmax ->
// draw. The draw is an inverse CDF in vocabulary order with a uniform number that the host derives
// from (seed, number of tokens generated), so a request's tokens do not depend on the batch it
// was sampled in. The reference samples on the host (cpp/python/ni/scheduler.py:89-147).
#include "common.cuh"

// ---------------------------------------------------------------------------------- penalty
// seen: flat list of distinct token ids per row, seen_start[row]..seen_start[row+1].
__global__ void penalty_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ seen,
                               const int* __restrict__ seen_start, const float* __restrict__ penalty) {
    const int row = blockIdx.x;
    const float p = penalty[row];
    if (p == 1.0f) return;
    float* l = logits + (size_t)row * vocab;
    for (int i = seen_start[row] + threadIdx.x; i < seen_start[row + 1]; i += blockDim.x) {
        const int id = seen[i];
        if (id < 0 || id >= vocab) continue;
        const float s = l[id];
        l[id] = s > 0.f ? s / p : s * p;
    }
}

NIB_API int nib_repetition_penalty(float* logits, int rows, int vocab, const int* seen, const int* seen_start,
                                   const float* penalty, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && vocab > 0, "penalty: bad sizes");
    if (rows == 0) return 0;
    penalty_kernel<<<rows, 256, 0, stream>>>(logits, vocab, seen, seen_start, penalty);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- argmax
constexpr int SAMP_THREADS = 1024;

__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// First index of the maximum of each row. NaN entries never win.
__global__ void __launch_bounds__(SAMP_THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
    __shared__ float sv[SAMP_THREADS / 32];
    __shared__ int si[SAMP_THREADS / 32];
    const float* l = logits + (size_t)blockIdx.x * vocab;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += SAMP_THREADS) argmax_combine(v, idx, l[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_combine(v, idx, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = v; si[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        v = sv[threadIdx.x];
        idx = si[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            argmax_combine(v, idx, ov, oi);
        }
        if (threadIdx.x == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

NIB_API int nib_argmax(const float* logits, int rows, int vocab, int* out, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && vocab > 0, "argmax: bad sizes");
    if (rows == 0) return 0;
    argmax_kernel<<<rows, SAMP_THREADS, 0, stream>>>(logits, vocab, out);
    NIB_LAUNCH_CHECK();
    return 0;
}

// The same with every row cut into `chunks` pieces that different CTAs scan: a few rows of a large
// vocabulary otherwise keep a few SMs busy and the rest idle. A piece's best (value, index) is packed
// into 64 bits (order-preserving bits of the value above the complement of the index), so the maximum
// of the packed words is the largest value at its first index, in whatever order they are compared. The
// CTA that finishes a row's last piece (a counter per row, left at zero) writes the result.
__device__ __forceinline__ unsigned long long argmax_pack(float x, int i) {
    if (x != x) return 0ull;                                   // NaN never wins
    const unsigned b = __float_as_uint(x);
    const unsigned key = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - (unsigned)i);
}

__global__ void __launch_bounds__(256)
argmax_chunk_kernel(const float* __restrict__ logits, int vocab, int chunk, int chunks, unsigned long long* __restrict__ part,
                    int* __restrict__ counters, int* __restrict__ out, unsigned long long* trace, int trace_cap) {
    __shared__ unsigned long long s_best[8];
    __shared__ int s_last;
    if (threadIdx.x == 0) nib_trace_mark(trace, trace_cap, NIB_TK_ARGMAX, 0, 1);
    const int row = blockIdx.y, cid = blockIdx.x;
    const float* l = logits + (size_t)row * vocab;
    const int begin = cid * chunk, end = min(vocab, begin + chunk);
    unsigned long long best = 0ull;
    for (int i = begin + threadIdx.x; i < end; i += 256) best = max(best, argmax_pack(l[i], i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0) s_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < 8; ++w) best = max(best, s_best[w]);
        part[(size_t)row * chunks + cid] = best;
        __threadfence();
        s_last = (atomicAdd(&counters[row], 1) == chunks - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    best = 0ull;
    for (int c = threadIdx.x; c < chunks; c += 256) best = max(best, __ldcg(part + (size_t)row * chunks + c));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0) s_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < 8; ++w) best = max(best, s_best[w]);
        out[row] = best == 0ull ? 0 : (int)(0xffffffffu - (unsigned)(best & 0xffffffffull));
        counters[row] = 0;                                      // ready for the next launch
    }
}

// scratch: rows * chunks 64-bit words; counters: rows ints that are zero between launches.
NIB_API int nib_argmax_chunked(const float* logits, int rows, int vocab, int* out, int chunks, unsigned long long* scratch,
                               int* counters, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && vocab > 0 && chunks >= 1 && chunks <= 65535 && rows <= 65535, "argmax: bad sizes");
    NIB_REQUIRE(scratch != nullptr && counters != nullptr, "argmax (chunked): scratch and counters are needed");
    if (rows == 0) return 0;
    const int chunk = ceil_div(vocab, chunks);
    argmax_chunk_kernel<<<dim3(chunks, rows), 256, 0, stream>>>(logits, vocab, chunk, chunks, scratch, counters, out, nib_trace_buffer(), nib_trace_capacity());
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- sampling
// Order-preserving map from float to unsigned: larger float <-> larger key.
__device__ __forceinline__ unsigned key_of(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float float_of_key(unsigned k) {
    const unsigned b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}

__device__ float block_max(float v, float* scratch) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = scratch[0];
    for (int i = 1; i < SAMP_THREADS / 32; ++i) r = fmaxf(r, scratch[i]);
    __syncthreads();
    return r;
}

// Sum over the block in a fixed order.
__device__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < SAMP_THREADS / 32; ++i) r += scratch[i];
    __syncthreads();
    return r;
}

// Scaled probabilities are histogrammed as 64-bit fixed point so that sums do not depend on the
// order in which threads add (integer addition is associative): sampling stays reproducible.
constexpr float FIX_ONE = 1099511627776.0f;  // 2^40

// A mass into the three histograms of 14-bit chunks. 64-bit adds to shared memory are loops of compare-and-swap, and
// the first radix pass (the key's top 8 bits: sign and exponent of the scaled logit) puts almost every element of a
// row into a handful of bins: a thousand threads queueing there with such loops made a pure top-p row cost two
// milliseconds. 32-bit adds to one address are combined by the hardware. A row's masses sum to 2^40, so every
// chunk's sum over up to 2^17 elements stays below 2^32.
__device__ __forceinline__ void mass_add(unsigned (*m)[256], unsigned bin, unsigned long long q) {
    const unsigned a = (unsigned)(q & 0x3fffull), b = (unsigned)((q >> 14) & 0x3fffull), c = (unsigned)(q >> 28);
    if (a) atomicAdd(&m[0][bin], a);
    if (b) atomicAdd(&m[1][bin], b);
    if (c) atomicAdd(&m[2][bin], c);
}

// f(x) for every scaled logit x = l[i] / temperature of a row, in no particular order: 16-byte loads, two of them in
// flight per thread, where the row allows (a thread with one 4-byte load in flight waits out the whole latency of the
// memory system for every element; a pass over 152K logits took 30 us that way). Rows that are not 16-byte aligned or
// whose length is no multiple of 4 are read element by element.
template <typename F>
__device__ __forceinline__ void for_each_scaled(const float* __restrict__ l, int vocab, float inv_t, F&& f) {
    const int tid = threadIdx.x;
    if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(l) & 15) == 0) {
        const float4* l4 = reinterpret_cast<const float4*>(l);
        const int n4 = vocab >> 2;
        int i = tid;
        for (; i + SAMP_THREADS < n4; i += 2 * SAMP_THREADS) {
            const float4 a = l4[i], b = l4[i + SAMP_THREADS];
            f(a.x * inv_t); f(a.y * inv_t); f(a.z * inv_t); f(a.w * inv_t);
            f(b.x * inv_t); f(b.y * inv_t); f(b.z * inv_t); f(b.w * inv_t);
        }
        if (i < n4) {
            const float4 a = l4[i];
            f(a.x * inv_t); f(a.y * inv_t); f(a.z * inv_t); f(a.w * inv_t);
        }
    } else {
        for (int i = tid; i < vocab; i += SAMP_THREADS) f(l[i] * inv_t);
    }
}

// f(i, x) for i = begin .. end - 1 in ascending order (a thread's chunk of a row), until f returns false. 16-byte loads,
// all of a group of 16 elements issued before the first is used, where begin is a multiple of 4 and the row is aligned.
template <typename F>
__device__ __forceinline__ void for_chunk(const float* __restrict__ l, int begin, int end, float inv_t, F&& f) {
    int i = begin;
    if ((begin & 3) == 0 && (reinterpret_cast<uintptr_t>(l) & 15) == 0) {
        for (; i + 16 <= end; i += 16) {
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = *reinterpret_cast<const float4*>(l + i + 4 * j);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (!f(i + 4 * j, v[j].x * inv_t)) return;
                if (!f(i + 4 * j + 1, v[j].y * inv_t)) return;
                if (!f(i + 4 * j + 2, v[j].z * inv_t)) return;
                if (!f(i + 4 * j + 3, v[j].w * inv_t)) return;
            }
        }
    }
    for (; i < end; ++i)
        if (!f(i, l[i] * inv_t)) return;
}

// The unnormalised probability of a scaled logit d = x - max <= 0, the same function wherever the kernel needs it. The
// fast exponential (2 ulp) is plenty for a draw: one SM works through a whole row, several times, and the accurate
// one tripled the instructions per element.
__device__ __forceinline__ float weight(float d) { return __expf(d); }

// One block per row. temperature > 0 for every row given to this kernel.
__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
    __shared__ float scratch[SAMP_THREADS / 32];
    __shared__ unsigned hist[256];
    // the masses of a radix pass as three histograms of 14-bit chunks (64-bit adds to shared memory are loops of
    // compare-and-swap; a chunk's sum over a row of up to 2^18 elements fits 32 bits): mass = m0 + m1 * 2^14 + m2 * 2^28
    __shared__ unsigned mass3[3][256];
    __shared__ unsigned s_prefix;
    __shared__ unsigned s_remaining;
    __shared__ unsigned long long s_above;
    __shared__ float chunk_sum[SAMP_THREADS];
    __shared__ int s_pick;

    const int row = blockIdx.x;
    const float* l = logits + (size_t)row * vocab;
    const float inv_t = 1.0f / temperature[row];
    const int tid = threadIdx.x;

    float mx = -INFINITY;
    for_each_scaled(l, vocab, inv_t, [&](float x) { mx = fmaxf(mx, x); });
    mx = block_max(mx, scratch);

    // ---- top-k: key of the k-th largest scaled logit (0 keeps everything)
    unsigned kth_key = 0u;
    int k = top_k[row];
    if (k > 0 && k < vocab) {
        if (tid == 0) { s_prefix = 0u; s_remaining = (unsigned)k; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += SAMP_THREADS) hist[b] = 0u;
            __syncthreads();
            const unsigned prefix = s_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for_each_scaled(l, vocab, inv_t, [&](float x) {
                const unsigned key = key_of(x);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
            });
            __syncthreads();
            if (tid == 0) {
                unsigned remaining = s_remaining;
                int b = 255;
                for (; b > 0; --b) {
                    if (hist[b] >= remaining) break;
                    remaining -= hist[b];
                }
                s_prefix = prefix | ((unsigned)b << shift);
                s_remaining = remaining;
            }
            __syncthreads();
        }
        kth_key = s_prefix;
    }

    // ---- normaliser over what top-k kept
    float z = 0.f;
    for_each_scaled(l, vocab, inv_t, [&](float x) {
        if (key_of(x) >= kth_key) z += weight(x - mx);
    });
    z = block_sum(z, scratch);
    const float fix_over_z = FIX_ONE / z;

    // ---- top-p: smallest key whose "probability of strictly larger keys" is <= p
    unsigned p_key = kth_key;
    long long ties_kept = -1;  // -1: every element equal to p_key stays
    const float tp = top_p[row];
    if (tp < 1.0f) {
        const unsigned long long limit = (unsigned long long)((double)tp * (double)FIX_ONE);
        if (tid == 0) { s_prefix = 0u; s_above = 0ull; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += SAMP_THREADS) { mass3[0][b] = mass3[1][b] = mass3[2][b] = 0u; hist[b] = 0u; }
            __syncthreads();
            const unsigned prefix = s_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for_each_scaled(l, vocab, inv_t, [&](float x) {
                const unsigned key = key_of(x);
                if (key >= kth_key && (key & mask) == prefix) {
                    mass_add(mass3, (key >> shift) & 255u, (unsigned long long)(weight(x - mx) * fix_over_z));
                    atomicAdd(&hist[(key >> shift) & 255u], 1u);
                }
            });
            __syncthreads();
            if (tid == 0) {
                // walk down from the largest bin; stay in the lowest non-empty bin whose
                // "mass above" is still within the limit
                unsigned long long above = s_above;
                int chosen = -1;
                unsigned long long chosen_above = above;
                for (int b = 255; b >= 0; --b) {
                    if (hist[b] == 0u) continue;
                    if (above <= limit || chosen < 0) {   // the very first (largest) element always stays
                        if (above <= limit || chosen < 0) { chosen = b; chosen_above = above; }
                    }
                    if (above > limit) break;
                    above += (unsigned long long)mass3[0][b] + ((unsigned long long)mass3[1][b] << 14) + ((unsigned long long)mass3[2][b] << 28);
                }
                s_prefix = prefix | ((unsigned)(chosen < 0 ? 0 : chosen) << shift);
                s_above = chosen_above;
            }
            __syncthreads();
        }
        p_key = s_prefix;
        if (p_key < kth_key) p_key = kth_key;
        // ties at p_key: the r-th of them (in vocabulary order) stays iff above + r*q <= limit
        const float xv = float_of_key(p_key);
        const unsigned long long q = (unsigned long long)(weight(xv - mx) * fix_over_z);
        const unsigned long long above = s_above;
        if (q > 0ull && above <= limit) ties_kept = (long long)((limit - above) / q) + 1;
        else ties_kept = 1;
    }

    // ---- inverse CDF in vocabulary order over what is kept
    const int per = ((vocab + SAMP_THREADS - 1) / SAMP_THREADS + 3) & ~3;       // a multiple of 4: chunks start on 16 bytes
    const int begin = min(vocab, tid * per), end = min(vocab, begin + per);
    // rank of ties before this thread's chunk
    __shared__ int tie_count[SAMP_THREADS];
    int my_ties = 0;
    if (ties_kept >= 0)
        for_chunk(l, begin, end, inv_t, [&](int, float x) { my_ties += key_of(x) == p_key; return true; });
    tie_count[tid] = my_ties;
    __syncthreads();
    if (ties_kept >= 0 && tid < 32) {   // exclusive scan by one warp: lane j takes chunks 32j..32j+31 (integers: any order)
        int mine = 0;
        for (int t = 0; t < 32; ++t) mine += tie_count[tid * 32 + t];
        int before = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, before, o);
            if (tid >= o) before += v;
        }
        int run = before - mine;
        for (int t = 0; t < 32; ++t) { const int c = tie_count[tid * 32 + t]; tie_count[tid * 32 + t] = run; run += c; }
    }
    __syncthreads();
    float csum = 0.f;
    {
        long long tie_rank = tie_count[tid];
        for_chunk(l, begin, end, inv_t, [&](int, float x) {
            const unsigned key = key_of(x);
            bool keep = key >= p_key;
            if (keep && ties_kept >= 0 && key == p_key) keep = (tie_rank++) < ties_kept;
            if (keep) csum += weight(x - mx);
            return true;
        });
    }
    chunk_sum[tid] = csum;
    __syncthreads();
    // Which chunk holds the drawn point of the row's mass. The order of the sums is fixed, in two levels, so that one
    // warp does in a hundred steps what one thread did in three thousand: lane j adds the sums of chunks 32j..32j+31 in
    // order; lane 0 adds the 32 lane totals in order and finds the lane whose chunks hold the target; that lane then
    // walks its 32 chunks.
    __shared__ float lane_total[32];
    if (tid < 32) {
        float mine = 0.f;
        for (int t = 0; t < 32; ++t) mine += chunk_sum[tid * 32 + t];
        lane_total[tid] = mine;
        __syncwarp();
        float total = 0.f;
        for (int j = 0; j < 32; ++j) total += lane_total[j];              // every lane: the same sum in the same order
        const float target = uniform[row] * total;
        float run = 0.f;
        int lane_pick = -1, last_lane = 31;
        for (int j = 0; j < 32; ++j) {
            if (lane_total[j] > 0.f) last_lane = j;                      // last lane with mass, if rounding runs past
            if (lane_pick < 0 && run + lane_total[j] > target && lane_total[j] > 0.f) lane_pick = j;
            if (lane_pick < 0) run += lane_total[j];
        }
        if (lane_pick < 0) {                                             // rounding ran past the end: the last chunk with mass
            lane_pick = last_lane;
            run = 0.f;
            for (int j = 0; j < lane_pick; ++j) run += lane_total[j];
        }
        if (tid == lane_pick) {
            int pick = tid * 32 + 31;
            float before = run;
            bool found = false;
            for (int t = 0; t < 32; ++t) {
                const float c = chunk_sum[tid * 32 + t];
                if (c > 0.f) pick = tid * 32 + t;                        // last chunk with mass so far
                if (before + c > target && c > 0.f) { pick = tid * 32 + t; found = true; break; }
                before += c;
            }
            if (!found) {                                                // take the last chunk with mass, and the mass before it
                before = run;
                for (int t = tid * 32; t < pick; ++t) before += chunk_sum[t];
            }
            s_pick = pick;
            scratch[0] = target;
            scratch[1] = before;
        }
    }
    __syncthreads();
    if (tid == s_pick) {
        const float target = scratch[0];
        float run = scratch[1];
        long long tie_rank = tie_count[tid];
        int chosen = -1, last_kept = -1;
        for_chunk(l, begin, end, inv_t, [&](int i, float x) {
            const unsigned key = key_of(x);
            bool keep = key >= p_key;
            if (keep && ties_kept >= 0 && key == p_key) keep = (tie_rank++) < ties_kept;
            if (!keep) return true;
            last_kept = i;
            run += weight(x - mx);
            if (run > target) { chosen = i; return false; }
            return true;
        });
        out[row] = chosen >= 0 ? chosen : (last_kept >= 0 ? last_kept : 0);
    }
}

NIB_API int nib_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                       const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes");
    if (rows == 0) return 0;
    sample_kernel<<<rows, SAMP_THREADS, 0, stream>>>(logits, vocab, temperature, top_k, top_p, uniform, out);
    NIB_LAUNCH_CHECK();
    return 0;
}
