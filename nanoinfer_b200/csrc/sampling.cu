// Choosing the next token on the device from 32-bit logits [rows, vocab].
//
// Pipeline, in the reference's order (nanoinfer/sampling.py:126-151, cpp/src/sampling.cpp:90-108):
// repetition penalty on the raw logits -> greedy (first index of the maximum) when temperature is 0
// -> logits / temperature -> top-k (ties at the k-th value stay) -> top-p (a token is dropped iff the
// probability of those before it, in descending order, exceeds p; the first stays) -> softmax ->
// draw. The draw is an inverse CDF in vocabulary order with a uniform number that the host derives
// from (seed, number of tokens generated), so a request's tokens do not depend on the batch it
// was sampled in. The reference samples on the host (cpp/python/ni/scheduler.py:89-147).
#include "pipeline.cuh"

// ---------------------------------------------------------------------------------- penalty
// seen: flat list of distinct token ids per row, seen_start[row]..seen_start[row+1]. pending (may be null): one more id
// per row that is still on the device (the token of a step whose result the host has not read yet); it is penalised
// too unless the row's list holds it already, so no logit is penalised twice.
__global__ void penalty_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ seen,
                               const int* __restrict__ seen_start, const float* __restrict__ penalty,
                               const int* __restrict__ pending) {
    __shared__ int listed;
    const int row = blockIdx.x;
    const float p = penalty[row];
    if (p == 1.0f) return;
    const int extra = pending ? pending[row] : -1;
    if (threadIdx.x == 0) listed = 0;
    __syncthreads();
    float* l = logits + (size_t)row * vocab;
    for (int i = seen_start[row] + threadIdx.x; i < seen_start[row + 1]; i += blockDim.x) {
        const int id = seen[i];
        if (id < 0 || id >= vocab) continue;
        if (id == extra) listed = 1;
        const float s = l[id];
        l[id] = s > 0.f ? s / p : s * p;
    }
    __syncthreads();
    if (threadIdx.x == 0 && extra >= 0 && extra < vocab && !listed) {
        const float s = l[extra];
        l[extra] = s > 0.f ? s / p : s * p;
    }
}

NIB_API int nib_repetition_penalty(float* logits, int rows, int vocab, const int* seen, const int* seen_start,
                                   const float* penalty, const int* pending, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && vocab > 0, "penalty: bad sizes");
    if (rows == 0) return 0;
    penalty_kernel<<<rows, 256, 0, stream>>>(logits, vocab, seen, seen_start, penalty, pending);
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

// ---- the sampling kernel: a cluster of CS CTAs per row. One SM working through a row of 152K logits a dozen times was
// the whole cost (0.1 to 2 ms for eight rows); with the row cut into CS slices every pass is CS times shorter, and what
// the CTAs have to tell each other (maxima, sums, histograms, the radix digit chosen) goes through distributed shared
// memory between cluster barriers. Everything that decides a token is either an integer sum (histograms of counts
// and of fixed-point masses: any order gives the same) or a float sum in a fixed order (threads, warps, lanes and CTAs
// in ascending order), so a row's token depends on the row alone.
constexpr int ST = 256;      // threads of a CTA
constexpr int CS = 8;        // CTAs of the cluster that shares a row

__device__ __forceinline__ unsigned ld_peer_u32(unsigned addr) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];\n" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_peer_u64(unsigned addr) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];\n" : "=l"(v) : "r"(addr) : "memory");
    return v;
}

// f(x) for every scaled logit x = l[i] / temperature of the CTA's slice [begin, end) of a row, in no particular order:
// 16-byte loads, two of them in flight per thread, where the slice allows (a thread with one 4-byte load in flight waits
// out the whole latency of the memory system for every element). begin is a multiple of 4.
template <typename F>
__device__ __forceinline__ void for_each_scaled(const float* __restrict__ l, int begin, int end, float inv_t, F&& f) {
    const int tid = threadIdx.x;
    int done = begin;
    if ((reinterpret_cast<uintptr_t>(l) & 15) == 0) {
        const float4* l4 = reinterpret_cast<const float4*>(l + begin);
        const int n4 = (end - begin) >> 2;
        int i = tid;
        for (; i + ST < n4; i += 2 * ST) {
            const float4 a = l4[i], b = l4[i + ST];
            f(a.x * inv_t); f(a.y * inv_t); f(a.z * inv_t); f(a.w * inv_t);
            f(b.x * inv_t); f(b.y * inv_t); f(b.z * inv_t); f(b.w * inv_t);
        }
        if (i < n4) {
            const float4 a = l4[i];
            f(a.x * inv_t); f(a.y * inv_t); f(a.z * inv_t); f(a.w * inv_t);
        }
        done = begin + 4 * n4;
    }
    for (int i = done + tid; i < end; i += ST) f(l[i] * inv_t);
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
// fast exponential (2 ulp) is plenty for a draw.
__device__ __forceinline__ float weight(float d) { return __expf(d); }

// temperature > 0 for every row given to this kernel. grid: CS CTAs (one cluster) per row.
__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out) {
    using namespace nibp;
    __shared__ float scratch[ST / 32];
    __shared__ unsigned hist[256];                  // this CTA's histogram of a radix pass
    // ... and its masses as three histograms of 14-bit chunks: mass = m0 + m1 * 2^14 + m2 * 2^28
    __shared__ unsigned mass3[3][256];
    __shared__ unsigned tot_hist[256];              // CTA 0: the cluster's sums
    __shared__ unsigned long long tot_mass[256];
    __shared__ unsigned dec_prefix, dec_remaining;  // CTA 0: what a radix pass decided, read by every CTA
    __shared__ unsigned long long dec_above;
    __shared__ float x_max, x_z, x_total;           // what this CTA tells the others
    __shared__ int x_ties;
    __shared__ float chunk_sum[ST];
    __shared__ int tie_count[ST];
    __shared__ float lane_total[32];
    __shared__ int s_pick;

    const int row = blockIdx.x / CS;
    const unsigned rank = cluster_rank();
    const float* l = logits + (size_t)row * vocab;
    const float inv_t = 1.0f / temperature[row];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // a thread's chunk of the row (vocabulary order: rank, then thread), a multiple of 4 long so that chunks start on 16 bytes
    const int per = ((vocab + CS * ST - 1) / (CS * ST) + 3) & ~3;
    const int begin = min(vocab, ((int)rank * ST + tid) * per), end = min(vocab, begin + per);
    const int s_begin = min(vocab, (int)rank * ST * per), s_end = min(vocab, s_begin + ST * per);

    auto cta_reduce = [&](float v, bool is_max) -> float {      // over the CTA, in a fixed order
        v = is_max ? warp_max(v) : warp_sum(v);
        if (lane == 0) scratch[warp] = v;
        __syncthreads();
        float r = scratch[0];
        for (int i = 1; i < ST / 32; ++i) r = is_max ? fmaxf(r, scratch[i]) : r + scratch[i];
        __syncthreads();
        return r;
    };

    // ---- the row's maximum
    float mx = -INFINITY;
    for_each_scaled(l, s_begin, s_end, inv_t, [&](float x) { mx = fmaxf(mx, x); });
    mx = cta_reduce(mx, true);
    if (tid == 0) x_max = mx;
    cluster_sync();
    for (unsigned r = 0; r < CS; ++r) mx = fmaxf(mx, ld_peer_f32(peer_smem(&x_max, r)));

    // One radix pass over the slice: histogram (and masses), summed over the cluster by CTA 0, whose thread 0 then
    // chooses the digit (``choose``) and leaves the decision where every CTA reads it after the second barrier.
    auto radix_pass = [&](bool with_mass, auto&& add, auto&& choose) {
        for (int b = tid; b < 256; b += ST) { hist[b] = 0u; mass3[0][b] = mass3[1][b] = mass3[2][b] = 0u; }
        __syncthreads();
        for_each_scaled(l, s_begin, s_end, inv_t, add);
        __syncthreads();
        cluster_sync();
        if (rank == 0) {
            for (int b = tid; b < 256; b += ST) {
                unsigned n = 0u;
                unsigned long long m = 0ull;
                for (unsigned r = 0; r < CS; ++r) {
                    n += ld_peer_u32(peer_smem(&hist[b], r));
                    if (with_mass)
                        m += (unsigned long long)ld_peer_u32(peer_smem(&mass3[0][b], r)) +
                             ((unsigned long long)ld_peer_u32(peer_smem(&mass3[1][b], r)) << 14) +
                             ((unsigned long long)ld_peer_u32(peer_smem(&mass3[2][b], r)) << 28);
                }
                tot_hist[b] = n;
                tot_mass[b] = m;
            }
            __syncthreads();
            if (tid < 32) choose();          // warp 0: lane j looks at the bins 8j..8j+7
        }
        cluster_sync();
    };

    // ---- top-k: key of the k-th largest scaled logit (0 keeps everything)
    unsigned kth_key = 0u;
    const int k = top_k[row];
    if (k > 0 && k < vocab) {
        unsigned prefix = 0u, remaining = (unsigned)k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            radix_pass(false,
                       [&](float x) {
                           const unsigned key = key_of(x);
                           if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
                       },
                       [&]() {
                           // the highest bin b >= 1 with (elements in bins >= b) >= remaining, else bin 0; what is still to
                           // find inside it: remaining - (elements in the bins above b)
                           unsigned mine = 0u;
                           for (int i = 0; i < 8; ++i) mine += tot_hist[lane * 8 + i];
                           unsigned above = mine;                       // inclusive sum over this lane and the lanes above
#pragma unroll
                           for (int o = 1; o < 32; o <<= 1) {
                               const unsigned v = __shfl_down_sync(0xffffffffu, above, o);
                               if (lane + o < 32) above += v;
                           }
                           above -= mine;                               // elements in the bins above this lane's
                           int found = -1;
                           unsigned rem_found = 0u, run = above;
                           for (int i = 7; i >= 0; --i) {
                               const int b = lane * 8 + i;
                               if (found < 0 && b > 0 && run + tot_hist[b] >= remaining) { found = b; rem_found = remaining - run; }
                               run += tot_hist[b];
                           }
                           const unsigned has = __ballot_sync(0xffffffffu, found >= 0);
                           const int top = has ? 31 - __clz(has) : 0;   // the highest lane that found one holds the highest bin
                           const int b = __shfl_sync(0xffffffffu, found, top);
                           const unsigned r = __shfl_sync(0xffffffffu, rem_found, top);
                           const unsigned all = __shfl_sync(0xffffffffu, above + mine, 0);       // every element that matched
                           if (lane == 0) {
                               dec_prefix = prefix | ((unsigned)(has ? b : 0) << shift);
                               dec_remaining = has ? r : remaining - (all - tot_hist[0]);
                           }
                       });
            prefix = ld_peer_u32(peer_smem(&dec_prefix, 0));
            remaining = ld_peer_u32(peer_smem(&dec_remaining, 0));
        }
        kth_key = prefix;
    }

    // ---- normaliser over what top-k kept: threads, warps, CTAs in ascending order
    float z = 0.f;
    for_each_scaled(l, s_begin, s_end, inv_t, [&](float x) {
        if (key_of(x) >= kth_key) z += weight(x - mx);
    });
    z = cta_reduce(z, false);
    if (tid == 0) x_z = z;
    cluster_sync();
    z = 0.f;
    for (unsigned r = 0; r < CS; ++r) z += ld_peer_f32(peer_smem(&x_z, r));
    const float fix_over_z = FIX_ONE / z;

    // ---- top-p: smallest key whose "probability of strictly larger keys" is <= p
    unsigned p_key = kth_key;
    long long ties_kept = -1;  // -1: every element equal to p_key stays
    const float tp = top_p[row];
    if (tp < 1.0f) {
        const unsigned long long limit = (unsigned long long)((double)tp * (double)FIX_ONE);
        unsigned prefix = 0u;
        unsigned long long above0 = 0ull;
        for (int shift = 24; shift >= 0; shift -= 8) {
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            radix_pass(true,
                       [&](float x) {
                           const unsigned key = key_of(x);
                           if (key >= kth_key && (key & mask) == prefix) {
                               mass_add(mass3, (key >> shift) & 255u, (unsigned long long)(weight(x - mx) * fix_over_z));
                               atomicAdd(&hist[(key >> shift) & 255u], 1u);
                           }
                       },
                       [&]() {
                           // the lowest non-empty bin whose "mass above" (the bins above it, and what earlier passes left
                           // above) is still within the limit; the very first (largest) element always stays, so if even
                           // the highest non-empty bin is past the limit, that one
                           unsigned long long mine = 0ull;
                           for (int i = 0; i < 8; ++i) mine += tot_mass[lane * 8 + i];
                           unsigned long long above = mine;
#pragma unroll
                           for (int o = 1; o < 32; o <<= 1) {
                               const unsigned long long v = __shfl_down_sync(0xffffffffu, above, o);
                               if (lane + o < 32) above += v;
                           }
                           above = above - mine + above0;               // mass above this lane's bins
                           int low = -1, high = -1;
                           unsigned long long low_above = 0ull, high_above = 0ull, run = above;
                           for (int i = 7; i >= 0; --i) {
                               const int b = lane * 8 + i;
                               if (tot_hist[b] != 0u) {
                                   if (high < 0) { high = b; high_above = run; }
                                   if (run <= limit) { low = b; low_above = run; }
                               }
                               run += tot_mass[b];
                           }
                           const unsigned within = __ballot_sync(0xffffffffu, low >= 0), any = __ballot_sync(0xffffffffu, high >= 0);
                           int chosen = 0;
                           unsigned long long chosen_above = above0;
                           if (within) {                                // the lowest lane with one holds the lowest such bin
                               const int src = __ffs(within) - 1;
                               chosen = __shfl_sync(0xffffffffu, low, src);
                               chosen_above = __shfl_sync(0xffffffffu, low_above, src);
                           } else if (any) {
                               const int src = 31 - __clz(any);
                               chosen = __shfl_sync(0xffffffffu, high, src);
                               chosen_above = __shfl_sync(0xffffffffu, high_above, src);
                           }
                           if (lane == 0) {
                               dec_prefix = prefix | ((unsigned)chosen << shift);
                               dec_above = chosen_above;
                           }
                       });
            prefix = ld_peer_u32(peer_smem(&dec_prefix, 0));
            above0 = ld_peer_u64(peer_smem(&dec_above, 0));
        }
        p_key = prefix;
        if (p_key < kth_key) p_key = kth_key;
        // ties at p_key: the r-th of them (in vocabulary order) stays iff above + r*q <= limit
        const float xv = float_of_key(p_key);
        const unsigned long long q = (unsigned long long)(weight(xv - mx) * fix_over_z);
        if (q > 0ull && above0 <= limit) ties_kept = (long long)((limit - above0) / q) + 1;
        else ties_kept = 1;
    }

    // ---- inverse CDF in vocabulary order over what is kept
    // rank of the ties before this thread's chunk: the CTAs before this one, then the threads before it (lane j of warp
    // 0 takes the chunks 8j..8j+7; integers, so any order gives the same)
    long long tie_rank = 0;
    if (ties_kept >= 0) {
        int my_ties = 0;
        for_chunk(l, begin, end, inv_t, [&](int, float x) { my_ties += key_of(x) == p_key; return true; });
        tie_count[tid] = my_ties;
        __syncthreads();
        if (tid < 32) {
            constexpr int G = ST / 32;
            int mine = 0;
            for (int t = 0; t < G; ++t) mine += tie_count[tid * G + t];
            int before = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, before, o);
                if (tid >= o) before += v;
            }
            if (tid == 31) x_ties = before;
            int run = before - mine;
            for (int t = 0; t < G; ++t) { const int c = tie_count[tid * G + t]; tie_count[tid * G + t] = run; run += c; }
        }
        __syncthreads();
        cluster_sync();
        tie_rank = tie_count[tid];
        for (unsigned r = 0; r < rank; ++r) tie_rank += (int)ld_peer_u32(peer_smem(&x_ties, r));
    }
    float csum = 0.f;
    {
        long long tr = tie_rank;
        for_chunk(l, begin, end, inv_t, [&](int, float x) {
            const unsigned key = key_of(x);
            bool keep = key >= p_key;
            if (keep && ties_kept >= 0 && key == p_key) keep = (tr++) < ties_kept;
            if (keep) csum += weight(x - mx);
            return true;
        });
    }
    chunk_sum[tid] = csum;
    __syncthreads();
    // The sums in a fixed order, in three levels: lane j of warp 0 adds the sums of the CTA's chunks 8j..8j+7 in order and
    // the 32 lane totals in order; the CTAs' totals are added in rank order. The CTA whose chunks hold the drawn point
    // of the row's mass finds the lane, the lane its chunk, the chunk's thread the element.
    constexpr int G = ST / 32;
    if (tid < 32) {
        float mine = 0.f;
        for (int t = 0; t < G; ++t) mine += chunk_sum[tid * G + t];
        lane_total[tid] = mine;
        __syncwarp();
        if (tid == 0) {
            float total = 0.f;
            for (int j = 0; j < 32; ++j) total += lane_total[j];
            x_total = total;
        }
    }
    __syncthreads();
    cluster_sync();
    float cta_total[CS], total = 0.f;
    for (unsigned r = 0; r < CS; ++r) { cta_total[r] = ld_peer_f32(peer_smem(&x_total, r)); total += cta_total[r]; }
    const float target = uniform[row] * total;
    // which CTA: the first whose totals reach past the target; if rounding runs past the end, the last with mass
    int cta_pick = -1, last_cta = CS - 1;
    float cta_before = 0.f;
    {
        float run = 0.f;
        for (int r = 0; r < CS; ++r) {
            if (cta_total[r] > 0.f) last_cta = r;
            if (cta_pick < 0 && run + cta_total[r] > target && cta_total[r] > 0.f) { cta_pick = r; cta_before = run; }
            if (cta_pick < 0) run += cta_total[r];
        }
        if (cta_pick < 0) {
            cta_pick = last_cta;
            cta_before = 0.f;
            for (int r = 0; r < cta_pick; ++r) cta_before += cta_total[r];
        }
    }
    if ((int)rank == cta_pick) {
        if (tid < 32) {
            float run = cta_before;
            int lane_pick = -1, last_lane = 31;
            for (int j = 0; j < 32; ++j) {
                if (lane_total[j] > 0.f) last_lane = j;
                if (lane_pick < 0 && run + lane_total[j] > target && lane_total[j] > 0.f) lane_pick = j;
                if (lane_pick < 0) run += lane_total[j];
            }
            if (lane_pick < 0) {
                lane_pick = last_lane;
                run = cta_before;
                for (int j = 0; j < lane_pick; ++j) run += lane_total[j];
            }
            if (tid == lane_pick) {
                int pick = tid * G + G - 1;
                float before = run;
                bool found = false;
                for (int t = 0; t < G; ++t) {
                    const float c = chunk_sum[tid * G + t];
                    if (c > 0.f) pick = tid * G + t;
                    if (before + c > target && c > 0.f) { pick = tid * G + t; found = true; break; }
                    before += c;
                }
                if (!found) {
                    before = run;
                    for (int t = tid * G; t < pick; ++t) before += chunk_sum[t];
                }
                s_pick = pick;
                scratch[0] = before;
            }
        }
        __syncthreads();
        if (tid == s_pick) {
            float run = scratch[0];
            long long tr = tie_rank;
            int chosen = -1, last_kept = -1;
            for_chunk(l, begin, end, inv_t, [&](int i, float x) {
                const unsigned key = key_of(x);
                bool keep = key >= p_key;
                if (keep && ties_kept >= 0 && key == p_key) keep = (tr++) < ties_kept;
                if (!keep) return true;
                last_kept = i;
                run += weight(x - mx);
                if (run > target) { chosen = i; return false; }
                return true;
            });
            out[row] = chosen >= 0 ? chosen : (last_kept >= 0 ? last_kept : 0);
        }
    }
    cluster_sync();         // nobody leaves while a peer may still read its shared memory
}

NIB_API int nib_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                       const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes");
    if (rows == 0) return 0;
    NIB_REQUIRE((long long)vocab <= (1LL << 17) * 8, "sample: a row of %d logits is more than the fixed-point histograms hold", vocab);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * CS);
    cfg.blockDim = dim3(ST);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NIB_CUDA(cudaLaunchKernelEx(&cfg, sample_kernel, logits, vocab, temperature, top_k, top_p, uniform, out));
    NIB_LAUNCH_CHECK();
    return 0;
}
