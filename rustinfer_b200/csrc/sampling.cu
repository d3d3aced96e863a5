// Choosing the next token on the device: greedy argmax, and temperature sampling with
// top-k, min-p and top-p filters.
//
// Greedy follows crates/infer-backend-cuda/src/kernels/sampler/sampler.cu:66-105 (the
// lowest index wins ties).  The filtered draw follows RustInfer's host sampler
// (crates/infer-worker/src/application/sampler_stack.rs:242-351): logit/T, sort
// descending, top-k, exp(x - max), min-p, normalise, top-p (keep until the cumulative
// share reaches p, at least one), then walk the cumulative weights with draw * total.
// The reference copies the logits to the host for this and sorts the whole row.  Here one CTA
// per row never sorts the row: every quantity the filters need is a count or a sum of
// weights over a prefix of the sorted order, and the token that is drawn is the one where a
// running sum of weights crosses a target.  So the row is cut into 2,048 buckets by
// (max - logit) / T (a monotone function of the logit: buckets are in sorted order), one pass
// counts each bucket and sums its weights, a scan over the buckets finds the bucket in which a
// boundary lies (the k-th token, the cumulative share p, the drawn target), and only that
// bucket's few hundred tokens are gathered and sorted (64-bit keys made of the logit and the
// token id, so equal logits are ordered by ascending id).  Weights are exp in 32-bit and are
// summed as integers (w * 2^44), so a sum does not depend on the order in which threads add:
// the same row gives the same token whatever shares its batch.  A row whose boundary bucket
// holds more than 4,096 tokens (thousands of equal logits), or whose maximum is not finite,
// is left to the kernel that sorts the whole row (64-bit sums in rank order), which is kept
// for that.
#include "common.cuh"
#include <cooperative_groups.h>

namespace {

__device__ __forceinline__ unsigned int ordered_bits(float v) {
    if (v != v) v = -INFINITY;                           // NaN sorts last
    unsigned int u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_ordered(unsigned int k) {
    unsigned int u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(u);
}

// ------------------------------------------------------------------------- argmax
// grid (blocks per row, rows).  Every CTA reduces its slice of a row to a 64-bit key
// (ordered logit, ~index), merges it into state[row] with atomicMax, and the CTA that
// arrives last writes the token and puts state and counter back to zero, so the scratch
// is ready for the next call without a memset.  `state` and `count` start as zeros.
__global__ void __launch_bounds__(256)
argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out,
              unsigned long long* __restrict__ state, unsigned int* __restrict__ count) {
    pdl_trigger();
    pdl_wait();
    __shared__ unsigned long long best[8];
    const int row_id = blockIdx.y;
    const float* row = logits + (size_t)row_id * ld;
    unsigned long long mine = 0ull;                      // (ordered logit << 32) | ~index
    const int stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;
    if ((ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        const int n4 = vocab >> 2;                       // 16-byte loads over the aligned part of the row
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int i = first; i < n4; i += stride) {
            const float4 v = row4[i];
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const unsigned long long key = ((unsigned long long)ordered_bits(e[k]) << 32) |
                                               (unsigned int)(0xffffffffu - (unsigned int)(4 * i + k));
                mine = key > mine ? key : mine;
            }
        }
        for (int i = 4 * n4 + first; i < vocab; i += stride) {
            const unsigned long long key =
                ((unsigned long long)ordered_bits(row[i]) << 32) | (unsigned int)(0xffffffffu - (unsigned int)i);
            mine = key > mine ? key : mine;
        }
    } else {
        for (int i = first; i < vocab; i += stride) {
            const unsigned long long key =
                ((unsigned long long)ordered_bits(row[i]) << 32) | (unsigned int)(0xffffffffu - (unsigned int)i);
            mine = key > mine ? key : mine;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
        mine = other > mine ? other : mine;
    }
    if ((threadIdx.x & 31) == 0) best[threadIdx.x >> 5] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) mine = best[w] > mine ? best[w] : mine;
        atomicMax(&state[row_id], mine);
        __threadfence();
        const unsigned int ticket = atomicAdd(&count[row_id], 1u);
        if (ticket == gridDim.x - 1) {
            __threadfence();
            const unsigned long long top = atomicExch(&state[row_id], 0ull);
            out[row_id] = (int)(0xffffffffu - (unsigned int)(top & 0xffffffffu));
            count[row_id] = 0u;
        }
    }
}

// ---------------------------------------------------------------- filtered sampling
constexpr int ST = 1024;

// exp((logit - max) / T); a maximum of +inf leaves weight to the +inf logits alone, one of -inf (every
// logit -inf) gives every token the same weight
// (crates/infer-worker/src/application/sampler_stack.rs:277-285)
__device__ __forceinline__ double weight_of(unsigned long long key, float top, double inv_t) {
    const float v = from_ordered((unsigned int)(key >> 32));
    if (top == INFINITY) return v == INFINITY ? 1.0 : 0.0;
    if (top == -INFINITY) return 1.0;
    if (v == -INFINITY) return 0.0;
    return exp(((double)v - (double)top) * inv_t);
}

// Exclusive scan of one double per thread in thread order; returns this thread's prefix,
// *total gets the sum.  Serial over 1024 values: the order of additions is fixed.
__device__ double exclusive_scan(double v, double* buf, double* total) {
    __syncthreads();
    buf[threadIdx.x] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double run = 0.0;
        for (int i = 0; i < ST; ++i) { const double t = buf[i]; buf[i] = run; run += t; }
        buf[ST] = run;
    }
    __syncthreads();
    *total = buf[ST];
    return buf[threadIdx.x];
}

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, int vpad,
              unsigned long long* __restrict__ scratch, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const double* __restrict__ draw,
              int* __restrict__ out, const int* __restrict__ only_flagged) {
    pdl_trigger();
    pdl_wait();
    __shared__ double buf[ST + 1];
    __shared__ int found;
    const int r = blockIdx.x, tid = threadIdx.x;
    if (only_flagged && !only_flagged[r]) return;        // the bucketed kernel has chosen this row's token
    const float* row = logits + (size_t)r * ld;
    unsigned long long* s = scratch + (size_t)r * vpad;

    for (int i = tid; i < vpad; i += ST)
        s[i] = i < vocab ? (((unsigned long long)ordered_bits(row[i]) << 32) |
                            (unsigned int)(0xffffffffu - (unsigned int)i)) : 0ull;
    __syncthreads();
    for (int k = 2; k <= vpad; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < vpad; i += ST) {
                const int p = i ^ j;
                if (p > i) {
                    const unsigned long long a = s[i], b = s[p];
                    const bool desc = (i & k) == 0;
                    if (desc ? a < b : a > b) { s[i] = b; s[p] = a; }
                }
            }
            __syncthreads();
        }
    }
    const float temp = temperature[r];
    const int tk = top_k[r];
    const float tp = top_p[r], mp = min_p[r];
    if (!(temp > 0.f) || tk == 1 || !(tp > 0.f)) {       // greedy
        if (tid == 0) out[r] = (int)(0xffffffffu - (unsigned int)(s[0] & 0xffffffffu));
        return;
    }
    const double inv_t = 1.0 / (double)temp;
    const float top = from_ordered((unsigned int)(s[0] >> 32));
    int n = vocab;
    if (tk > 0 && tk < n) n = tk;
    int seg = (n + ST - 1) / ST;
    int lo = min(tid * seg, n), hi = min(lo + seg, n);

    // min-p: weights fall with rank, so the kept set is a prefix
    if (mp > 0.f) {
        if (tid == 0) found = n;
        __syncthreads();
        const double thr = (double)mp;                   // the largest weight is exp(0) = 1
        for (int i = lo; i < hi; ++i)
            if (weight_of(s[i], top, inv_t) < thr) { atomicMin(&found, i); break; }
        __syncthreads();
        n = max(found, 1);
        __syncthreads();
        seg = (n + ST - 1) / ST;
        lo = min(tid * seg, n); hi = min(lo + seg, n);
    }
    double part = 0.0, total = 0.0;
    for (int i = lo; i < hi; ++i) part += weight_of(s[i], top, inv_t);
    double prefix = exclusive_scan(part, buf, &total);

    if (tp < 1.f) {                                      // top-p
        if (tid == 0) found = n;
        __syncthreads();
        double cum = prefix;
        for (int i = lo; i < hi; ++i) {
            cum += weight_of(s[i], top, inv_t);
            if (cum / total >= (double)tp) { atomicMin(&found, i + 1); break; }
        }
        __syncthreads();
        n = max(found, 1);
        __syncthreads();
        seg = (n + ST - 1) / ST;
        lo = min(tid * seg, n); hi = min(lo + seg, n);
        part = 0.0;
        for (int i = lo; i < hi; ++i) part += weight_of(s[i], top, inv_t);
        prefix = exclusive_scan(part, buf, &total);
    }
    double u = draw[r];
    u = u < 0.0 ? 0.0 : (u > 1.0 - 2.220446049250313e-16 ? 1.0 - 2.220446049250313e-16 : u);
    const double target = u * total;
    if (tid == 0) found = n - 1;
    __syncthreads();
    double cum = prefix;
    for (int i = lo; i < hi; ++i) {
        cum += weight_of(s[i], top, inv_t);
        if (target < cum) { atomicMin(&found, i); break; }
    }
    __syncthreads();
    if (tid == 0) out[r] = (int)(0xffffffffu - (unsigned int)(s[found] & 0xffffffffu));
}
// ------------------------------------------------ filtered sampling without sorting the row
constexpr int SB = 2048;                 // buckets of (max - logit) / T
constexpr int CAP = 4096;                // most tokens of one bucket that are sorted in shared memory
constexpr int CL_MAX = 8;                // most CTAs of a cluster that share a row: each walks its part of it
constexpr float FIXED_ONE = 17592186044416.0f;            // 2^44: weights are summed as integers
constexpr size_t SELECT_SMEM = (SB + 1) * sizeof(unsigned long long) + 2 * (size_t)CAP * sizeof(unsigned long long) +
                               64 * sizeof(unsigned long long) + SB * sizeof(unsigned int);

__device__ __forceinline__ float clean(float v) { return v != v ? -INFINITY : v; }
// exp((logit - max) / T) in 32-bit (2^x on the special-function unit, relative error 2^-22)
__device__ __forceinline__ float weight32(float v, float top, float inv_t_log2e) {
    if (v == -INFINITY) return 0.f;
    float y;
    const float x = (v - top) * inv_t_log2e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned long long fixed_of(float w) { return (unsigned long long)(w * FIXED_ONE); }
__device__ __forceinline__ int bucket_of(float v, float top, float inv_t, float per_unit) {
    const float d = (top - v) * inv_t * per_unit;         // +inf for a logit of -inf: the last bucket
    return d >= (float)(SB - 1) ? SB - 1 : (int)d;
}

// f(index, logit) for the logits [begin, end) of a row, sixteen loads in flight per thread
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int begin, int end, F&& f) {
    const int tid = threadIdx.x;
    const float* base = row + begin;
    const int n = end - begin;
    if (n <= 0) return;
    if ((reinterpret_cast<uintptr_t>(base) & 15) == 0) {
        const float4* r4 = reinterpret_cast<const float4*>(base);
        const int n4 = n >> 2;
        int i = tid;
        for (; i + 3 * ST < n4; i += 4 * ST) {
            const float4 a = r4[i], b = r4[i + ST], c = r4[i + 2 * ST], d = r4[i + 3 * ST];
            const int ia = begin + 4 * i, ib = ia + 4 * ST, ic = ib + 4 * ST, id = ic + 4 * ST;
            f(ia, a.x); f(ia + 1, a.y); f(ia + 2, a.z); f(ia + 3, a.w);
            f(ib, b.x); f(ib + 1, b.y); f(ib + 2, b.z); f(ib + 3, b.w);
            f(ic, c.x); f(ic + 1, c.y); f(ic + 2, c.z); f(ic + 3, c.w);
            f(id, d.x); f(id + 1, d.y); f(id + 2, d.z); f(id + 3, d.w);
        }
        for (; i < n4; i += ST) {
            const float4 a = r4[i];
            const int ia = begin + 4 * i;
            f(ia, a.x); f(ia + 1, a.y); f(ia + 2, a.z); f(ia + 3, a.w);
        }
        for (int j = 4 * n4 + tid; j < n; j += ST) f(begin + j, base[j]);
    } else {
        for (int i = tid; i < n; i += ST) f(begin + i, base[i]);
    }
}

__device__ unsigned long long block_max_u64(unsigned long long v, unsigned long long* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { const unsigned long long t = __shfl_xor_sync(0xffffffffu, v, o); v = t > v ? t : v; }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        unsigned long long t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { const unsigned long long u = __shfl_xor_sync(0xffffffffu, t, o); t = u > t ? u : t; }
        if (threadIdx.x == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        unsigned long long t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// One cluster of 2, 4 or 8 CTAs per row (the launch decides: eight while all rows fit one wave of
// the GPU, fewer for many rows).  Every CTA walks its part of the row (largest logit, then
// counts and weights per bucket into its own shared memory); the first CTA of the cluster adds the
// histograms up through distributed shared memory, scans them and finds the bucket each
// boundary lies in; for such a bucket it tells the others, all gather the bucket's tokens from
// their part of the row into its list, and it sorts the list, sums it up and reads the boundary off.
__global__ void __launch_bounds__(ST)
sample_select_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
                     const int* __restrict__ top_k, const float* __restrict__ top_p,
                     const float* __restrict__ min_p, const double* __restrict__ draw,
                     int* __restrict__ out, int* __restrict__ flagged) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char select_smem[];
    unsigned long long* wsum = reinterpret_cast<unsigned long long*>(select_smem);      // [SB + 1] sums, then sums before a bucket
    unsigned long long* list = wsum + SB + 1;                                              // [CAP] keys of one bucket
    unsigned long long* cum = list + CAP;                                                  // [CAP] running weight over the sorted list
    unsigned long long* red = cum + CAP;                                                   // [64] reductions
    unsigned int* cnt = reinterpret_cast<unsigned int*>(red + 64);                         // [SB] counts, then counts before a bucket
    __shared__ unsigned long long x_best, x_low, x_nmp, x_wmp;     // this CTA's part, read by the others
    __shared__ int s_cmd, s_listed, s_found;
    const unsigned rank = cluster.block_rank(), CL = cluster.num_blocks();
    const int r = blockIdx.x / (int)CL, tid = threadIdx.x;
    const float* row = logits + (size_t)r * ld;
    const int per = ((vocab + (int)CL * 4 - 1) / ((int)CL * 4)) * 4;
    const int begin = min(vocab, (int)rank * per), end = min(vocab, begin + per);

    // ---- the largest logit (lowest id among equals) and the smallest finite one
    unsigned long long best = 0ull, low = 0ull;
    for_each_logit(row, begin, end, [&](int i, float raw) {
        const float v = clean(raw);
        const unsigned long long key = ((unsigned long long)ordered_bits(v) << 32) | (unsigned int)(0xffffffffu - (unsigned int)i);
        best = key > best ? key : best;
        if (v != -INFINITY) { const unsigned long long inv = ~(unsigned long long)ordered_bits(v); low = inv > low ? inv : low; }
    });
    best = block_max_u64(best, red);
    low = block_max_u64(low, red);
    if (tid == 0) { x_best = best; x_low = low; }
    cluster.sync();
    for (unsigned k = 0; k < CL; ++k) {
        const unsigned long long ob = *cluster.map_shared_rank(&x_best, k), ol = *cluster.map_shared_rank(&x_low, k);
        best = ob > best ? ob : best;
        low = ol > low ? ol : low;
    }
    const float top = from_ordered((unsigned int)(best >> 32));
    const float temp = temperature[r];
    const int tk = top_k[r];
    const float tp = top_p[r], mp = min_p[r];
    const bool greedy = !(temp > 0.f) || tk == 1 || !(tp > 0.f);
    const bool odd = !(top > -INFINITY && top < INFINITY);   // all -inf, or +inf among them: the sorting kernel's rules
    if (greedy || odd) {
        if (rank == 0 && tid == 0) {
            if (greedy) out[r] = (int)(0xffffffffu - (unsigned int)(best & 0xffffffffu));
            flagged[r] = greedy ? 0 : 1;
        }
        cluster.sync();                                    // nobody leaves while its shared memory may be read
        return;
    }
    const float inv_t = 1.f / temp, inv_t_log2e = inv_t * 1.4426950408889634f;
    const float bottom = from_ordered((unsigned int)(~low));
    // buckets cover (max - logit) / T from 0 to the row's range, at most 64 (weights below e^-64 are nothing)
    const float range = fminf(fmaxf((top - bottom) * inv_t, 1e-3f), 64.f);
    const float per_unit = (float)(SB - 1) / range;

    // ---- this CTA's part: count and weight of every bucket; count and weight of what min-p keeps
    for (int i = tid; i < SB; i += ST) { cnt[i] = 0u; wsum[i] = 0ull; }
    __syncthreads();
    unsigned long long n_mp = 0ull, w_mp = 0ull;
    for_each_logit(row, begin, end, [&](int, float raw) {
        const float v = clean(raw);
        const float w = weight32(v, top, inv_t_log2e);
        const unsigned long long wf = fixed_of(w);
        const int b = bucket_of(v, top, inv_t, per_unit);
        atomicAdd(&cnt[b], 1u);
        atomicAdd(&wsum[b], wf);
        if (w >= mp) { ++n_mp; w_mp += wf; }
    });
    n_mp = block_sum_u64(n_mp, red);
    w_mp = block_sum_u64(w_mp, red);
    if (tid == 0) { x_nmp = n_mp; x_wmp = w_mp; s_cmd = -2; }
    cluster.sync();

    // gather this CTA's tokens of the buckets lo..hi (a command is lo + hi * 65536) into the first CTA's list
    auto gather = [&](int cmd) {
        const int b_lo = cmd & 0xffff, b_hi = cmd >> 16;
        unsigned long long* far_list = cluster.map_shared_rank(list, 0);
        int* far_listed = cluster.map_shared_rank(&s_listed, 0);
        for_each_logit(row, begin, end, [&](int i, float raw) {
            const float v = clean(raw);
            const int bk = bucket_of(v, top, inv_t, per_unit);
            if (bk >= b_lo && bk <= b_hi) {
                const int at = atomicAdd(far_listed, 1);
                if (at < CAP) far_list[at] = ((unsigned long long)ordered_bits(v) << 32) | (unsigned int)(0xffffffffu - (unsigned int)i);
            }
        });
    };
    if (rank != 0) {
        // ---- the others: gather whatever bucket the first CTA names, until it names none
        for (;;) {
            cluster.sync();                                // a command is there
            const int b = *cluster.map_shared_rank(&s_cmd, 0);
            if (b < 0) break;
            gather(b);
            cluster.sync();                                // the list is complete
        }
        cluster.sync();                                    // the first CTA has seen everyone read the last command
        return;
    }

    // ---- the first CTA: all eight histograms in one, counts and weights before each bucket
    for (int i = tid; i < SB; i += ST) {
        unsigned int c = 0u;
        unsigned long long w = 0ull;
        for (unsigned k = 0; k < CL; ++k) { c += cluster.map_shared_rank(cnt, k)[i]; w += cluster.map_shared_rank(wsum, k)[i]; }
        cnt[i] = c; wsum[i] = w;
    }
    n_mp = 0ull; w_mp = 0ull;
    for (unsigned k = 0; k < CL; ++k) { n_mp += *cluster.map_shared_rank(&x_nmp, k); w_mp += *cluster.map_shared_rank(&x_wmp, k); }
    __syncthreads();
    {
        // counts and weights before each bucket: two buckets a thread, a scan over the warp, then over the warps
        static_assert(SB == 2 * ST, "two buckets a thread");
        const unsigned int c0 = cnt[2 * tid], c1 = cnt[2 * tid + 1];
        const unsigned long long w0 = wsum[2 * tid], w1 = wsum[2 * tid + 1];
        unsigned int c_incl = c0 + c1;
        unsigned long long w_incl = w0 + w1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int ct = __shfl_up_sync(0xffffffffu, c_incl, o);
            const unsigned long long wt = __shfl_up_sync(0xffffffffu, w_incl, o);
            if ((tid & 31) >= o) { c_incl += ct; w_incl += wt; }
        }
        __syncthreads();                                   // every thread has read its buckets and `red` is free
        if ((tid & 31) == 31) { red[tid >> 5] = w_incl; red[32 + (tid >> 5)] = c_incl; }
        __syncthreads();
        if (tid < 32) {
            unsigned long long wt = red[tid], wi = wt;
            unsigned long long ct = red[32 + tid], ci = ct;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long a = __shfl_up_sync(0xffffffffu, wi, o), c = __shfl_up_sync(0xffffffffu, ci, o);
                if (tid >= o) { wi += a; ci += c; }
            }
            red[tid] = wi - wt; red[32 + tid] = ci - ct;    // what lies before each warp
            if (tid == 31) wsum[SB] = wi;
        }
        __syncthreads();
        const unsigned int c_before = (unsigned int)red[32 + (tid >> 5)] + c_incl - (c0 + c1);
        const unsigned long long w_before = red[tid >> 5] + w_incl - (w0 + w1);
        cnt[2 * tid] = c_before; cnt[2 * tid + 1] = c_before + c0;
        wsum[2 * tid] = w_before; wsum[2 * tid + 1] = w_before + w0;
    }
    __syncthreads();
    const unsigned long long total_all = wsum[SB];
    auto count_of = [&](int b) -> int { return (int)((b + 1 < SB ? cnt[b + 1] : (unsigned int)vocab) - cnt[b]); };
    // the bucket that holds the token of this rank (0-based): the last one that starts at or before it
    auto bucket_of_rank = [&](int rk) -> int {
        int lo = 0, hi = SB - 1;
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if ((int)cnt[mid] <= rk) lo = mid; else hi = mid - 1; }
        return lo;
    };
    // The list holds the tokens of the buckets cur_lo..cur_hi, sorted (largest logit first, lowest id
    // among equals), with the running weight over them; base_c tokens of weight base_w lie before them.
    int cur_lo = -1, cur_hi = -2, cur_n = 0, base_c = 0;
    unsigned long long base_w = 0ull;
    // buckets lo..hi into the list; false: too many tokens for it
    auto load_range = [&](int lo, int hi) -> bool {
        if (lo >= cur_lo && hi <= cur_hi) return true;
        const int n = (int)((hi + 1 < SB ? cnt[hi + 1] : (unsigned int)vocab) - cnt[lo]);
        if (n > CAP) return false;
        int pad = 1;
        while (pad < n) pad <<= 1;
        for (int i = tid; i < pad; i += ST) list[i] = 0ull;
        if (tid == 0) { s_listed = 0; s_cmd = lo | (hi << 16); }
        cluster.sync();                                    // the command is there (and the list is clear)
        gather(lo | (hi << 16));
        cluster.sync();                                    // the list is complete
        for (int k = 2; k <= pad; k <<= 1)
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int i = tid; i < pad; i += ST) {
                    const int q = i ^ j;
                    if (q > i) {
                        const unsigned long long a = list[i], c = list[q];
                        const bool desc = (i & k) == 0;
                        if (desc ? a < c : a > c) { list[i] = c; list[q] = a; }
                    }
                }
                __syncthreads();
            }
        // running weight: four tokens a thread, then a scan over the threads
        unsigned long long mine[4], sum = 0ull;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = 4 * tid + e;
            mine[e] = j < n ? fixed_of(weight32(from_ordered((unsigned int)(list[j] >> 32)), top, inv_t_log2e)) : 0ull;
            sum += mine[e];
        }
        unsigned long long incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
            if ((tid & 31) >= o) incl += t;
        }
        if ((tid & 31) == 31) red[tid >> 5] = incl;
        __syncthreads();
        if (tid < 32) {
            unsigned long long t = red[tid], u = t;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long x = __shfl_up_sync(0xffffffffu, u, o);
                if (tid >= o) u += x;
            }
            red[32 + tid] = u - t;                         // weight before this warp
        }
        __syncthreads();
        unsigned long long run = red[32 + (tid >> 5)] + incl - sum;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            run += mine[e];
            if (4 * tid + e < CAP) cum[4 * tid + e] = run;
        }
        __syncthreads();
        cur_lo = lo; cur_hi = hi; cur_n = n; base_c = (int)cnt[lo]; base_w = wsum[lo];
        return true;
    };
    // One bucket.  `more`: something is asked after this, and it lies in this bucket or an earlier one
    // (the top-k cut bounds the top-p prefix, and that the draw): where the buckets from the first one
    // up to this one hold no more than a thousand tokens, all of them are listed at once, one pass over
    // the row and one sort instead of up to three.
    auto load_bucket = [&](int b, bool more) -> bool {
        if (b >= cur_lo && b <= cur_hi) return true;
        if (more && (b + 1 < SB ? cnt[b + 1] : (unsigned int)vocab) <= 1024u) return load_range(0, b);
        return load_range(b, b);
    };
    // the first token j of the list (its rank below `limit`) for which pred(running weight) holds;
    // -1 if none
    auto first_where = [&](int limit, auto pred) -> int {
        if (tid == 0) s_found = 0x7fffffff;
        __syncthreads();
        for (int j = tid; j < cur_n; j += ST)
            if (base_c + j < limit && pred(base_w + cum[j])) { atomicMin(&s_found, j); break; }
        __syncthreads();
        const int j = s_found;
        __syncthreads();
        return j == 0x7fffffff ? -1 : j;
    };
    bool fine = true;
    int token = -1;

    // ---- what top-k and min-p keep: a prefix of `kept` tokens of the sorted order, of weight `total`
    const int K = (tk > 0 && tk < vocab) ? tk : vocab;
    int kept;
    unsigned long long total;
    if (mp > 0.f && (long long)n_mp <= (long long)K) {
        kept = (int)(n_mp > 0ull ? n_mp : 1ull);
        total = w_mp;
    } else if (K < vocab) {
        const int b = bucket_of_rank(K - 1);
        fine = load_bucket(b, true);
        kept = K;
        total = fine ? base_w + cum[K - 1 - base_c] : 0ull;
    } else {
        kept = vocab;
        total = total_all;
    }
    // ---- top-p: the shortest prefix whose share of `total` reaches p
    unsigned long long final_total = total;
    if (fine && tp < 1.f) {
        const double need = (double)tp * (double)total;
        int lo = 0, hi = SB - 1;                           // the first bucket at whose end the running weight has reached `need`
        while (lo < hi) { const int mid = (lo + hi) >> 1; if ((double)wsum[mid + 1] >= need) hi = mid; else lo = mid + 1; }
        fine = load_bucket(lo, true);
        if (fine) {
            const int j = first_where(kept, [&](unsigned long long c) { return (double)c >= need; });
            if (j >= 0) { kept = base_c + j + 1; final_total = base_w + cum[j]; }
        }
    }
    // ---- the draw: the first token at which the running weight passes u * final_total
    if (fine) {
        double u = draw[r];
        u = u < 0.0 ? 0.0 : (u > 1.0 - 2.220446049250313e-16 ? 1.0 - 2.220446049250313e-16 : u);
        const double target = u * (double)final_total;
        int lo = 0, hi = SB - 1;                           // the first bucket whose end lies beyond the target
        while (lo < hi) { const int mid = (lo + hi) >> 1; if ((double)wsum[mid + 1] > target) hi = mid; else lo = mid + 1; }
        int b = lo;
        if ((int)cnt[b] >= kept) b = bucket_of_rank(kept - 1);     // the target lies past the kept prefix: its last token
        fine = load_bucket(b, false);
        if (fine) {
            int j = first_where(kept, [&](unsigned long long c) { return target < (double)c; });
            if (j < 0) j = min(cur_n, kept - base_c) - 1;          // never passed inside the prefix: its last token here
            if (j >= 0) token = (int)(0xffffffffu - (unsigned int)(list[j] & 0xffffffffu));
            else fine = false;
        }
    }
    if (tid == 0) {
        s_cmd = -1;                                        // nothing more to gather
        flagged[r] = fine ? 0 : 1;
        if (fine) out[r] = token;
    }
    cluster.sync();                                        // the last command is there
    cluster.sync();                                        // ... and has been read
}

// ------------------------------------------------------- stop check and token feedback
// After the tokens of a decode step are chosen: per row, count the token, decide whether the
// request stops (a stop id unless ignored, or generated >= max_tokens; the host twin of this
// rule is crates/infer-core/src/ports/pipeline_ops.rs:117-120), and put the token where the
// next step reads its input ids, so that the next step can start before the host has seen
// anything.  slot_state[slot] = {generated, max_tokens, ignore_eos, last_token}.
__global__ void decode_feedback_kernel(const int* __restrict__ sampled, const int* __restrict__ state_slots,
                                       int rows, int* __restrict__ slot_state, const int* __restrict__ eos_ids,
                                       int n_eos, int* __restrict__ result, int* __restrict__ token_feed) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int tok = sampled[r];
    int* st = slot_state + 4 * state_slots[r];
    const int generated = st[0] + 1;
    bool stop = generated >= st[1];
    if (!st[2])
        for (int e = 0; e < n_eos; ++e) stop = stop || tok == eos_ids[e];
    st[0] = generated;
    st[3] = tok;
    result[r] = tok;                                      // [rows] tokens, then [rows] stop flags
    result[rows + r] = stop ? 1 : 0;
    if (token_feed) token_feed[r] = tok;
}
}  // namespace

RI_API int ri_decode_feedback(const int* sampled, const int* state_slots, int rows, int* slot_state,
                              const int* eos_ids, int n_eos, int* result, int* token_feed, void* stream) {
    if (rows <= 0) return 0;
    RI_CHECKED(ri_launch(decode_feedback_kernel, dim3((rows + 127) / 128), dim3(128), 0, (cudaStream_t)stream,
                         sampled, state_slots, rows, slot_state, eos_ids, n_eos, result, token_feed));
    return ri_launch_status();
}

// state: rows 64-bit words, count: rows 32-bit words, both zero before the first call (the
// kernel leaves them zero).  Calls that share them must not overlap on the GPU.
RI_API int ri_argmax(const float* logits, int ld, int rows, int vocab, int* out,
                     unsigned long long* state, unsigned int* count, void* stream) {
    if (rows <= 0) return 0;
    int per_row = (vocab + 2047) / 2048;                 // 8 elements per thread
    const int cap = (4 * ri_device_sms() + rows - 1) / rows;         // about four CTAs per SM in all
    if (per_row > cap) per_row = cap;
    if (per_row < 1) per_row = 1;
    RI_CHECKED(ri_launch(argmax_kernel, dim3(dim3(per_row, rows)), dim3(256), 0, (cudaStream_t)stream, logits, ld, vocab, out, state, count));
    return ri_launch_status();
}

// scratch: rows * vpad + rows 64-bit words, vpad = vocab rounded up to a power of two (the sorting
// kernel's room for the rows it is left with, then one flag per row).
RI_API int ri_sample(const float* logits, int ld, int rows, int vocab, int vpad,
                     unsigned long long* scratch, const float* temperature, const int* top_k,
                     const float* top_p, const float* min_p, const double* draw, int* out,
                     void* stream) {
    if (rows <= 0) return 0;
    if (vpad < vocab || (vpad & (vpad - 1)) != 0) return (int)cudaErrorInvalidValue;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SELECT_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int* flagged = reinterpret_cast<int*>(scratch + (size_t)rows * vpad);
    {
        // CTAs per row: eight while the rows then fit one wave of the GPU, else four, else two
        const int sms = ri_device_sms();
        const int cl = rows * 8 <= sms ? 8 : (rows * 4 <= 2 * sms ? 4 : 2);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(rows * cl);
        cfg.blockDim = dim3(ST);
        cfg.dynamicSmemBytes = SELECT_SMEM;
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ri_pdl_flag() ? 2 : 1;
        RI_CHECKED((int)cudaLaunchKernelEx(&cfg, sample_select_kernel, logits, ld, vocab, temperature, top_k, top_p, min_p,
                                           draw, out, flagged));
    }
    RI_CHECKED(ri_launch(sample_kernel, dim3(rows), dim3(ST), 0, (cudaStream_t)stream, logits, ld, vocab, vpad, scratch, temperature,
                                                         top_k, top_p, min_p, draw, out, (const int*)flagged));
    return ri_launch_status();
}

// the sorting kernel alone, for every row (the reference for the bucketed one)
RI_API int ri_sample_by_sorting(const float* logits, int ld, int rows, int vocab, int vpad,
                                unsigned long long* scratch, const float* temperature, const int* top_k,
                                const float* top_p, const float* min_p, const double* draw, int* out,
                                void* stream) {
    if (rows <= 0) return 0;
    if (vpad < vocab || (vpad & (vpad - 1)) != 0) return (int)cudaErrorInvalidValue;
    RI_CHECKED(ri_launch(sample_kernel, dim3(rows), dim3(ST), 0, (cudaStream_t)stream, logits, ld, vocab, vpad, scratch, temperature,
                                                         top_k, top_p, min_p, draw, out, (const int*)nullptr));
    return ri_launch_status();
}
