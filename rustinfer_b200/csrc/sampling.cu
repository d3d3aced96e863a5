// Choosing the next token on the device: greedy argmax, and temperature sampling with
// top-k, min-p and top-p filters.
//
// Greedy follows crates/infer-backend-cuda/src/kernels/sampler/sampler.cu:66-105 (the
// lowest index wins ties).  The filtered draw follows RustInfer's host sampler
// (crates/infer-worker/src/application/sampler_stack.rs:242-351): logit/T, sort
// descending, top-k, exp(x - max), min-p, normalise, top-p (keep until the cumulative
// share reaches p, at least one), then walk the cumulative weights with draw * total.
// The reference copies the logits to the host for this; here one CTA per row sorts the
// row in a scratch buffer on the device (bitonic, 64-bit keys made of the logit and the
// token id, so equal logits are ordered by ascending id) and does the sums in fp64, in
// rank order within each thread's contiguous segment.
#include "common.cuh"

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

__device__ __forceinline__ double weight_of(unsigned long long key, float top, double inv_t) {
    const float v = from_ordered((unsigned int)(key >> 32));
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
              int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ double buf[ST + 1];
    __shared__ int found;
    const int r = blockIdx.x, tid = threadIdx.x;
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

// scratch: rows * vpad 64-bit words, vpad = vocab rounded up to a power of two.
RI_API int ri_sample(const float* logits, int ld, int rows, int vocab, int vpad,
                     unsigned long long* scratch, const float* temperature, const int* top_k,
                     const float* top_p, const float* min_p, const double* draw, int* out,
                     void* stream) {
    if (rows <= 0) return 0;
    if (vpad < vocab || (vpad & (vpad - 1)) != 0) return (int)cudaErrorInvalidValue;
    RI_CHECKED(ri_launch(sample_kernel, dim3(rows), dim3(ST), 0, (cudaStream_t)stream, logits, ld, vocab, vpad, scratch, temperature,
                                                         top_k, top_p, min_p, draw, out));
    return ri_launch_status();
}
