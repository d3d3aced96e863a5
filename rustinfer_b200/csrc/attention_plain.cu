// Paged causal GQA attention over the cache, any head size (compiled for one
// RI_HEAD_DIM, a multiple of 16), storage fp32 or bf16, all arithmetic fp32 on CUDA
// cores.  It is the attention of the true-32-bit path and the fallback of the bf16
// path; it serves whole prompts, portions of prompts and single decoded tokens alike.
//
// What it computes is RustInfer's paged attention
// (crates/infer-core/src/ports/fused_ops.rs:484-523): the query at position p of a
// request sees keys 0..p (with a window w: p-w+1..p), kv head = q head / (Hq/Hkv),
// scores (q.k)*scale, softmax with the maximum subtracted.  The reference has no fp32
// attention on the GPU (crates/infer-backend-cuda/src/kernels/flash_attn_gqa/flash_attn_gqa.h:30).
//
// One CTA of 128 threads handles a tile of 16 consecutive query tokens of one request
// and one q head.  Keys are visited in chunks of KC that start at multiples of KC from
// key 0, with an online softmax; the order of every sum is therefore the same however
// the tokens were cut into steps or tiles, and so are the bits of the result.
#include "common.cuh"

#ifndef RI_HEAD_DIM
#error "compile with -DRI_HEAD_DIM=<head size>"
#endif

namespace {
constexpr int HD = RI_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 512, "head size must be a multiple of 16 up to 512");
constexpr int QT = 16;                         // query rows per CTA
constexpr int KC = HD <= 128 ? 64 : 32;        // keys per chunk
constexpr int THREADS = 128;
constexpr int NCOL = KC / 8;                   // score columns per thread
constexpr int NACC = HD / 8;                   // output dims per thread
constexpr int QS = HD + 1, KS = HD + 1, PS = KC + 1;
constexpr size_t SMEM_FLOATS = (size_t)QT * QS + (size_t)KC * KS + (size_t)KC * HD + (size_t)QT * PS;

template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_plain_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                       const T* __restrict__ cache, const int* __restrict__ block_table,
                       int table_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                       const int* __restrict__ tile_entry, const int* __restrict__ tile_q0,
                       int Hq, int Hkv, int page_size, float scale, int window) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* Qs = smem;
    float* Ks = Qs + QT * QS;
    float* Vs = Ks + KC * KS;
    float* Ps = Vs + KC * HD;

    const int tile = blockIdx.x, h = blockIdx.y;
    const int b = tile_entry[tile];
    if (b < 0) return;                                   // padding tile
    const int j0 = tile_q0[tile];
    const int q_begin = cu_q[b], q_len = cu_q[b + 1] - q_begin;
    const int kvl = kv_len[b];
    const int pos0 = kvl - q_len;                        // position of the entry's first token
    const int g = h / (Hq / Hkv);
    const int tid = threadIdx.x;
    const int row = tid >> 3, l8 = tid & 7;
    const int rows_here = min(QT, q_len - j0);
    if (rows_here <= 0) return;

    for (int e = tid; e < QT * HD; e += THREADS) {
        const int r = e / HD, d = e - r * HD;
        Qs[r * QS + d] = r < rows_here
            ? to_f32<T>(q[(size_t)(q_begin + j0 + r) * q_stride + (size_t)h * HD + d]) : 0.f;
    }

    const bool row_valid = row < rows_here;
    const int p_row = pos0 + j0 + row;                   // this row's position
    const int lo_row = window > 0 ? max(0, p_row - window + 1) : 0;
    const int p_last = pos0 + j0 + rows_here - 1;        // last key any row of the tile sees
    const int lo_tile = window > 0 ? max(0, pos0 + j0 - window + 1) : 0;

    float m = -INFINITY, l = 0.f;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;

    const int* bt = block_table + (size_t)b * table_stride;
    const size_t head_step = (size_t)page_size * HD;
    for (int kb = (lo_tile / KC) * KC; kb <= p_last; kb += KC) {
        __syncthreads();                                 // previous chunk's Vs/Ps reads are done
        for (int e = tid; e < KC * HD; e += THREADS) {
            const int kk = e / HD, d = e - kk * HD;
            const int key = kb + kk;
            float kval = 0.f, vval = 0.f;
            if (key >= lo_tile && key <= p_last) {
                const int page = bt[key / page_size], off = key % page_size;
                const size_t base = ((size_t)(page * 2) * Hkv + g) * head_step + (size_t)off * HD + d;
                kval = to_f32<T>(cache[base]);
                vval = to_f32<T>(cache[base + (size_t)Hkv * head_step]);
            }
            Ks[kk * KS + d] = kval;
            Vs[kk * HD + d] = vval;
        }
        __syncthreads();

        float s[NCOL];
        float cmax = -INFINITY;
#pragma unroll
        for (int c = 0; c < NCOL; ++c) {
            const int kk = l8 + 8 * c;
            const int key = kb + kk;
            float dot = 0.f;
            const float* qr = Qs + row * QS;
            const float* kr = Ks + kk * KS;
#pragma unroll 8
            for (int d = 0; d < HD; ++d) dot = fmaf(qr[d], kr[d], dot);
            const bool seen = row_valid && key <= p_row && key >= lo_row;
            s[c] = seen ? dot * scale : -INFINITY;
            cmax = fmaxf(cmax, s[c]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
        const float m_new = fmaxf(m, cmax);
        float alpha = 1.f, psum = 0.f;
        if (m_new == -INFINITY) {
#pragma unroll
            for (int c = 0; c < NCOL; ++c) Ps[row * PS + l8 + 8 * c] = 0.f;
        } else {
            alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
#pragma unroll
            for (int c = 0; c < NCOL; ++c) {
                const float p = (s[c] == -INFINITY) ? 0.f : expf(s[c] - m_new);
                Ps[row * PS + l8 + 8 * c] = p;
                psum += p;
            }
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        l = l * alpha + psum;
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        __syncthreads();
        const float* pr = Ps + row * PS;
        for (int kk = 0; kk < KC; ++kk) {
            const float p = pr[kk];
            const float* vr = Vs + kk * HD + l8;
#pragma unroll
            for (int i = 0; i < NACC; ++i) acc[i] = fmaf(p, vr[8 * i], acc[i]);
        }
    }
    if (row_valid) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* o = out + (size_t)(q_begin + j0 + row) * out_stride + (size_t)h * HD + l8;
#pragma unroll
        for (int i = 0; i < NACC; ++i) o[8 * i] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T>
int launch(const void* q, int q_stride, void* out, int out_stride, const void* cache,
           const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
           const int* tile_entry, const int* tile_q0, int n_tiles, int Hq, int Hkv, int page_size,
           float scale, int window, cudaStream_t s) {
    static bool configured = false;
    const size_t smem = SMEM_FLOATS * sizeof(float);
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_plain_kernel<T>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, Hq);
    RI_CHECKED(ri_launch(attention_plain_kernel<T>, dim3(grid), dim3(THREADS), smem, s, 
        (const T*)q, q_stride, (T*)out, out_stride, (const T*)cache, block_table, table_stride,
        cu_q, kv_len, tile_entry, tile_q0, Hq, Hkv, page_size, scale, window));
    return ri_launch_status();
}
}  // namespace

RI_API int ri_attention_plain_head_dim() { return HD; }
RI_API int ri_attention_plain_tile_rows() { return QT; }

// q: rows of `q_stride` elements, head h at column h*HD; out likewise with out_stride.
// cache: one layer, [page][K|V][kv head][slot][HD].  tile_entry[i] = batch entry of tile i
// (-1: skip), tile_q0[i] = its first query row within that entry.
RI_API int ri_attention_plain(const void* q, int q_stride, void* out, int out_stride,
                              const void* cache, int dtype, const int* block_table, int table_stride,
                              const int* cu_q, const int* kv_len, const int* tile_entry,
                              const int* tile_q0, int n_tiles, int Hq, int Hkv, int page_size,
                              float scale, int window, void* stream) {
    if (n_tiles <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv != 0) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RI_BF16)
        return launch<bf16>(q, q_stride, out, out_stride, cache, block_table, table_stride, cu_q,
                            kv_len, tile_entry, tile_q0, n_tiles, Hq, Hkv, page_size, scale, window, s);
    return launch<float>(q, q_stride, out, out_stride, cache, block_table, table_stride, cu_q,
                         kv_len, tile_entry, tile_q0, n_tiles, Hq, Hkv, page_size, scale, window, s);
}

RI_API void ri_set_pdl(int on) { ri_pdl_flag() = on ? 1 : 0; }
