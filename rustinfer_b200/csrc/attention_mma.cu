// Paged causal GQA attention in bf16 on the tensor cores (mma.sync m16n8k16, fp32
// accumulate), compiled for one RI_HEAD_DIM (a multiple of 16, at most 256).  Scores,
// softmax and the output accumulators are fp32; probabilities are rounded to bf16 for
// the P*V product, as in RustInfer's flash kernels
// (crates/infer-backend-cuda/src/kernels/flash_attn_gqa/flash_attn_paged_prefill.cu:442-511).
//
// Two kernels share the tile loader and the fragment code:
//
//  prefill  one CTA = 64 rows x one kv head, a row being (query token, q head of the kv
//           head's group), so the heads of a group share every K/V tile that is loaded
//           (the reference runs one CTA per q head, :539-568, and fetches K/V with
//           synchronous scalar loads, :379-407).  4 warps x 16 rows; K/V tiles of 64 keys
//           gathered page by page with cp.async into a double buffer.
//  decode   one CTA = the q heads of one kv head for one request's single new token and
//           one split of its keys; the 4 warps take 16 keys each of every 64-key tile and
//           merge their online-softmax states at the end.  With several splits the partial
//           outputs and log-sum-exps go to scratch and a second kernel combines them
//           (split-KV as in flash_attn_paged_decode.cu:75-340, but with the group's heads
//           as the M dimension of the MMA instead of scalar dot products).
//
// Cache layout of one layer: [page][K|V][kv head][slot in page][head_dim], so a page's
// keys of one head are one contiguous run.
#include "common.cuh"
#include <cuda.h>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#ifndef RI_HEAD_DIM
#error "compile with -DRI_HEAD_DIM=<head size>"
#endif

namespace {
constexpr int HD = RI_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "mma attention: head size multiple of 16, at most 256");
constexpr int KT = 64;                 // keys per tile
constexpr int ROW = HD + 8;            // padded smem row (elements): rows shift by 16 B, ldmatrix is conflict-free
constexpr int CH = HD / 8;             // 16-byte chunks per row
constexpr int KS = HD / 16;            // k-steps of Q*K^T
constexpr int NT = HD / 8;             // n-tiles of the output
constexpr int THREADS = 128;
constexpr int MT = 64;                 // rows per prefill CTA
// K/V tiles a decode CTA keeps in flight: decode is a pure stream of the cache, and what
// bounds it is how many bytes every SM has on the way
// Measured on B200 (32/8 heads of 64, 4,096 keys; us for batch 8 / batch 64, best split each):
// 4 warps x 2 stages 20.6 / 107, 4 x 4 22.0 / 127, 8 x 2 22.8 / 114, 6 x 2 24.2 / 129.  More CTAs
// per SM (5 at 39 KB each) beat deeper rings.
#ifndef RI_DEC_WARPS
#define RI_DEC_WARPS 4
#endif
#ifndef RI_DEC_STAGES
#define RI_DEC_STAGES 2
#endif
constexpr int DWARPS = RI_DEC_WARPS;                 // warps of a decode CTA, 16 keys of every tile each
constexpr int DTHREADS = 32 * DWARPS;
constexpr int DKT = 16 * DWARPS;                     // keys per decode tile
constexpr int DSTAGES = RI_DEC_STAGES;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;      // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// K and V rows of keys k0 .. k0+KT-1 of one kv head into smem; keys outside [k_lo, k_hi)
// are zero-filled and their pages are never looked up.
template <int TILE_KEYS, int NTHREADS>
__device__ __forceinline__ void load_kv_tile(bf16* Ks, bf16* Vs, const bf16* __restrict__ cache,
                                             const int* __restrict__ bt, int k0, int k_lo, int k_hi,
                                             int Hkv, int kvh, int page_size) {
    const size_t head_step = (size_t)page_size * HD;
    const int shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;   // power of two: no division
    for (int c = threadIdx.x; c < TILE_KEYS * CH; c += NTHREADS) {
        const int kk = c / CH, ch = c - kk * CH;
        const int key = k0 + kk;
        const bool ok = key >= k_lo && key < k_hi;
        const bf16* sk = cache;
        const bf16* sv = cache;
        if (ok) {
            const int blk = shift >= 0 ? key >> shift : key / page_size;
            const int page = bt[blk], off = key - blk * page_size;
            sk = cache + ((size_t)(page * 2) * Hkv + kvh) * head_step + (size_t)off * HD + ch * 8;
            sv = sk + (size_t)Hkv * head_step;
        }
        cp_async16(Ks + kk * ROW + ch * 8, sk, ok);
        cp_async16(Vs + kk * ROW + ch * 8, sv, ok);
    }
}

// ================================================================== prefill / ragged
__global__ void __launch_bounds__(THREADS)
prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
               const bf16* __restrict__ cache, const int* __restrict__ block_table, int table_stride,
               const int* __restrict__ cu_q, const int* __restrict__ kv_len,
               const int* __restrict__ tile_entry, const int* __restrict__ tile_tok0,
               int Hq, int Hkv, int Gc, int chunks, int tpt, int page_size, float scale_log2, int window) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);            // [MT][ROW]
    bf16* KVs = Qs + MT * ROW;                               // [2 buffers][K|V][KT][ROW]

    const int b = tile_entry[blockIdx.x];
    if (b < 0) return;
    const int tok0 = tile_tok0[blockIdx.x];
    const int G = Hq / Hkv;
    const int kvh = blockIdx.y / chunks, hc = blockIdx.y - kvh * chunks;
    const int head0 = kvh * G + hc * Gc;
    const int nheads = min(Gc, G - hc * Gc);
    const int q_begin = cu_q[b], q_len = cu_q[b + 1] - q_begin;
    const int kvl = kv_len[b];
    const int pos0 = kvl - q_len;
    const int ntok = min(tpt, q_len - tok0);
    if (ntok <= 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // Q rows: row r = (token tok0 + r / Gc, head head0 + r % Gc)
    for (int c = tid; c < MT * CH; c += THREADS) {
        const int r = c / CH, ch = c - r * CH;
        const int jj = r / Gc, hh = r - jj * Gc;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (jj < ntok && hh < nheads)
            v = *reinterpret_cast<const uint4*>(q + (size_t)(q_begin + tok0 + jj) * q_stride +
                                                (size_t)(head0 + hh) * HD + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * ROW + ch * 8) = v;
    }

    const int p_first = pos0 + tok0, p_last = p_first + ntok - 1;
    const int lo_tile = window > 0 ? max(0, p_first - window + 1) : 0;
    const int t_begin = lo_tile / KT, t_end = p_last / KT + 1;
    const int* bt = block_table + (size_t)b * table_stride;

    load_kv_tile<KT, THREADS>(KVs, KVs + KT * ROW, cache, bt, t_begin * KT, lo_tile, p_last + 1, Hkv, kvh, page_size);
    cp_async_commit();
    __syncthreads();                                          // Qs is written

    // this thread's two rows: r0 = 16*warp + lane/4 and r0 + 8
    int p_row[2], lo_row[2];
    bool ok_row[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + (lane >> 2) + 8 * i;
        const int jj = r / Gc, hh = r - jj * Gc;
        ok_row[i] = jj < ntok && hh < nheads;
        p_row[i] = p_first + jj;
        lo_row[i] = window > 0 ? max(0, p_row[i] - window + 1) : 0;
    }

    const int p_warp_first = p_first + (warp * 16) / Gc;     // position of the warp's first row
    unsigned qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qf[ks], Qs + (warp * 16 + (lane & 15)) * ROW + ks * 16 + (lane >> 4) * 8);

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) & 1;
        bf16* Ks = KVs + buf * 2 * KT * ROW;
        bf16* Vs = Ks + KT * ROW;
        if (t + 1 < t_end) {
            bf16* Kn = KVs + (buf ^ 1) * 2 * KT * ROW;
            load_kv_tile<KT, THREADS>(Kn, Kn + KT * ROW, cache, bt, (t + 1) * KT, lo_tile, p_last + 1, Hkv, kvh, page_size);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        float s[KT / 8][4];
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < KT / 16; ++np) {
                unsigned kf[4];
                ldmatrix_x4(kf, Ks + (np * 16 + (lane & 7) + (lane >> 4) * 8) * ROW + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[2 * np], qf[ks], kf[0], kf[1]);
                mma_bf16(s[2 * np + 1], qf[ks], kf[2], kf[3]);
            }
        }
        // Scores stay unscaled; the scale rides on the exponent: p = 2^(s*scale - m).  Only
        // tiles that reach past the warp's first row (the diagonal) or a window need masks.
        const int key0 = t * KT + (lane & 3) * 2;
        float mx[2] = {-INFINITY, -INFINITY};
        if (window > 0 || t * KT + KT - 1 > p_warp_first) {
#pragma unroll
            for (int n = 0; n < KT / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + n * 8 + (e & 1);
                    const int i = e >> 1;
                    const bool seen = ok_row[i] && key <= p_row[i] && key >= lo_row[i];
                    s[n][e] = seen ? s[n][e] : -INFINITY;
                    mx[i] = fmaxf(mx[i], s[n][e]);
                }
            }
        } else {
#pragma unroll
            for (int n = 0; n < KT / 8; ++n) {
                mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
            }
        }
        float alpha[2], muse[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float mnew = fmaxf(m[i], mx[i] * scale_log2);       // m is kept in scaled units
            muse[i] = mnew == -INFINITY ? 0.f : mnew;
            alpha[i] = exp2f(m[i] - muse[i]);
            m[i] = mnew;
            l[i] *= alpha[i];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
            o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
        }
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[n][e] = exp2f(fmaf(s[n][e], scale_log2, -muse[e >> 1]));
                l[e >> 1] += s[n][e];
            }
        }
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            unsigned pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                unsigned vf[4];
                ldmatrix_x4_trans(vf, Vs + (kk * 16 + (lane & 15)) * ROW + np * 16 + (lane >> 4) * 8);
                mma_bf16(o[2 * np], pa, vf[0], vf[1]);
                mma_bf16(o[2 * np + 1], pa, vf[2], vf[3]);
            }
        }
        __syncthreads();                                      // all warps are done with this buffer
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        if (!ok_row[i]) continue;
        const int r = warp * 16 + (lane >> 2) + 8 * i;
        const int jj = r / Gc, hh = r - jj * Gc;
        const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
        bf16* dst = out + (size_t)(q_begin + tok0 + jj) * out_stride + (size_t)(head0 + hh) * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NT; ++n)
            *reinterpret_cast<unsigned*>(dst + n * 8) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    }
}

// ========================================================================== decode
// grid (kv heads * head chunks, splits, decode entries).  part_o [entries][Hq][splits][HD]
// fp32 and part_lse [entries][Hq][splits] (base-2 log-sum-exp) are written when splits > 1.
__global__ void __launch_bounds__(DTHREADS)
decode_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
              const bf16* __restrict__ cache, const int* __restrict__ block_table, int table_stride,
              const int* __restrict__ cu_q, const int* __restrict__ kv_len,
              const int* __restrict__ entry_list, int Hq, int Hkv, int Gc, int chunks, int page_size,
              float scale_log2, int window, int splits, float* __restrict__ part_o,
              float* __restrict__ part_lse) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);            // [16][ROW]
    bf16* KVs = Qs + 16 * ROW;                               // [DSTAGES][K|V][DKT][ROW]

    const int slot = blockIdx.z;
    const int b = entry_list ? entry_list[slot] : slot;
    if (b < 0) return;
    const int split = blockIdx.y;
    const int G = Hq / Hkv;
    const int kvh = blockIdx.x / chunks, hc = blockIdx.x - kvh * chunks;
    const int head0 = kvh * G + hc * Gc;
    const int nheads = min(Gc, G - hc * Gc);
    const int tok = cu_q[b + 1] - 1;                          // the entry's (last) token row
    const int kvl = kv_len[b];
    const int lo = window > 0 ? max(0, kvl - window) : 0;
    const int t_first = lo / DKT, t_count = (kvl + DKT - 1) / DKT - t_first;
    const int per = (t_count + splits - 1) / splits;
    const int t_begin = t_first + split * per, t_end = min(t_begin + per, t_first + t_count);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int* bt = block_table + (size_t)b * table_stride;

    // prologue of the ring: tiles t_begin .. t_begin + DSTAGES - 2 (a group per tile, empty or not)
#pragma unroll
    for (int i = 0; i < DSTAGES - 1; ++i) {
        if (t_begin + i < t_end) {
            bf16* Kb = KVs + i * 2 * DKT * ROW;
            load_kv_tile<DKT, DTHREADS>(Kb, Kb + DKT * ROW, cache, bt, (t_begin + i) * DKT, lo, kvl, Hkv, kvh, page_size);
        }
        cp_async_commit();
    }
    for (int c = tid; c < 16 * CH; c += DTHREADS) {
        const int r = c / CH, ch = c - r * CH;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < nheads)
            v = *reinterpret_cast<const uint4*>(q + (size_t)tok * q_stride + (size_t)(head0 + r) * HD + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * ROW + ch * 8) = v;
    }
    __syncthreads();
    unsigned qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qf[ks], Qs + (lane & 15) * ROW + ks * 16 + (lane >> 4) * 8);

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int kw0 = warp * 16;                                // this warp's 16 keys of every tile

    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) % DSTAGES;
        bf16* Ks = KVs + buf * 2 * DKT * ROW;
        bf16* Vs = Ks + DKT * ROW;
        cp_async_wait<DSTAGES - 2>();                         // tile t has landed (this thread's part)
        __syncthreads();                                      // ... everyone's part; and tile t-1 is consumed
        {
            const int tn = t + DSTAGES - 1;                   // refill the buffer tile t-1 used
            if (tn < t_end) {
                bf16* Kn = KVs + ((tn - t_begin) % DSTAGES) * 2 * DKT * ROW;
                load_kv_tile<DKT, DTHREADS>(Kn, Kn + DKT * ROW, cache, bt, tn * DKT, lo, kvl, Hkv, kvh, page_size);
            }
            cp_async_commit();
        }
        if (t * DKT + kw0 < kvl) {                             // the warp's keys are not all past the end
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                unsigned kf[4];
                ldmatrix_x4(kf, Ks + (kw0 + (lane & 7) + (lane >> 4) * 8) * ROW + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[0], qf[ks], kf[0], kf[1]);
                mma_bf16(s[1], qf[ks], kf[2], kf[3]);
            }
            const int key0 = t * DKT + kw0 + (lane & 3) * 2;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + n * 8 + (e & 1);
                    s[n][e] = (key >= lo && key < kvl) ? s[n][e] * scale_log2 : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
                }
            float alpha[2], muse[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float mnew = fmaxf(m[i], mx[i]);
                muse[i] = mnew == -INFINITY ? 0.f : mnew;
                alpha[i] = exp2f(m[i] - muse[i]);
                m[i] = mnew;
                l[i] *= alpha[i];
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[n][e] = exp2f(s[n][e] - muse[e >> 1]);
                    l[e >> 1] += s[n][e];
                }
            unsigned pa[4];
            pa[0] = pack_bf16(s[0][0], s[0][1]);
            pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[2] = pack_bf16(s[1][0], s[1][1]);
            pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                unsigned vf[4];
                ldmatrix_x4_trans(vf, Vs + (kw0 + (lane & 15)) * ROW + np * 16 + (lane >> 4) * 8);
                mma_bf16(o[2 * np], pa, vf[0], vf[1]);
                mma_bf16(o[2 * np + 1], pa, vf[2], vf[3]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // merge the warps' states through shared memory (the K/V buffers are free now)
    float* Os = reinterpret_cast<float*>(KVs);               // [DWARPS][16][HD]
    float* Ms = Os + DWARPS * 16 * HD;                       // [DWARPS][16]
    float* Ls = Ms + DWARPS * 16;                            // [DWARPS][16]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        const int r = (lane >> 2) + 8 * i;
        float* orow = Os + ((size_t)warp * 16 + r) * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            orow[n * 8] = o[n][2 * i];
            orow[n * 8 + 1] = o[n][2 * i + 1];
        }
        if ((lane & 3) == 0) {
            Ms[warp * 16 + r] = m[i];
            Ls[warp * 16 + r] = l[i];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < nheads * HD; idx += DTHREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DWARPS; ++w) M = fmaxf(M, Ms[w * 16 + r]);
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < DWARPS; ++w) {
                const float f = exp2f(Ms[w * 16 + r] - M);
                L += Ls[w * 16 + r] * f;
                O += Os[((size_t)w * 16 + r) * HD + d] * f;
            }
        }
        const int head = head0 + r;
        const float val = L > 0.f ? O / L : 0.f;
        if (splits == 1) {
            out[(size_t)tok * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(val);
        } else {
            const size_t p = ((size_t)slot * Hq + head) * splits + split;
            part_o[p * HD + d] = val;
            if (d == 0) part_lse[p] = L > 0.f ? M + log2f(L) : -INFINITY;
        }
    }
}

#if RI_HEAD_DIM == 64 || RI_HEAD_DIM == 128
// ============================================================ decode, keys and values by TMA
// The same arithmetic as decode_kernel (a warp takes 16 keys of every 64-key tile, mma.sync,
// fp32 online softmax, the warps' states merged at the end), but no thread computes an address
// in the cache: a fifth warp issues a TMA box per page and kv head (each box from a lane of its
// own) into a ring of 128-byte-swizzled stages (full/empty mbarriers), and the warps read them with ldmatrix
// through the swizzle.  The cp.async kernel above spends its issue slots on page look-ups and
// address arithmetic (3.4 TB/s at batch 8, 4.5 at batch 64); this one is bound by the ring.
// Head sizes 64 and 128, pages of 8, 16, 32 or a multiple of 64 keys.
constexpr int TSTAGES = 3;
constexpr int TKB = HD / 64;                                   // 64-column blocks of a head
constexpr int T_TILE_BYTES = DKT * 128 * TKB;                  // K (or V) of one tile
constexpr int T_STAGE_BYTES = 2 * T_TILE_BYTES;
constexpr int TTHREADS = DTHREADS + 32;
constexpr unsigned T_SPIN_LIMIT = 1u << 20;
constexpr size_t DECODE_TMA_SMEM = 1024 /*alignment*/ + (size_t)TSTAGES * T_STAGE_BYTES + 16 * (size_t)ROW * sizeof(bf16) + 256;
static_assert((size_t)TSTAGES * T_STAGE_BYTES >= (DWARPS * 16 * (size_t)HD + 2 * DWARPS * 16) * sizeof(float), "the merge reuses the ring");

__device__ __forceinline__ unsigned tsm(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tsm(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void tbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tsm(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tsm(bar)) : "memory");
}
__device__ __forceinline__ bool tbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(tsm(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// bounded: false after T_SPIN_LIMIT tries, with 21 in *error
__device__ __forceinline__ bool tbar_wait(uint64_t* bar, unsigned parity, int* error) {
#pragma unroll 1
    for (unsigned i = 0; i < T_SPIN_LIMIT; ++i) {
        if (tbar_try_wait(bar, parity)) return true;
        if (i > 1024) __nanosleep(64);
    }
    atomicExch(error, 21);
    return false;
}
__device__ __forceinline__ void t_tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(tsm(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(tsm(bar)), "r"(x), "r"(y) : "memory");
}
// where the 16 bytes of columns col..col+7 of key row `row` lie in a tile [TKB][DKT rows][128 B]
// written by TMA with the 128-byte swizzle
__device__ __forceinline__ const unsigned char* swz(const unsigned char* tile, int row, int col) {
    return tile + (col >> 6) * (DKT * 128) + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(TTHREADS)
decode_tma_kernel(const __grid_constant__ CUtensorMap cache_map, const bf16* __restrict__ q, int q_stride,
                  bf16* __restrict__ out, int out_stride, const int* __restrict__ block_table, int table_stride,
                  const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                  const int* __restrict__ entry_list, int Hq, int Hkv, int Gc, int chunks, int page_size, int box_rows,
                  float scale_log2, int window, int splits, float* __restrict__ part_o,
                  float* __restrict__ part_lse, int* __restrict__ error) {
    // The kernel before this one (rotary encoding and cache write, alone or at the end of a chain)
    // writes q and the keys and values of this step's tokens only; what the step was told
    // (entries, lengths, block table) and every earlier key were written before it began.  So
    // only the loads of q and of the tile that holds the newest key wait for it.
    pdl_trigger();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    bf16* Qs = reinterpret_cast<bf16*>(ring + (size_t)TSTAGES * T_STAGE_BYTES);    // [16][ROW]
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(Qs) + 16 * ROW * sizeof(bf16));
    uint64_t* empty = full + TSTAGES;

    const int slot = blockIdx.z;
    const int b = entry_list ? entry_list[slot] : slot;
    if (b < 0) return;
    const int split = blockIdx.y;
    const int G = Hq / Hkv;
    const int kvh = blockIdx.x / chunks, hc = blockIdx.x - kvh * chunks;
    const int head0 = kvh * G + hc * Gc;
    const int nheads = min(Gc, G - hc * Gc);
    const int tok = cu_q[b + 1] - 1;
    const int kvl = kv_len[b];
    const int lo = window > 0 ? max(0, kvl - window) : 0;
    const int t_first = lo / DKT, t_count = (kvl + DKT - 1) / DKT - t_first;
    const int per = (t_count + splits - 1) / splits;
    const int t_begin = t_first + split * per, t_end = min(t_begin + per, t_first + t_count);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == DWARPS * 32) {                              // the producer: its first tiles go out before the others are ready
        for (int s = 0; s < TSTAGES; ++s) { tbar_init(&full[s], 1); tbar_init(&empty[s], DWARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < DTHREADS) {
        pdl_wait();
        for (int c = tid; c < 16 * CH; c += DTHREADS) {
            const int r = c / CH, ch = c - r * CH;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < nheads)
                v = *reinterpret_cast<const uint4*>(q + (size_t)tok * q_stride + (size_t)(head0 + r) * HD + ch * 8);
            *reinterpret_cast<uint4*>(Qs + r * ROW + ch * 8) = v;
        }
    }
    // ------------------------------------------------------------------------ TMA producer
    // The fifth warp.  Lane 0 waits for a free stage and announces the bytes; every box of the tile
    // (a page's keys or values, one 64-column block) goes out from a lane of its own, since one
    // thread sends a box only every 74 ns and 8 to 16 boxes a tile from one thread paced the CTA.
    // No division in the loop, page numbers read one tile ahead.  Pages past the request's last
    // one are never allocated: its first page is read instead (those keys are masked, their V rows
    // zeroed before use).  The first tiles go out before the other warps have q.
    const bool producer = warp == DWARPS;
    const int* bt = block_table + (size_t)b * table_stride;
    const int boxes = DKT / box_rows;                      // at most 8 pages meet a tile
    const bool small_pages = page_size < DKT;
    const int kv_step = Hkv * page_size;
    const int t_newest = t_first + t_count - 1;            // the tile with this step's key
    int blk = (t_begin * DKT) / page_size, off = small_pages ? 0 : (t_begin * DKT) % page_size;
    // this lane's box of a tile: keys or values, page p_c of the tile, 64-column block p_kb
    const int p_kv = lane / (boxes * TKB), p_rem = lane - p_kv * boxes * TKB;
    const int p_c = p_rem / TKB, p_kb = p_rem - p_c * TKB;
    const bool p_mine = producer && lane < 2 * boxes * TKB;
    auto look_up = [&](int key0, int blk0, bool live) -> int {
        return (live && p_mine) ? bt[key0 + p_c * box_rows < kvl ? blk0 + p_c : 0] : 0;
    };
    int page = 0;
    bool p_ok = true, waited = false;
    int p_s = 0;
    unsigned p_par = 1;
    auto issue = [&](int t) {                              // the whole producer warp
        const int key0 = t * DKT;
        int blk_n = blk, off_n = off;
        if (small_pages) blk_n += boxes;
        else if ((off_n += DKT) >= page_size) { off_n = 0; ++blk_n; }
        const int page_next = look_up(key0 + DKT, blk_n, t + 1 < t_end);
        int good = 1;
        if (lane == 0 && t - t_begin >= TSTAGES && !tbar_try_wait(&empty[p_s], p_par) && !tbar_wait(&empty[p_s], p_par, error)) good = 0;
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) { p_ok = false; return; }
        if (t >= t_newest && !waited) { pdl_wait(); waited = true; }
        unsigned char* dst = ring + (size_t)p_s * T_STAGE_BYTES;
        if (lane == 0) tbar_expect_tx(&full[p_s], T_STAGE_BYTES);
        if (p_mine) {
            const int row = (page * 2 * Hkv + kvh) * page_size + p_kv * kv_step + (key0 + p_c * box_rows < kvl ? off : 0);
            t_tma_load_2d(dst + p_kv * T_TILE_BYTES + p_kb * (DKT * 128) + p_c * box_rows * 128, &cache_map, &full[p_s], p_kb * 64, row);
        }
        page = page_next;
        blk = blk_n; off = off_n;
        if (++p_s == TSTAGES) { p_s = 0; p_par ^= 1u; }
    };
    const int t_early = min(t_end, t_begin + TSTAGES);
    if (producer) {
        __syncwarp();                                      // lane 0 has set the barriers up
        page = look_up(t_begin * DKT, blk, t_begin < t_end);
        for (int t = t_begin; t < t_early && p_ok; ++t) issue(t);
    }
    __syncwarp();
    __syncthreads();

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (warp == DWARPS) {
        for (int t = t_early; t < t_end && p_ok; ++t) issue(t);
    } else {
        // ---------------------------------------------------------------------- the warps
        unsigned qf[KS][4];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
            ldmatrix_x4(qf[ks], Qs + (lane & 15) * ROW + ks * 16 + (lane >> 4) * 8);
        const int kw0 = warp * 16;
        bool ok = true;
        int s = 0;
        unsigned par = 0;
        for (int t = t_begin; t < t_end && ok; ++t) {
            const unsigned char* Kt = ring + (size_t)s * T_STAGE_BYTES;
            unsigned char* Vt = ring + (size_t)s * T_STAGE_BYTES + T_TILE_BYTES;
            if (!tbar_try_wait(&full[s], par) && !tbar_wait(&full[s], par, error)) { ok = false; break; }
            if (t * DKT + kw0 < kvl) {
                // value rows of keys past the end, or before the window (their pages may have been
                // given back and belong to another request by now), hold whatever the cache holds
                // there: they meet probability zero, but zero times NaN is NaN, so they are cleared
                if (t * DKT + kw0 + 16 > kvl || t * DKT + kw0 < lo) {
                    for (int i = lane; i < 16 * TKB * 8; i += 32) {
                        const int r = kw0 + (i / (TKB * 8)), c8 = i % (TKB * 8);
                        if (t * DKT + r >= kvl || t * DKT + r < lo)
                            *reinterpret_cast<uint4*>(const_cast<unsigned char*>(swz(Vt, r, c8 * 8))) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    __syncwarp();
                }
                float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    unsigned kf[4];
                    ldmatrix_x4(kf, swz(Kt, kw0 + (lane & 7) + (lane >> 4) * 8, ks * 16 + ((lane >> 3) & 1) * 8));
                    mma_bf16(sc[0], qf[ks], kf[0], kf[1]);
                    mma_bf16(sc[1], qf[ks], kf[2], kf[3]);
                }
                const int key0 = t * DKT + kw0 + (lane & 3) * 2;
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + n * 8 + (e & 1);
                        sc[n][e] = (key >= lo && key < kvl) ? sc[n][e] * scale_log2 : -INFINITY;
                        mx[e >> 1] = fmaxf(mx[e >> 1], sc[n][e]);
                    }
                float alpha[2], muse[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                    const float mnew = fmaxf(m[i], mx[i]);
                    muse[i] = mnew == -INFINITY ? 0.f : mnew;
                    alpha[i] = exp2f(m[i] - muse[i]);
                    m[i] = mnew;
                    l[i] *= alpha[i];
                }
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                    o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
                }
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        sc[n][e] = exp2f(sc[n][e] - muse[e >> 1]);
                        l[e >> 1] += sc[n][e];
                    }
                unsigned pa[4];
                pa[0] = pack_bf16(sc[0][0], sc[0][1]);
                pa[1] = pack_bf16(sc[0][2], sc[0][3]);
                pa[2] = pack_bf16(sc[1][0], sc[1][1]);
                pa[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    unsigned vf[4];
                    ldmatrix_x4_trans(vf, swz(Vt, kw0 + (lane & 15), np * 16 + (lane >> 4) * 8));
                    mma_bf16(o[2 * np], pa, vf[0], vf[1]);
                    mma_bf16(o[2 * np + 1], pa, vf[2], vf[3]);
                }
            }
            __syncwarp();
            if (lane == 0) tbar_arrive(&empty[s]);             // this warp is done with the stage
            if (++s == TSTAGES) { s = 0; par ^= 1u; }
        }
    }
    __syncthreads();                                           // every stage is consumed, no copy is in flight

    // merge the warps' states through shared memory (the ring is free now)
    float* Os = reinterpret_cast<float*>(ring);                // [DWARPS][16][HD]
    float* Ms = Os + DWARPS * 16 * HD;                         // [DWARPS][16]
    float* Ls = Ms + DWARPS * 16;                              // [DWARPS][16]
    if (warp < DWARPS) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
            l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
            const int r = (lane >> 2) + 8 * i;
            float* orow = Os + ((size_t)warp * 16 + r) * HD + (lane & 3) * 2;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                orow[n * 8] = o[n][2 * i];
                orow[n * 8 + 1] = o[n][2 * i + 1];
            }
            if ((lane & 3) == 0) {
                Ms[warp * 16 + r] = m[i];
                Ls[warp * 16 + r] = l[i];
            }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < nheads * HD; idx += TTHREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DWARPS; ++w) M = fmaxf(M, Ms[w * 16 + r]);
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < DWARPS; ++w) {
                const float f = exp2f(Ms[w * 16 + r] - M);
                L += Ls[w * 16 + r] * f;
                O += Os[((size_t)w * 16 + r) * HD + d] * f;
            }
        }
        const int head = head0 + r;
        const float val = L > 0.f ? O / L : 0.f;
        if (splits == 1) {
            out[(size_t)tok * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(val);
        } else {
            const size_t p = ((size_t)slot * Hq + head) * splits + split;
            part_o[p * HD + d] = val;
            if (d == 0) part_lse[p] = L > 0.f ? M + log2f(L) : -INFINITY;
        }
    }
}
#endif

// out[token, head, :] = sum_s w_s * part_o[s] / sum_s w_s, w_s = 2^(lse_s - max lse)
__global__ void combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                               bf16* __restrict__ out, int out_stride, const int* __restrict__ cu_q,
                               const int* __restrict__ entry_list, int Hq, int splits) {
    // (which token this is was settled before the step's first kernel: read before the wait for
    // the partial results)
    pdl_trigger();
    const int slot = blockIdx.x, head = blockIdx.y;
    const int b = entry_list ? entry_list[slot] : slot;
    if (b < 0) return;
    const int tok = cu_q[b + 1] - 1;
    pdl_wait();
    const size_t p = ((size_t)slot * Hq + head) * splits;
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, part_lse[p + s]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float W = 0.f, O = 0.f;
        if (M != -INFINITY) {
            for (int s = 0; s < splits; ++s) {
                const float w = exp2f(part_lse[p + s] - M);
                W += w;
                O += w * part_o[(p + s) * HD + d];
            }
        }
        out[(size_t)tok * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(W > 0.f ? O / W : 0.f);
    }
}

constexpr size_t PREFILL_SMEM = ((size_t)MT * ROW + 4 * (size_t)KT * ROW) * sizeof(bf16);
constexpr size_t DECODE_SMEM_KV = 2 * (size_t)DSTAGES * DKT * ROW * sizeof(bf16);
constexpr size_t DECODE_SMEM_MERGE = (DWARPS * 16 * (size_t)HD + 2 * DWARPS * 16) * sizeof(float);
constexpr size_t DECODE_SMEM = 16 * (size_t)ROW * sizeof(bf16) +
                               (DECODE_SMEM_KV > DECODE_SMEM_MERGE ? DECODE_SMEM_KV : DECODE_SMEM_MERGE);

#if RI_HEAD_DIM == 64 || RI_HEAD_DIM == 128
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct TMapKey {
    const void* ptr; long long rows; int box_rows;
    bool operator==(const TMapKey& o) const { return ptr == o.ptr && rows == o.rows && box_rows == o.box_rows; }
};
struct TMapHash {
    size_t operator()(const TMapKey& k) const {
        return reinterpret_cast<size_t>(k.ptr) ^ ((size_t)k.rows * 0x9E3779B97F4A7C15ull) ^ ((size_t)k.box_rows << 50);
    }
};
// One layer of the cache, [page][K|V][kv head][slot][HD], seen as a matrix of HD-wide rows, in
// boxes of 64 columns x box_rows rows with the 128-byte swizzle.
int decode_cache_map(const void* ptr, long long rows, int box_rows, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<TMapKey, CUtensorMap, TMapHash> cache;
    static EncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    const TMapKey key{ptr, rows, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return (int)cudaErrorNotSupported;
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return (int)cudaErrorInvalidValue;
    if (cache.size() > 1024) cache.clear();
    cache.emplace(key, *out);
    return 0;
}
bool decode_tma_takes(int page_size) {
    static const bool off = getenv("RUSTINFER_B200_DECODE_ATTENTION") && !strcmp(getenv("RUSTINFER_B200_DECODE_ATTENTION"), "cp.async");
    return !off && DWARPS == 4 &&
           (page_size == 8 || page_size == 16 || page_size == 32 || (page_size > 0 && page_size % 64 == 0));
}
#endif

int configure() {
    static int status = -1;
    if (status < 0) {
        cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)PREFILL_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
#if RI_HEAD_DIM == 64 || RI_HEAD_DIM == 128
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_TMA_SMEM);
#endif
        status = (int)e;
    }
    return status;
}
}  // namespace

RI_API int ri_attention_mma_head_dim() { return HD; }
RI_API int ri_attention_decode_tile_keys() { return DKT; }
// CTAs of the decode kernel that fit one SM (by shared memory), for the choice of key ranges
RI_API int ri_attention_decode_ctas_per_sm() {
    const int by_smem = (int)((227 * 1024) / (DECODE_SMEM + 1024));
    const int by_threads = 2048 / DTHREADS;
    return by_smem < by_threads ? (by_smem < 1 ? 1 : by_smem) : by_threads;
}
// ... of the kernel that fetches keys and values by TMA (0: not built for this head size)
RI_API int ri_attention_decode_tma_ctas_per_sm(int page_size) {
#if RI_HEAD_DIM == 64 || RI_HEAD_DIM == 128
    if (!decode_tma_takes(page_size)) return 0;
    const int by_smem = (int)((227 * 1024) / (DECODE_TMA_SMEM + 1024));
    const int by_threads = 2048 / TTHREADS;
    return by_smem < by_threads ? (by_smem < 1 ? 1 : by_smem) : by_threads;
#else
    return 0;
#endif
}

// Tokens per prefill tile for a model with `group` q heads per kv head: 64 rows hold
// 64 / min(group, 64) tokens of min(group, 64) heads each.
RI_API int ri_attention_mma_tokens_per_tile(int group) {
    const int gc = group < MT ? group : MT;
    return MT / gc;
}

RI_API int ri_attention_prefill_bf16(const void* q, int q_stride, void* out, int out_stride,
                                     const void* cache, const int* block_table, int table_stride,
                                     const int* cu_q, const int* kv_len, const int* tile_entry,
                                     const int* tile_tok0, int n_tiles, int Hq, int Hkv, int page_size,
                                     float scale, int window, void* stream) {
    if (n_tiles <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv != 0) return (int)cudaErrorInvalidValue;
    int st = configure();
    if (st != 0) return st;
    const int G = Hq / Hkv, Gc = G < MT ? G : MT, chunks = (G + Gc - 1) / Gc, tpt = MT / Gc;
    dim3 grid(n_tiles, Hkv * chunks);
    RI_CHECKED(ri_launch(prefill_kernel, dim3(grid), dim3(THREADS), PREFILL_SMEM, (cudaStream_t)stream, 
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)cache, block_table, table_stride,
        cu_q, kv_len, tile_entry, tile_tok0, Hq, Hkv, Gc, chunks, tpt, page_size,
        scale * 1.4426950408889634f, window));
    return ri_launch_status();
}

// Scratch for `splits` > 1: part_o holds entries*Hq*splits*HD floats, part_lse entries*Hq*splits.
// With `merge` 0 and several key ranges the partial results are left there for the caller to merge
// (the chained products do it while they lay out their first operand) and `out` is not written.
RI_API int ri_attention_decode_bf16(const void* q, int q_stride, void* out, int out_stride,
                                    const void* cache, const int* block_table, int table_stride,
                                    const int* cu_q, const int* kv_len, const int* entry_list,
                                    int n_entries, int Hq, int Hkv, int page_size, float scale, int window,
                                    int splits, float* part_o, float* part_lse, long long n_pages, int* error,
                                    int merge, void* stream) {
    if (n_entries <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv != 0 || splits < 1 || (splits > 1 && (!part_o || !part_lse)))
        return (int)cudaErrorInvalidValue;
    int st = configure();
    if (st != 0) return st;
    const int G = Hq / Hkv, Gc = G < 16 ? G : 16, chunks = (G + Gc - 1) / Gc;
    dim3 grid(Hkv * chunks, splits, n_entries);
    cudaStream_t s = (cudaStream_t)stream;
#if RI_HEAD_DIM == 64 || RI_HEAD_DIM == 128
    // with the cache's size and an error flag at hand, keys and values come by TMA
    if (n_pages > 0 && error && decode_tma_takes(page_size) && (reinterpret_cast<uintptr_t>(cache) & 15) == 0) {
        const int box_rows = page_size < DKT ? page_size : DKT;
        CUtensorMap map;
        st = decode_cache_map(cache, n_pages * 2 * Hkv * page_size, box_rows, &map);
        if (st != 0) return st;
        RI_CHECKED(ri_launch(decode_tma_kernel, dim3(grid), dim3(TTHREADS), DECODE_TMA_SMEM, s, map,
            (const bf16*)q, q_stride, (bf16*)out, out_stride, block_table, table_stride, cu_q, kv_len, entry_list,
            Hq, Hkv, Gc, chunks, page_size, box_rows, scale * 1.4426950408889634f, window, splits, part_o, part_lse, error));
        st = ri_launch_status();
        if (st != 0 || splits == 1 || !merge) return st;
        RI_CHECKED(ri_launch(combine_kernel, dim3(dim3(n_entries, Hq)), dim3(HD < 128 ? 64 : 128), 0, s,
            part_o, part_lse, (bf16*)out, out_stride, cu_q, entry_list, Hq, splits));
        return ri_launch_status();
    }
#endif
    RI_CHECKED(ri_launch(decode_kernel, dim3(grid), dim3(DTHREADS), DECODE_SMEM, s, 
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)cache, block_table, table_stride,
        cu_q, kv_len, entry_list, Hq, Hkv, Gc, chunks, page_size, scale * 1.4426950408889634f, window,
        splits, part_o, part_lse));
    st = ri_launch_status();
    if (st != 0 || splits == 1 || !merge) return st;
    RI_CHECKED(ri_launch(combine_kernel, dim3(dim3(n_entries, Hq)), dim3(HD < 128 ? 64 : 128), 0, s, 
        part_o, part_lse, (bf16*)out, out_stride, cu_q, entry_list, Hq, splits));
    return ri_launch_status();
}

// ===================================================== decode without an allocator
// See attention_decode_static.h: the same two kernels as ri_attention_decode_bf16, with
// the split partials in an array that lives inside this library.
#include "attention_decode_static.h"
#include <stdio.h>

namespace {
static __device__ __align__(256) float g_decode_static_scratch[RI_DECODE_STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
// Device address of the array per device; in host code the array's name is only a handle
// for cudaGetSymbolAddress, never a pointer a kernel could be given.
float* g_decode_static_ptr[MAX_DEVICES] = {nullptr};
thread_local char g_decode_static_msg[256] = "";

int decode_static_setup(int device, float** ptr) {
    // two host threads may make a device's first call at once: the look-up runs under a lock
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (g_decode_static_ptr[device] == nullptr) {
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_decode_static_scratch);
        if (e != cudaSuccess) {
            snprintf(g_decode_static_msg, sizeof g_decode_static_msg,
                     "cudaGetSymbolAddress for the static scratch failed: %s", cudaGetErrorString(e));
            return (int)e;
        }
        e = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
        if (e != cudaSuccess) {
            snprintf(g_decode_static_msg, sizeof g_decode_static_msg,
                     "raising the decode kernel's shared-memory limit failed: %s", cudaGetErrorString(e));
            return (int)e;
        }
        g_decode_static_ptr[device] = p;
    }
    *ptr = g_decode_static_ptr[device];
    return 0;
}
}  // namespace

const char* ri_attention_decode_static_error(void) { return g_decode_static_msg; }

int ri_attention_decode_bf16_static(const void* q, int q_stride, void* out, int out_stride,
                                    const void* cache, const int* block_table, int table_stride,
                                    const int* cu_q, const int* kv_len, const int* entry_list,
                                    int n_entries, int Hq, int Hkv, int page_size, float scale,
                                    int window, int splits, void* stream) {
    g_decode_static_msg[0] = 0;
    if (n_entries <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv != 0 || splits < 1) {
        snprintf(g_decode_static_msg, sizeof g_decode_static_msg,
                 "bad sizes: q heads %d, kv heads %d, splits %d", Hq, Hkv, splits);
        return (int)cudaErrorInvalidValue;
    }
    const long long need = (long long)n_entries * Hq * splits * (HD + 1);
    if (need > (long long)RI_DECODE_STATIC_SCRATCH_FLOATS) {
        snprintf(g_decode_static_msg, sizeof g_decode_static_msg,
                 "entries %d x q heads %d x splits %d x (head_dim %d + 1) = %lld floats exceed the static "
                 "scratch of %d floats; use fewer splits or entries, or ri_attention_decode_bf16 with "
                 "scratch of your own", n_entries, Hq, splits, HD, need, RI_DECODE_STATIC_SCRATCH_FLOATS);
        return (int)cudaErrorInvalidValue;
    }
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
        snprintf(g_decode_static_msg, sizeof g_decode_static_msg, "no usable current device (%d)", device);
        return (int)(e != cudaSuccess ? e : cudaErrorInvalidDevice);
    }
    float* scratch = nullptr;
    int st = decode_static_setup(device, &scratch);
    if (st != 0) return st;
    float* part_o = scratch;                                               // [entries][Hq][splits][HD]
    float* part_lse = scratch + (size_t)n_entries * Hq * splits * HD;      // [entries][Hq][splits]
    const int G = Hq / Hkv, Gc = G < 16 ? G : 16, chunks = (G + Gc - 1) / Gc;
    dim3 grid(Hkv * chunks, splits, n_entries);
    cudaStream_t s = (cudaStream_t)stream;
    RI_CHECKED(ri_launch(decode_kernel, dim3(grid), dim3(DTHREADS), DECODE_SMEM, s, 
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)cache, block_table, table_stride,
        cu_q, kv_len, entry_list, Hq, Hkv, Gc, chunks, page_size, scale * 1.4426950408889634f, window,
        splits, part_o, part_lse));
    st = ri_launch_status();
    if (st != 0 || splits == 1) return st;
    RI_CHECKED(ri_launch(combine_kernel, dim3(dim3(n_entries, Hq)), dim3(HD < 128 ? 64 : 128), 0, s, 
        part_o, part_lse, (bf16*)out, out_stride, cu_q, entry_list, Hq, splits));
    return ri_launch_status();
}

RI_API void ri_set_pdl(int on) { ri_pdl_flag() = on ? 1 : 0; }
