// A chain of few-token products in ONE kernel: out_i (+)= f_i(x_i) W_i^T for i = 0..n-1, each
// reading what the one before wrote, optionally followed by the rotary encoding and the
// write of keys and values into the paged cache.  One decode step of a pre-norm decoder is
// then three launches a layer (this chain, attention over the cache, its combine) instead of
// nine, and the weights of all products stream through one ring of shared memory without a
// pause at the seams: the TMA producer of a CTA runs ahead into the next product while the
// others wait at the grid barrier between two products.
//
// RustInfer runs these as separate cuBLASLt / GEMV, RMSNorm, RoPE, SwiGLU and add kernels
// (crates/infer-worker/src/components/decoder_block.rs:13-32 over attention.rs, ffn_dense.rs,
// norm.rs); the arithmetic here is the same, the fusion is this engine's own.
//
//   warp 0      TMA producer: weight tiles [a_box rows x 64] of every product, in order
//   warp 1      tensor memory; one thread issues tcgen05.mma (A = weight tile, B = activations)
//   warps 2-5   make the activation operand in shared memory (bf16 copy, or the fp32 stream
//               times a norm weight; the RMS scale is applied to the accumulator instead, so
//               the sum of squares is computed while the weights stream), read the
//               accumulator back, run the epilogue, and meet the other CTAs at the barrier
//
// Products whose output is added into an fp32 buffer may be cut along K (every slice adds its
// part with red.global.add); the others are cut along N only.  A grid barrier separates two
// products; the kernel is launched cooperatively with one CTA per SM, so all CTAs are
// resident.  Every wait (mbarrier or grid barrier) is bounded: on a time-out the kernel
// records a code in *error, stops issuing work, drains its copies, frees its tensor memory
// and returns (the output is then meaningless and the host raises).
#include "common.cuh"
#include "tc_primitives.cuh"
#include <cuda.h>

#include "decode_chain_api.h"

namespace {
using namespace ri_tc;
constexpr int BM = 128, BK = 64, THREADS = 192;
constexpr int SUB_BYTES = BM * BK * 2;         // one 64-column tile of 128 weight rows: 16 KB, whatever a_box is
constexpr int SUBS = 2;                        // tiles per ring stage: one wait and one commit serve 8 MMAs
constexpr int STAGE_BYTES = SUBS * SUB_BYTES;
constexpr int KSTEP = SUBS * BK;               // K columns per stage
constexpr int MAX_PHASES = 6, MAX_STAGES = 6;
constexpr int HEAD_BYTES = 1024;               // barriers and row scales in front of the ring
constexpr int ROW_STAGE_BYTES = 64 * 1024;     // most bytes of fp32 stream rows staged at a time
constexpr int SMEM_LIMIT = 225 * 1024;

enum XKind { X_BF16 = 0, X_NORM = 1, X_PARTIALS = 2 };
enum OutKind { OUT_ADD_F32 = 0, OUT_SILU_BF16 = 1, OUT_BF16 = 2 };
enum ErrorCode { ERR_CHAIN_PRODUCER = 11, ERR_CHAIN_MMA = 12, ERR_CHAIN_EPILOGUE = 13, ERR_CHAIN_GRID = 14 };

struct Phase {
    int N, K;                   // weight [N][K]
    int a_box, tiles, splits, per;   // weight rows per tile, tiles along N, K slices, stages (KSTEP columns) per slice
    int x_kind, ld_x;
    const void* x;              // X_BF16: bf16 [M][ld_x];  X_NORM: fp32 [M][ld_x];  X_PARTIALS: fp32 partial attention outputs
    const float* part_lse;      // X_PARTIALS: log-sum-exps of the key ranges
    int part_splits, part_heads, part_hd;
    const void* norm_w;         // X_NORM: [K]
    int norm_w_bf16;
    float eps;
    int out_kind, ld_out;
    void* out;
};

struct Rope {
    int enabled;
    float* qkv;                 // fp32 [M][ld]: q heads, k heads, v heads; zeroed again after use
    int ld;
    const int* positions;
    const float* cos_t;         // [positions][rot/2]
    const float* sin_t;
    const int* slot_of_token;   // flat slot in the paged cache, -1: no write
    bf16* q_out;                // [M][ld_q]
    int ld_q;
    bf16* cache;                // [page][K|V][kv head][slot][hd]
    int Hq, Hkv, hd, rot, page_size;
};

struct Params {
    int M, n_phases, stages, xs_off;
    int x_kb_bytes;             // bytes of one 64-column block of the activation operand (1024 when rows 8..15 alias rows 0..7)
    int stage_off, stage_rows;  // where rows of the fp32 stream are staged, and how many at a time
    int nw_off;                 // where the norm weight is staged
    Phase ph[MAX_PHASES];
    Rope rope;
    unsigned* grid_bar;         // [0] arrivals, [1] exits; zero between launches
    int* error;
};

struct Maps { CUtensorMap m[MAX_PHASES]; CUtensorMap x[MAX_PHASES]; };   // weights; bf16 activation matrices

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void bulk_load(void* smem, const void* g, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem)), "l"(g), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld4(unsigned addr, float (&v)[4]) {
    unsigned r[4];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}

// All CTAs have arrived `target` times in total.  One thread spins (bounded).
__device__ __forceinline__ bool grid_wait(const unsigned* bar, unsigned target, int* error) {
#pragma unroll 1
    for (unsigned i = 0; i < SPIN_LIMIT; ++i) {
        if (ld_acquire(bar) >= target) return true;
        if (i > 64) __nanosleep(32);
    }
    atomicExch(error, ERR_CHAIN_GRID);
    return false;
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
decode_chain_kernel(const __grid_constant__ Maps maps, const __grid_constant__ Params p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(base);          // [MAX_STAGES]
    uint64_t* empty = full + MAX_STAGES;                         // [MAX_STAGES]
    uint64_t* x_ready = empty + MAX_STAGES;
    uint64_t* acc_full = x_ready + 1;
    uint64_t* x_land = acc_full + 1;                              // TMA copies of activations have landed
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(x_land + 1);
    unsigned* go_slot = tmem_slot + 1;                            // 1 while the grid barriers hold
    float* row_scale = reinterpret_cast<float*>(base + 384);     // [BN]
    unsigned char* ring = base + HEAD_BYTES;
    unsigned char* xs = base + p.xs_off;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, STAGES = p.stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(x_ready, 4);
        mbar_init(acc_full, 1);
        mbar_init(x_land, 1);
        *go_slot = 1;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        // Weights are written by no kernel, so none of these loads waits for anything but a
        // free stage: the ring runs ahead of the barriers, into the products that follow.
        pdl_trigger();
        bool ok = true;
        int it = 0;
        for (int ph = 0; ph < p.n_phases && ok; ++ph) {
            const Phase& P = p.ph[ph];
            // (copied out: a field read through P inside the loop is fetched from the parameter bank each time)
            const int a_box = P.a_box, tiles = P.tiles, items = P.tiles * P.splits, per = P.per;
            const int kblocks = (P.K + KSTEP - 1) / KSTEP;
            const unsigned tx = (unsigned)a_box * BK * 2 * SUBS;       // a box past the last column still counts, as zeros
            const CUtensorMap* wmap = &maps.m[ph];
            for (int item = blockIdx.x; item < items && ok; item += G) {
                const int tile = item % tiles, kb0 = (item / tiles) * per;
                const int n_kb = min(per, kblocks - kb0);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES, round = it / STAGES;
                    if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, p.error, ERR_CHAIN_PRODUCER)) { ok = false; break; }
                    mbar_expect_tx(&full[s], tx);
#pragma unroll
                    for (int h = 0; h < SUBS; ++h)
                        tma_load_2d(ring + (size_t)s * STAGE_BYTES + h * SUB_BYTES, wmap, &full[s],
                                    (kb0 + i) * KSTEP + h * BK, tile * a_box);
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
        // one scalar thread feeds the tensor core: descriptors are made once and stepped by adds,
        // the ring position is counted, not divided
        // with at most 8 tokens the second group of 8 rows of the operand is the first one again
        // (group stride 0), which halves the activation region
        const uint64_t desc_ring = smem_desc(smem_u32(ring));
        const uint64_t desc_xs = p.x_kb_bytes == 1024 ? (smem_desc(smem_u32(xs)) & ~(0x3fffull << 32)) : smem_desc(smem_u32(xs));
        const unsigned x_step = (unsigned)p.x_kb_bytes >> 4;
        bool ok = true;
        int s = 0, n = 0;
        unsigned par = 0;
        for (int ph = 0; ph < p.n_phases && ok; ++ph) {
            const Phase& P = p.ph[ph];
            const int kblocks = (P.K + KSTEP - 1) / KSTEP;
            for (int item = blockIdx.x; item < P.tiles * P.splits && ok; item += G, ++n) {
                const int n_kb = min(P.per, kblocks - (item / P.tiles) * P.per);
                // the activations of this item are in place, and the accumulator has been read
                if (!mbar_wait(x_ready, n & 1, p.error, ERR_CHAIN_MMA)) { ok = false; break; }
                tc_fence_after();
                uint64_t db = desc_xs;
                for (int i = 0; i < n_kb; ++i) {
                    if (!mbar_try_wait(&full[s], par) && !mbar_wait(&full[s], par, p.error, ERR_CHAIN_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t da = desc_ring + (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
                    for (int h = 0; h < SUBS; ++h)
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            mma_bf16_ss(tmem_base, da + (uint64_t)(h * (SUB_BYTES >> 4) + k * 2),
                                        db + (uint64_t)(h * x_step + k * 2), idesc, (i > 0 || h > 0 || k > 0) ? 1u : 0u);
                    tc_commit(&empty[s]);
                    db += (uint64_t)(SUBS * x_step);
                    if (++s == STAGES) { s = 0; par ^= 1u; }
                }
                if (ok) tc_commit(acc_full);
            }
        }
        if (!ok) {
            // what was loaded last must have landed before shared memory is given up
            for (int s = 0; s < STAGES; ++s)
                for (int par = 0; par < 2; ++par)
                    if (mbar_try_wait(&full[s], par)) break;
#pragma unroll 1
            for (unsigned spin = 0; spin < 4096; ++spin) __nanosleep(256);
        }
    } else if (warp >= 2) {
        // ------------------------------------------------- activations, epilogue, barrier
        const int quarter = warp & 3;                     // the 32 TMEM lanes this warp may read
        const int te = threadIdx.x - 64, M = p.M;
        const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16);
        bool ok = true;
        int n = 0, xl = 0;                                // items done; TMA batches of activations landed
        pdl_wait();                                       // everything but the weights belongs to earlier kernels till now
        for (int ph = 0; ph < p.n_phases; ++ph) {
            const Phase& P = p.ph[ph];
            const int kblocks = (P.K + KSTEP - 1) / KSTEP;
            if (ph > 0) {
                // what the product before wrote is complete on every CTA
                if (threadIdx.x == 64 && *go_slot && !grid_wait(p.grid_bar, (unsigned)G * ph, p.error)) *go_slot = 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                ok = ok && *go_slot;
            }
            bool nw_here = false;                             // this product's norm weight is staged
            for (int item = blockIdx.x; item < P.tiles * P.splits; item += G, ++n) {
                const int tile = item % P.tiles, st0 = (item / P.tiles) * P.per;
                const int kb0 = st0 * SUBS, n_kb = min(P.per, kblocks - st0) * SUBS;   // in 64-column blocks
                if (!ok) continue;
                // ---- the activation operand of this K slice, in the layout the tensor core
                // reads: 64-column blocks of 128-byte rows, 16-byte chunk c of row r at c ^ (r & 7).
                // This code runs once per product and launch, from a cold instruction cache and
                // against a full weight stream, where each trip to L2 takes well over a microsecond:
                // the copies are TMA's (one thread issues them), the loops are short and rolled.
                if (threadIdx.x == 64) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                if (P.x_kind == X_BF16) {
                    if (threadIdx.x == 64) {
                        mbar_expect_tx(x_land, (unsigned)(n_kb * p.x_kb_bytes));
                        for (int kbl = 0; kbl < n_kb; ++kbl)
                            tma_load_2d(xs + (size_t)kbl * p.x_kb_bytes, &maps.x[ph], x_land, (kb0 + kbl) * BK, 0);
                    }
                    ok = mbar_wait(x_land, xl & 1, p.error, ERR_CHAIN_EPILOGUE);
                    ++xl;
                } else if (P.x_kind == X_PARTIALS) {
                    // the attention before this chain left one partial output per key range: the
                    // operand's element (token r, head h, dim d) is their merge,
                    // sum_s 2^(lse_s - max) part_s / sum_s 2^(lse_s - max), formed here instead of
                    // by a kernel of its own (16 bytes of the operand a thread and turn)
                    const float* po = reinterpret_cast<const float*>(P.x);
                    const float* pl = P.part_lse;
                    const int S = P.part_splits, hd = P.part_hd, Hq = P.part_heads, Kc = P.K, x_kb_bytes = p.x_kb_bytes;
                    const int cpr = n_kb * (BK >> 3);                       // 16-byte chunks of a row in this K slice
                    for (int idx = te; idx < M * cpr; idx += 128) {
                        const int r = idx / cpr, c = idx - r * cpr;
                        const int k = kb0 * BK + c * 8;
                        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                        if (k < Kc) {
                            const int h = k / hd, d = k - h * hd;
                            const size_t at = ((size_t)r * Hq + h) * S;
                            float mx = -INFINITY;
                            for (int s = 0; s < S; ++s) mx = fmaxf(mx, pl[at + s]);
                            float W = 0.f;
                            if (mx != -INFINITY) {
                                for (int s = 0; s < S; ++s) {
                                    const float w = exp2f(pl[at + s] - mx);
                                    const float4 a = *reinterpret_cast<const float4*>(po + (at + s) * hd + d);
                                    const float4 b = *reinterpret_cast<const float4*>(po + (at + s) * hd + d + 4);
                                    W += w;
                                    acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * a.z; acc[3] += w * a.w;
                                    acc[4] += w * b.x; acc[5] += w * b.y; acc[6] += w * b.z; acc[7] += w * b.w;
                                }
                            }
                            const float inv = W > 0.f ? 1.f / W : 0.f;
#pragma unroll
                            for (int e = 0; e < 8; ++e) acc[e] *= inv;
                        }
                        *reinterpret_cast<uint4*>(xs + (size_t)(c >> 3) * x_kb_bytes + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = pack8(acc);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                } else {
                    // rows of the fp32 stream are staged whole: the sum of squares needs all of a
                    // row, the operand only this slice of it, times the norm weight (the RMS scale
                    // is applied to the accumulator later).  A warp owns a row.
                    const float* hs = reinterpret_cast<const float*>(P.x);
                    float* stg = reinterpret_cast<float*>(base + p.stage_off);
                    unsigned char* nws = base + p.nw_off;
                    const int upr = P.K >> 3;                               // units of 8 floats in a row
                    const int k_lo = kb0 * BK, k_hi = (kb0 + n_kb) * BK;
                    const int Kc = P.K, x_kb_bytes = p.x_kb_bytes;
                    const bool nw_bf16 = P.norm_w_bf16 != 0;
                    const float eps = P.eps;
                    const unsigned nw_bytes = (unsigned)Kc * (nw_bf16 ? 2u : 4u);
                    for (int r0 = 0; r0 < M && ok; r0 += p.stage_rows) {
                        const int rows = min(p.stage_rows, M - r0);
                        if (warp == 2) {
                            // a row's copy from a lane of its own (one thread sends a copy every 74 ns; nine
                            // from one thread were 0.7 us of each of the chain's two stagings)
                            if (lane == 0) mbar_expect_tx(x_land, (unsigned)rows * P.K * 4u + (nw_here ? 0u : nw_bytes));
                            __syncwarp();
                            if (lane < rows)
                                bulk_load(stg + (size_t)lane * P.K, hs + (size_t)(r0 + lane) * P.ld_x, (unsigned)P.K * 4u, x_land);
                            else if (lane == rows && !nw_here)
                                bulk_load(nws, P.norm_w, nw_bytes, x_land);
                        }
                        nw_here = true;
                        ok = mbar_wait(x_land, xl & 1, p.error, ERR_CHAIN_EPILOGUE);
                        ++xl;
                        // a warp norms rows quarter, quarter + 4, ... two at a time: the norm weight is
                        // read and widened once for both, and the loads of one row do not wait for the
                        // arithmetic of the other
                        for (int r = quarter; r < rows && ok; r += 8) {
                            const bool two = r + 4 < rows;
                            const float* row_a = stg + (size_t)r * Kc;
                            const float* row_b = stg + (size_t)(two ? r + 4 : r) * Kc;
                            const int ra = r0 + r, rb = ra + 4;
                            float ss_a = 0.f, ss_b = 0.f;
#pragma unroll 2
                            for (int u = lane; u < upr; u += 32) {
                                const int k = u * 8;
                                const float4 a0 = *reinterpret_cast<const float4*>(row_a + k);
                                const float4 a1 = *reinterpret_cast<const float4*>(row_a + k + 4);
                                const float4 b0 = *reinterpret_cast<const float4*>(row_b + k);
                                const float4 b1 = *reinterpret_cast<const float4*>(row_b + k + 4);
                                ss_a += (a0.x * a0.x + a0.y * a0.y) + (a0.z * a0.z + a0.w * a0.w)
                                      + (a1.x * a1.x + a1.y * a1.y) + (a1.z * a1.z + a1.w * a1.w);
                                ss_b += (b0.x * b0.x + b0.y * b0.y) + (b0.z * b0.z + b0.w * b0.w)
                                      + (b1.x * b1.x + b1.y * b1.y) + (b1.z * b1.z + b1.w * b1.w);
                                if (k >= k_lo && k < k_hi) {
                                    float w[8];
                                    if (nw_bf16) {
                                        const uint4 wv = *reinterpret_cast<const uint4*>(nws + (size_t)k * 2);
                                        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                                        for (int e = 0; e < 4; ++e) {
                                            const float2 f = __bfloat1622float2(wp[e]);
                                            w[2 * e] = f.x; w[2 * e + 1] = f.y;
                                        }
                                    } else {
                                        const float4 wa = *reinterpret_cast<const float4*>(nws + (size_t)k * 4);
                                        const float4 wb = *reinterpret_cast<const float4*>(nws + (size_t)k * 4 + 16);
                                        w[0] = wa.x; w[1] = wa.y; w[2] = wa.z; w[3] = wa.w; w[4] = wb.x; w[5] = wb.y; w[6] = wb.z; w[7] = wb.w;
                                    }
                                    unsigned char* dst = xs + (size_t)((k >> 6) - kb0) * x_kb_bytes;
                                    float x[8];
                                    x[0] = a0.x * w[0]; x[1] = a0.y * w[1]; x[2] = a0.z * w[2]; x[3] = a0.w * w[3];
                                    x[4] = a1.x * w[4]; x[5] = a1.y * w[5]; x[6] = a1.z * w[6]; x[7] = a1.w * w[7];
                                    *reinterpret_cast<uint4*>(dst + ra * 128 + (((u & 7) ^ (ra & 7)) << 4)) = pack8(x);
                                    if (two) {
                                        x[0] = b0.x * w[0]; x[1] = b0.y * w[1]; x[2] = b0.z * w[2]; x[3] = b0.w * w[3];
                                        x[4] = b1.x * w[4]; x[5] = b1.y * w[5]; x[6] = b1.z * w[6]; x[7] = b1.w * w[7];
                                        *reinterpret_cast<uint4*>(dst + rb * 128 + (((u & 7) ^ (rb & 7)) << 4)) = pack8(x);
                                    }
                                }
                            }
                            ss_a = warp_sum(ss_a);
                            ss_b = warp_sum(ss_b);
                            if (lane == 0) {
                                row_scale[ra] = rsqrtf(ss_a / (float)Kc + eps);
                                if (two) row_scale[rb] = rsqrtf(ss_b / (float)Kc + eps);
                            }
                        }
                        // the staged rows may be overwritten, the scales are there for all warps
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (threadIdx.x == 64) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    }
                    // columns of the last stage that lie beyond K meet zero weights: they must not be NaN
                    for (int u = max(upr, k_lo >> 3) + te; u < (k_hi >> 3); u += 128)
                        for (int r = 0; r < M; ++r)
                            *reinterpret_cast<uint4*>(xs + (size_t)((u >> 3) - kb0) * p.x_kb_bytes + r * 128 + (((u & 7) ^ (r & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(x_ready);
                // ---- the accumulator: lanes are weight rows (features), columns are tokens
                if (ok) ok = mbar_wait(acc_full, n & 1, p.error, ERR_CHAIN_EPILOGUE);
                tc_fence_after();
                const int fl = quarter * 32 + lane;
                const int feat = fl < P.a_box ? tile * P.a_box + fl : 0x3fffffff;
                // The lane's whole row (one feature, every token) comes out of tensor memory in one
                // round trip.  The product's numbers go into registers first: read through `P`
                // inside the loops they are fetched from the parameter bank again after every asm
                // statement, which made a token cost 270 cycles.
                const int out_kind = P.out_kind, ld_out = P.ld_out;
                const bool scaled = P.x_kind == X_NORM, live = feat < P.N;
                void* const out = P.out;
                float v[16];
                static_assert(BN == 16, "the epilogue reads 16 columns");
                if (ok) {
                    tmem_ld16(taddr, v);
                    if (scaled) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] *= row_scale[j];
                    }
                    if (out_kind == OUT_ADD_F32) {
                        float* o = reinterpret_cast<float*>(out) + (live ? feat : 0);
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < M && live) atomicAdd(o + (size_t)j * ld_out, v[j]);
                    } else if (out_kind == OUT_BF16) {
                        bf16* o = reinterpret_cast<bf16*>(out) + (live ? feat : 0);
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < M && live) o[(size_t)j * ld_out] = __float2bfloat16_rn(v[j]);
                    } else {
                        // rows of the weight alternate gate_j, up_j: an even lane holds the gate and
                        // its neighbour the up value of the same feature.  Of two tokens the even
                        // lane finishes the first and the odd lane the second, so every lane does
                        // one SiLU and one store per pair after one exchange.
                        bf16* o = reinterpret_cast<bf16*>(out) + (live ? (feat >> 1) : 0);
                        const bool odd = (lane & 1) != 0;
#pragma unroll
                        for (int j = 0; j < 16; j += 2) {
                            const float got = __shfl_xor_sync(0xffffffffu, odd ? v[j] : v[j + 1], 1);
                            const float g = odd ? got : v[j], u = odd ? v[j + 1] : got;
                            const int tok = j + (odd ? 1 : 0);
                            if (tok < M && live) o[(size_t)tok * ld_out] = __float2bfloat16_rn(silu_mul(g, u));
                        }
                    }
                }
                tc_fence_before();
                asm volatile("bar.sync 1, 128;" ::: "memory");     // row_scale and the accumulator are free again
            }
            // this CTA's part of the product is written
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) atomicAdd(p.grid_bar, 1u);
        }
        if (p.rope.enabled) {
            // ---------------- rotary encoding of q and k, keys and values into their pages
            const Rope& R = p.rope;
            const int heads = R.Hq + 2 * R.Hkv, half = R.rot >> 1;
            const size_t head_step = (size_t)R.page_size * R.hd;
            // What the warp's first row needs besides the product (its position, its place in the
            // cache, its angles) is fetched before the wait for the product: two trips to L2 that
            // run beside the barrier instead of after it.
            const int wi0 = blockIdx.x * 4 + quarter;
            int t0 = 0, slot0 = -1, pos0 = 0;
            float c0 = 1.f, s0 = 0.f;
            if (wi0 < M * heads) {
                t0 = wi0 / heads;
                slot0 = R.slot_of_token ? R.slot_of_token[t0] : -1;
                if (wi0 - t0 * heads < R.Hq + R.Hkv) {
                    pos0 = R.positions[t0];
                    if (lane < half) { c0 = R.cos_t[(size_t)pos0 * half + lane]; s0 = R.sin_t[(size_t)pos0 * half + lane]; }
                }
            }
            if (threadIdx.x == 64 && *go_slot && !grid_wait(p.grid_bar, (unsigned)G * p.n_phases, p.error)) *go_slot = 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            ok = ok && *go_slot;
            for (int wi = wi0; wi < M * heads && ok; wi += G * 4) {
                const bool first = wi == wi0;
                const int t = first ? t0 : wi / heads, hh = wi - t * heads;
                float* src = R.qkv + (size_t)t * R.ld + (size_t)hh * R.hd;
                const int slot = first ? slot0 : (R.slot_of_token ? R.slot_of_token[t] : -1);
                bf16* dst = nullptr;
                if (hh < R.Hq) {
                    dst = R.q_out + (size_t)t * R.ld_q + (size_t)hh * R.hd;
                } else if (slot >= 0 && R.cache) {
                    const int page = slot / R.page_size, off = slot - page * R.page_size;
                    const int kv = hh < R.Hq + R.Hkv ? 0 : 1, g = hh - R.Hq - kv * R.Hkv;
                    dst = R.cache + ((size_t)(page * 2 + kv) * R.Hkv * R.page_size + off) * R.hd + (size_t)g * head_step;
                }
                if (hh < R.Hq + R.Hkv) {
                    const int pos = first ? pos0 : R.positions[t];
                    const float* ct = R.cos_t + (size_t)pos * half;
                    const float* st = R.sin_t + (size_t)pos * half;
                    for (int j = lane; j < half; j += 32) {
                        const float x1 = __ldcg(src + j), x2 = __ldcg(src + j + half);
                        const bool have = first && j == lane;
                        const float c = have ? c0 : ct[j], s = have ? s0 : st[j];
                        if (dst) {
                            dst[j] = __float2bfloat16_rn(x1 * c - x2 * s);
                            dst[j + half] = __float2bfloat16_rn(x1 * s + x2 * c);
                        }
                    }
                    for (int j = R.rot + lane; j < R.hd; j += 32)
                        if (dst) dst[j] = __float2bfloat16_rn(__ldcg(src + j));
                } else {
                    for (int j = lane; j < R.hd; j += 32)
                        if (dst) dst[j] = __float2bfloat16_rn(__ldcg(src + j));
                }
                __syncwarp();
                for (int j = lane; j < R.hd; j += 32) src[j] = 0.f;      // the next chain adds into zeros
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0) {
        // the last CTA to leave puts the barrier back to zero for the next launch
        __threadfence();
        if (atomicAdd(p.grid_bar + 1, 1u) == (unsigned)G - 1) {
            p.grid_bar[0] = 0u;
            p.grid_bar[1] = 0u;
            __threadfence();
        }
    }
}

int round_up(int a, int b) { return (a + b - 1) / b * b; }

template <int BN>
int launch_chain(const Maps& maps, const Params& p, int grid, size_t smem, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_chain_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    // cooperative: the driver refuses the launch unless all CTAs can be resident together,
    // which the grid barrier needs.  (Launched with programmatic dependent launch instead, the
    // kernel starts during its predecessor's tail but the step is no faster: measured.)
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, decode_chain_kernel<BN>, maps, p);
}
}  // namespace

namespace {
// Where everything lies in shared memory for a chain of these products and M tokens; false
// if it does not fit.  [head | ring of weight stages | activation operand | staged rows | norm weight]
struct Layout { int bn, x_kb_bytes, xs_bytes, stage_rows, stage_bytes, nw_bytes, stages; };

bool plan_phase(const RiChainPhase& f, int sms, int* a_box, int* tiles, int* splits, int* per) {
    if (f.N < 1 || f.K < 8 || f.K % 8) return false;
    const int kblocks = (f.K + KSTEP - 1) / KSTEP, tiles128 = (f.N + BM - 1) / BM;
    if (f.out_kind == OUT_ADD_F32) {
        *a_box = BM; *tiles = tiles128;
        const int want = max(1, min(kblocks, sms / tiles128));
        *per = (kblocks + want - 1) / want;
        *splits = (kblocks + *per - 1) / *per;
    } else {
        // cut along N only, into a whole number of waves of nearly equal tiles
        const int waves = (tiles128 + sms - 1) / sms;
        *a_box = min(BM, round_up((f.N + waves * sms - 1) / (waves * sms), 16));
        *tiles = (f.N + *a_box - 1) / *a_box;
        *splits = 1; *per = kblocks;
    }
    return true;
}

bool plan_layout(const RiChainPhase* phases, int n_phases, int M, int sms, Layout* L) {
    if (n_phases < 1 || n_phases > MAX_PHASES || M < 1 || M > 16 || sms < 1) return false;
    L->bn = M <= 16 ? 16 : 32;
    L->x_kb_bytes = M <= 8 ? 1024 : L->bn * BK * 2;           // 8 tokens: one group of 8 rows, read twice
    L->xs_bytes = 0; L->stage_bytes = 0; L->nw_bytes = 0; L->stage_rows = 1;
    int k_norm = 0;
    for (int i = 0; i < n_phases; ++i) {
        int a_box, tiles, splits, per;
        if (!plan_phase(phases[i], sms, &a_box, &tiles, &splits, &per)) return false;
        L->xs_bytes = max(L->xs_bytes, per * SUBS * L->x_kb_bytes);
        if (phases[i].x_kind == X_NORM) {
            k_norm = max(k_norm, phases[i].K);
            L->nw_bytes = max(L->nw_bytes, round_up(phases[i].K * (phases[i].norm_w_dtype == RI_BF16 ? 2 : 4), 1024));
        }
    }
    // rows of the stream staged at a time: as many as leave the ring three stages, at least one
    const int fixed = SMEM_LIMIT - 1024 - HEAD_BYTES - L->xs_bytes - L->nw_bytes;
    if (k_norm > 0) {
        if (k_norm * 4 > ROW_STAGE_BYTES) return false;
        L->stage_rows = min(M, ROW_STAGE_BYTES / (k_norm * 4));
        while (L->stage_rows > 1 && fixed - round_up(L->stage_rows * k_norm * 4, 1024) < 3 * STAGE_BYTES) --L->stage_rows;
        L->stage_bytes = round_up(L->stage_rows * k_norm * 4, 1024);
    }
    const int ring = fixed - L->stage_bytes;
    L->stages = min(MAX_STAGES, ring / STAGE_BYTES);
    return L->stages >= 2;
}
}  // namespace

// Whether the chain can run these products with `M` tokens (1) or not (0): the caller uses
// this to decide between the chain and separate kernels.
RI_API int ri_decode_chain_fits(const RiChainPhase* phases, int n_phases, int M, int sms) {
    if (M > 16) return ri_decode_chain_wide_fits(phases, n_phases, M, sms);
    Layout L;
    return phases && plan_layout(phases, n_phases, M, sms, &L) ? 1 : 0;
}

RI_API int ri_decode_chain(const RiChainPhase* phases, int n_phases, const RiChainRope* rope, int M,
                           unsigned* grid_bar, int* error, int sms, void* stream) {
    if (M > 16) return ri_decode_chain_wide(phases, n_phases, rope, M, grid_bar, error, sms, stream);
    Layout L;
    if (!phases || !grid_bar || !error || !plan_layout(phases, n_phases, M, sms, &L)) return (int)cudaErrorInvalidValue;
    Maps maps;
    Params p = {};
    p.M = M; p.n_phases = n_phases; p.grid_bar = grid_bar; p.error = error;
    for (int i = 0; i < n_phases; ++i) {
        const RiChainPhase& f = phases[i];
        Phase& P = p.ph[i];
        if (!f.w || !f.x || !f.out || (reinterpret_cast<uintptr_t>(f.w) & 15) || (reinterpret_cast<uintptr_t>(f.x) & 15) ||
            f.out_kind < 0 || f.out_kind > 2 || f.x_kind < 0 || f.x_kind > 2)
            return (int)cudaErrorInvalidValue;
        if (f.x_kind == X_PARTIALS && (!f.part_lse || f.part_splits < 1 || f.part_head_dim < 8 || f.part_head_dim % 8 ||
                                       f.part_heads * f.part_head_dim != f.K))
            return (int)cudaErrorInvalidValue;
        if (f.x_kind == X_BF16 && (f.ld_x % 8 || f.x_rows < (M <= 8 ? 8 : L.bn))) return (int)cudaErrorInvalidValue;
        if (f.x_kind == X_NORM && (f.ld_x % 4 || !f.norm_w || (reinterpret_cast<uintptr_t>(f.norm_w) & 15))) return (int)cudaErrorInvalidValue;
        if (f.out_kind == OUT_SILU_BF16 && f.N % 2) return (int)cudaErrorInvalidValue;
        P.N = f.N; P.K = f.K;
        plan_phase(f, sms, &P.a_box, &P.tiles, &P.splits, &P.per);
        P.x_kind = f.x_kind; P.ld_x = f.ld_x; P.x = f.x; P.norm_w = f.norm_w;
        P.part_lse = f.part_lse; P.part_splits = f.part_splits; P.part_heads = f.part_heads; P.part_hd = f.part_head_dim;
        P.norm_w_bf16 = f.norm_w_dtype == RI_BF16 ? 1 : 0; P.eps = f.eps;
        P.out_kind = f.out_kind; P.ld_out = f.ld_out; P.out = f.out;
        RI_CHECKED(ri_tc_weight_map(f.w, f.N, f.K, P.a_box, &maps.m[i]));
        // a bf16 activation matrix is fetched by TMA, a block of 64 columns of the first rows at a time
        if (f.x_kind == X_BF16) RI_CHECKED(ri_tc_weight_map(f.x, f.x_rows, f.K, M <= 8 ? 8 : L.bn, &maps.x[i]));
        else maps.x[i] = maps.m[i];
    }
    p.stages = L.stages;
    p.x_kb_bytes = L.x_kb_bytes;
    p.xs_off = HEAD_BYTES + p.stages * STAGE_BYTES;
    p.stage_off = p.xs_off + L.xs_bytes;
    p.stage_rows = L.stage_rows;
    p.nw_off = p.stage_off + L.stage_bytes;
    if (rope) {
        Rope& R = p.rope;
        R.enabled = 1; R.qkv = rope->qkv; R.ld = rope->ld; R.positions = rope->positions; R.cos_t = rope->cos_t;
        R.sin_t = rope->sin_t; R.slot_of_token = rope->slot_of_token; R.q_out = reinterpret_cast<bf16*>(rope->q_out);
        R.ld_q = rope->ld_q; R.cache = reinterpret_cast<bf16*>(rope->cache); R.Hq = rope->Hq; R.Hkv = rope->Hkv;
        R.hd = rope->hd; R.rot = rope->rot; R.page_size = rope->page_size;
        if (!R.qkv || !R.positions || !R.cos_t || !R.sin_t || !R.q_out || R.rot > R.hd || R.rot % 2 || R.page_size < 1)
            return (int)cudaErrorInvalidValue;
    }
    const size_t smem = 1024 + (size_t)p.nw_off + L.nw_bytes;
    cudaStream_t s = (cudaStream_t)stream;
    return launch_chain<16>(maps, p, sms, smem, s);
}
