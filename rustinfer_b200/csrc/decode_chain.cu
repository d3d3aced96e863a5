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

namespace {
using namespace ri_tc;
constexpr int BM = 128, BK = 64, THREADS = 192;
constexpr int SUB_BYTES = BM * BK * 2;         // one 64-column tile of 128 weight rows: 16 KB, whatever a_box is
constexpr int SUBS = 2;                        // tiles per ring stage: one wait and one commit serve 8 MMAs
constexpr int STAGE_BYTES = SUBS * SUB_BYTES;
constexpr int KSTEP = SUBS * BK;               // K columns per stage
constexpr int MAX_PHASES = 6, MAX_STAGES = 6;
constexpr int HEAD_BYTES = 1024;               // barriers and row scales in front of the ring
constexpr int SMEM_LIMIT = 225 * 1024;

enum XKind { X_BF16 = 0, X_NORM = 1 };
enum OutKind { OUT_ADD_F32 = 0, OUT_SILU_BF16 = 1, OUT_BF16 = 2 };
enum ErrorCode { ERR_CHAIN_PRODUCER = 11, ERR_CHAIN_MMA = 12, ERR_CHAIN_EPILOGUE = 13, ERR_CHAIN_GRID = 14 };

struct Phase {
    int N, K;                   // weight [N][K]
    int a_box, tiles, splits, per;   // weight rows per tile, tiles along N, K slices, stages (KSTEP columns) per slice
    int x_kind, ld_x;
    const void* x;              // X_BF16: bf16 [M][ld_x];  X_NORM: fp32 [M][ld_x]
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
    Phase ph[MAX_PHASES];
    Rope rope;
    unsigned* grid_bar;         // [0] arrivals, [1] exits; zero between launches
    int* error;
};

struct Maps { CUtensorMap m[MAX_PHASES]; };

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs have arrived `target` times in total.  One thread spins (bounded).
__device__ __forceinline__ bool grid_wait(const unsigned* bar, unsigned target, int* error) {
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
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_full + 1);
    unsigned* go_slot = tmem_slot + 1;                            // 1 while the grid barriers hold
    float* row_scale = reinterpret_cast<float*>(base + 384);     // [BN]
    float* row_part = row_scale + BN;                            // [4 warps][BN]
    unsigned char* ring = base + HEAD_BYTES;
    unsigned char* xs = base + p.xs_off;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, STAGES = p.stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(x_ready, 4);
        mbar_init(acc_full, 1);
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
            const int kblocks = (P.K + KSTEP - 1) / KSTEP;
            const unsigned tx = (unsigned)P.a_box * BK * 2 * SUBS;     // a box past the last column still counts, as zeros
            for (int item = blockIdx.x; item < P.tiles * P.splits && ok; item += G) {
                const int tile = item % P.tiles, kb0 = (item / P.tiles) * P.per;
                const int n_kb = min(P.per, kblocks - kb0);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % STAGES, round = it / STAGES;
                    if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, p.error, ERR_CHAIN_PRODUCER)) { ok = false; break; }
                    mbar_expect_tx(&full[s], tx);
#pragma unroll
                    for (int h = 0; h < SUBS; ++h)
                        tma_load_2d(ring + (size_t)s * STAGE_BYTES + h * SUB_BYTES, &maps.m[ph], &full[s],
                                    (kb0 + i) * KSTEP + h * BK, tile * P.a_box);
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
        // one scalar thread feeds the tensor core: descriptors are made once and stepped by adds,
        // the ring position is counted, not divided
        const uint64_t desc_ring = smem_desc(smem_u32(ring)), desc_xs = smem_desc(smem_u32(xs));
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
                                        db + (uint64_t)(h * ((BN * BK * 2) >> 4) + k * 2), idesc, (i > 0 || h > 0 || k > 0) ? 1u : 0u);
                    tc_commit(&empty[s]);
                    db += (uint64_t)(SUBS * ((BN * BK * 2) >> 4));
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
            for (unsigned spin = 0; spin < 4096; ++spin) __nanosleep(256);
        }
    } else if (warp >= 2) {
        // ------------------------------------------------- activations, epilogue, barrier
        const int quarter = warp & 3;                     // the 32 TMEM lanes this warp may read
        const int te = threadIdx.x - 64, M = p.M;
        const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16);
        bool ok = true;
        int n = 0;
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
            bool scaled = false;
            for (int item = blockIdx.x; item < P.tiles * P.splits; item += G, ++n) {
                const int tile = item % P.tiles, st0 = (item / P.tiles) * P.per;
                const int kb0 = st0 * SUBS, n_kb = min(P.per, kblocks - st0) * SUBS;   // in 64-column blocks
                if (!ok) continue;
                // ---- the activation operand of this K slice: the 16-byte chunk c of token r in
                // k-block kbl sits at chunk c ^ (r & 7) of its 128-byte row (the swizzle the
                // tensor core expects).  Every load of a batch is issued before the first use:
                // under a full weight stream one trip to L2 takes well over a microsecond.
                if (P.x_kind == X_BF16) {
                    const bf16* xb = reinterpret_cast<const bf16*>(P.x);
                    const int total = M * n_kb * 8;
                    for (int i0 = te; i0 < total; i0 += 128 * 8) {
                        uint4 v[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int idx = i0 + 128 * i, rest = idx >> 3;
                            const int kbl = rest % n_kb, r = rest / n_kb;
                            const int k = (kb0 + kbl) * BK + (idx & 7) * 8;
                            v[i] = make_uint4(0u, 0u, 0u, 0u);
                            if (idx < total && k < P.K) v[i] = __ldcg(reinterpret_cast<const uint4*>(xb + (size_t)r * P.ld_x + k));
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int idx = i0 + 128 * i, rest = idx >> 3, c = idx & 7;
                            const int kbl = rest % n_kb, r = rest / n_kb;
                            if (idx < total)
                                *reinterpret_cast<uint4*>(xs + (size_t)kbl * (BN * BK * 2) + r * 128 + ((c ^ (r & 7)) << 4)) = v[i];
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(x_ready);
                } else {
                    // the fp32 stream times the norm weight; the same pass over whole rows gives
                    // the sum of squares (needed once per product), so nothing is read twice
                    const float* hs = reinterpret_cast<const float*>(P.x);
                    const int upr = P.K >> 3;                               // units of 8 floats in a row
                    const int k_lo = kb0 * BK, k_hi = (kb0 + n_kb) * BK;
                    constexpr int RG = 8, UB = 2;                           // rows and units per batch
                    for (int r0 = 0; r0 < M; r0 += RG) {
                        float ss[RG];
#pragma unroll
                        for (int j = 0; j < RG; ++j) ss[j] = 0.f;
                        const int u_end = scaled ? min(upr, k_hi >> 3) : upr;      // later items only need their slice
                        for (int u0 = (scaled ? (k_lo >> 3) : 0) + te; u0 < u_end; u0 += 128 * UB) {
                            float4 a[RG][UB], b[RG][UB];
                            float w[UB][8];
#pragma unroll
                            for (int i = 0; i < UB; ++i) {
                                const int u = u0 + 128 * i, k = u * 8;
#pragma unroll
                                for (int j = 0; j < RG; ++j) {
                                    a[j][i] = make_float4(0.f, 0.f, 0.f, 0.f); b[j][i] = a[j][i];
                                    if (u < u_end && r0 + j < M) {
                                        const float* hr = hs + (size_t)(r0 + j) * P.ld_x + k;
                                        a[j][i] = __ldcg(reinterpret_cast<const float4*>(hr));
                                        b[j][i] = __ldcg(reinterpret_cast<const float4*>(hr + 4));
                                    }
                                }
#pragma unroll
                                for (int e = 0; e < 8; ++e) w[i][e] = 0.f;
                                if (u < u_end && k >= k_lo && k < k_hi) {
                                    if (P.norm_w_bf16) {
                                        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(P.norm_w) + k));
                                        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                                        for (int e = 0; e < 4; ++e) {
                                            const float2 f = __bfloat1622float2(wp[e]);
                                            w[i][2 * e] = f.x; w[i][2 * e + 1] = f.y;
                                        }
                                    } else {
                                        const float* wf = reinterpret_cast<const float*>(P.norm_w) + k;
                                        const float4 wa = __ldg(reinterpret_cast<const float4*>(wf));
                                        const float4 wb = __ldg(reinterpret_cast<const float4*>(wf + 4));
                                        w[i][0] = wa.x; w[i][1] = wa.y; w[i][2] = wa.z; w[i][3] = wa.w;
                                        w[i][4] = wb.x; w[i][5] = wb.y; w[i][6] = wb.z; w[i][7] = wb.w;
                                    }
                                }
                            }
#pragma unroll
                            for (int i = 0; i < UB; ++i) {
                                const int u = u0 + 128 * i, k = u * 8;
                                const bool mine = u < u_end && k >= k_lo && k < k_hi;
                                const int kbl = (k >> 6) - kb0, c = u & 7;
#pragma unroll
                                for (int j = 0; j < RG; ++j) {
                                    const float4 x0 = a[j][i], x1 = b[j][i];
                                    ss[j] += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w
                                           + x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
                                    const int r = r0 + j;
                                    if (mine && r < M) {
                                        float x[8];
                                        x[0] = x0.x * w[i][0]; x[1] = x0.y * w[i][1]; x[2] = x0.z * w[i][2]; x[3] = x0.w * w[i][3];
                                        x[4] = x1.x * w[i][4]; x[5] = x1.y * w[i][5]; x[6] = x1.z * w[i][6]; x[7] = x1.w * w[i][7];
                                        *reinterpret_cast<uint4*>(xs + (size_t)kbl * (BN * BK * 2) + r * 128 + ((c ^ (r & 7)) << 4)) = pack8(x);
                                    }
                                }
                            }
                        }
                        if (!scaled) {
#pragma unroll
                            for (int j = 0; j < RG; ++j) {
                                const float t = warp_sum(ss[j]);
                                if (lane == 0 && r0 + j < M) row_part[quarter * BN + r0 + j] = t;
                            }
                        }
                    }
                    // columns of the last stage that lie beyond K meet zero weights: they must not be NaN
                    for (int u = max(upr, k_lo >> 3) + te; u < (k_hi >> 3); u += 128)
                        for (int r = 0; r < M; ++r)
                            *reinterpret_cast<uint4*>(xs + (size_t)((u >> 3) - kb0) * (BN * BK * 2) + r * 128 + (((u & 7) ^ (r & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(x_ready);
                    if (!scaled) {
                        // the RMS scale of every token, applied to the accumulator later
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (te < M)
                            row_scale[te] = 1.0f / sqrtf((row_part[te] + row_part[BN + te] + row_part[2 * BN + te] + row_part[3 * BN + te])
                                                         / (float)P.K + P.eps);
                        scaled = true;
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                    }
                }
                // ---- the accumulator: lanes are weight rows (features), columns are tokens
                ok = mbar_wait(acc_full, n & 1, p.error, ERR_CHAIN_EPILOGUE);
                tc_fence_after();
                const int fl = quarter * 32 + lane;
                const int feat = fl < P.a_box ? tile * P.a_box + fl : 0x3fffffff;
                if (ok && n_kb > 0) {
                    for (int c0 = 0; c0 < BN && c0 < M; c0 += 16) {
                        float v[16];
                        tmem_ld16(taddr + c0, v);
                        if (P.x_kind == X_NORM) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] *= row_scale[min(c0 + j, BN - 1)];
                        }
                        if (P.out_kind == OUT_ADD_F32) {
                            float* o = reinterpret_cast<float*>(P.out);
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c0 + j < M && feat < P.N) atomicAdd(o + (size_t)(c0 + j) * P.ld_out + feat, v[j]);
                        } else if (P.out_kind == OUT_SILU_BF16) {
                            bf16* o = reinterpret_cast<bf16*>(P.out);
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const float up = __shfl_xor_sync(0xffffffffu, v[j], 1);   // even lane: gate, odd: up
                                if (c0 + j < M && feat < P.N && (lane & 1) == 0)
                                    o[(size_t)(c0 + j) * P.ld_out + (feat >> 1)] = __float2bfloat16_rn(silu_mul(v[j], up));
                            }
                        } else {
                            bf16* o = reinterpret_cast<bf16*>(P.out);
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c0 + j < M && feat < P.N) o[(size_t)(c0 + j) * P.ld_out + feat] = __float2bfloat16_rn(v[j]);
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
            if (threadIdx.x == 64 && *go_slot && !grid_wait(p.grid_bar, (unsigned)G * p.n_phases, p.error)) *go_slot = 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            ok = ok && *go_slot;
            const int heads = R.Hq + 2 * R.Hkv, half = R.rot >> 1;
            const size_t head_step = (size_t)R.page_size * R.hd;
            for (int wi = blockIdx.x * 4 + quarter; wi < M * heads && ok; wi += G * 4) {
                const int t = wi / heads, hh = wi - t * heads;
                float* src = R.qkv + (size_t)t * R.ld + (size_t)hh * R.hd;
                const int slot = R.slot_of_token ? R.slot_of_token[t] : -1;
                bf16* dst = nullptr;
                if (hh < R.Hq) {
                    dst = R.q_out + (size_t)t * R.ld_q + (size_t)hh * R.hd;
                } else if (slot >= 0 && R.cache) {
                    const int page = slot / R.page_size, off = slot - page * R.page_size;
                    const int kv = hh < R.Hq + R.Hkv ? 0 : 1, g = hh - R.Hq - kv * R.Hkv;
                    dst = R.cache + ((size_t)(page * 2 + kv) * R.Hkv * R.page_size + off) * R.hd + (size_t)g * head_step;
                }
                if (hh < R.Hq + R.Hkv) {
                    const int pos = R.positions[t];
                    const float* ct = R.cos_t + (size_t)pos * half;
                    const float* st = R.sin_t + (size_t)pos * half;
                    for (int j = lane; j < half; j += 32) {
                        const float x1 = __ldcg(src + j), x2 = __ldcg(src + j + half);
                        const float c = ct[j], s = st[j];
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

// One product of a chain, as the caller describes it.
struct RiChainPhase {
    const void* w;              // bf16 [N][K], K a multiple of 8, 16-byte aligned
    int N, K;
    int x_kind;                 // 0: x is bf16 [M][ld_x]; 1: x is the fp32 stream [M][ld_x] and the
    int ld_x;                   //    operand is x * norm_w * rsqrt(mean(x^2) + eps)
    const void* x;
    const void* norm_w;
    int norm_w_dtype;
    float eps;
    int out_kind;               // 0: fp32 out += product; 1: bf16 out[M][N/2] = silu(gate) * up over
    int ld_out;                 //    alternating weight rows; 2: bf16 out = product
    void* out;
};

struct RiChainRope {
    float* qkv; int ld;
    const int* positions; const float* cos_t; const float* sin_t; const int* slot_of_token;
    void* q_out; int ld_q;
    void* cache;
    int Hq, Hkv, hd, rot, page_size;
};

// Shared memory the chain would need with `M` tokens (0 if it cannot run): the caller uses
// this to decide between the chain and separate kernels.
RI_API int ri_decode_chain_fits(const RiChainPhase* phases, int n_phases, int M, int sms) {
    if (n_phases < 1 || n_phases > MAX_PHASES || M < 1 || M > 32 || sms < 1) return 0;
    const int bn = M <= 16 ? 16 : 32;
    int xs = 0;
    for (int i = 0; i < n_phases; ++i) {
        const RiChainPhase& f = phases[i];
        if (f.N < 1 || f.K < 8 || f.K % 8) return 0;
        const int kblocks = (f.K + KSTEP - 1) / KSTEP, tiles = (f.N + BM - 1) / BM;
        int splits = f.out_kind == OUT_ADD_F32 ? max(1, min(kblocks, sms / tiles)) : 1;
        const int per = (kblocks + splits - 1) / splits;
        xs = max(xs, per * SUBS * bn * BK * 2);
    }
    const int ring = SMEM_LIMIT - 1024 - HEAD_BYTES - xs;
    return ring >= 3 * STAGE_BYTES ? xs : 0;
}

RI_API int ri_decode_chain(const RiChainPhase* phases, int n_phases, const RiChainRope* rope, int M,
                           unsigned* grid_bar, int* error, int sms, void* stream) {
    if (!phases || n_phases < 1 || n_phases > MAX_PHASES || M < 1 || M > 32 || !grid_bar || !error || sms < 1)
        return (int)cudaErrorInvalidValue;
    const int bn = M <= 16 ? 16 : 32;
    Maps maps;
    Params p = {};
    p.M = M; p.n_phases = n_phases; p.grid_bar = grid_bar; p.error = error;
    int xs = 0;
    for (int i = 0; i < n_phases; ++i) {
        const RiChainPhase& f = phases[i];
        Phase& P = p.ph[i];
        if (!f.w || !f.x || !f.out || f.N < 1 || f.K < 8 || f.K % 8 || (reinterpret_cast<uintptr_t>(f.w) & 15) ||
            (reinterpret_cast<uintptr_t>(f.x) & 15) || f.out_kind < 0 || f.out_kind > 2 || f.x_kind < 0 || f.x_kind > 1)
            return (int)cudaErrorInvalidValue;
        if (f.x_kind == X_BF16 && f.ld_x % 8) return (int)cudaErrorInvalidValue;
        if (f.x_kind == X_NORM && (f.ld_x % 4 || !f.norm_w || (reinterpret_cast<uintptr_t>(f.norm_w) & 15))) return (int)cudaErrorInvalidValue;
        if (f.out_kind == OUT_SILU_BF16 && f.N % 2) return (int)cudaErrorInvalidValue;
        const int kblocks = (f.K + KSTEP - 1) / KSTEP, tiles128 = (f.N + BM - 1) / BM;
        P.N = f.N; P.K = f.K;
        if (f.out_kind == OUT_ADD_F32) {
            P.a_box = BM; P.tiles = tiles128;
            const int splits = max(1, min(kblocks, sms / tiles128));
            P.per = (kblocks + splits - 1) / splits;
            P.splits = (kblocks + P.per - 1) / P.per;
        } else {
            // cut along N only, into a whole number of waves of nearly equal tiles
            const int waves = (tiles128 + sms - 1) / sms;
            P.a_box = min(BM, round_up((f.N + waves * sms - 1) / (waves * sms), 16));
            P.tiles = (f.N + P.a_box - 1) / P.a_box;
            P.splits = 1; P.per = kblocks;
        }
        P.x_kind = f.x_kind; P.ld_x = f.ld_x; P.x = f.x; P.norm_w = f.norm_w;
        P.norm_w_bf16 = f.norm_w_dtype == RI_BF16 ? 1 : 0; P.eps = f.eps;
        P.out_kind = f.out_kind; P.ld_out = f.ld_out; P.out = f.out;
        xs = max(xs, P.per * SUBS * bn * BK * 2);
        RI_CHECKED(ri_tc_weight_map(f.w, f.N, f.K, P.a_box, &maps.m[i]));
    }
    const int ring = SMEM_LIMIT - 1024 - HEAD_BYTES - xs;
    if (ring < 3 * STAGE_BYTES) return (int)cudaErrorInvalidValue;
    p.stages = min(MAX_STAGES, ring / STAGE_BYTES);
    p.xs_off = HEAD_BYTES + p.stages * STAGE_BYTES;
    if (rope) {
        Rope& R = p.rope;
        R.enabled = 1; R.qkv = rope->qkv; R.ld = rope->ld; R.positions = rope->positions; R.cos_t = rope->cos_t;
        R.sin_t = rope->sin_t; R.slot_of_token = rope->slot_of_token; R.q_out = reinterpret_cast<bf16*>(rope->q_out);
        R.ld_q = rope->ld_q; R.cache = reinterpret_cast<bf16*>(rope->cache); R.Hq = rope->Hq; R.Hkv = rope->Hkv;
        R.hd = rope->hd; R.rot = rope->rot; R.page_size = rope->page_size;
        if (!R.qkv || !R.positions || !R.cos_t || !R.sin_t || !R.q_out || R.rot > R.hd || R.rot % 2 || R.page_size < 1)
            return (int)cudaErrorInvalidValue;
    }
    const size_t smem = 1024 + (size_t)p.xs_off + xs;
    cudaStream_t s = (cudaStream_t)stream;
    return bn == 16 ? launch_chain<16>(maps, p, sms, smem, s) : launch_chain<32>(maps, p, sms, smem, s);
}
