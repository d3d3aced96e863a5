// The chain of a decoder layer's products for steps of 17 to 64 tokens (see decode_chain.cu for
// the idea and for steps of up to 16).  With that many tokens the activation operand no longer
// fits in shared memory beside a useful ring, so it streams through the ring with the weights:
// a stage holds two 64-column blocks of weight rows and the same two blocks of the activations.
// Weights are fetched as early as a stage is free; the activation blocks of a product only once
// the grid barrier before it has been passed (the producer thread keeps two cursors).  A product
// that reads the RMS norm of the fp32 stream is preceded by a small phase of its own, spread over
// all CTAs: stream times norm weight to bf16 in global memory, and the rows' sums of squares
// added up with atomics; the product then applies rsqrt(mean + eps) to its accumulator.
//
//   warp 0      TMA producer (weights ahead, activations behind the barrier)
//   warp 1      tensor memory; one thread issues tcgen05.mma
//   warps 2-5   conversion phases, epilogues, grid barrier
//
// Every wait is bounded; on a time-out a code is left in *error and the kernel winds down.
#include "common.cuh"
#include "tc_primitives.cuh"
#include "decode_chain_api.h"
#include <cuda.h>

namespace {
using namespace ri_tc;
constexpr int BM = 128, BK = 64, THREADS = 192, SUBS = 2;
constexpr int KSTEP = SUBS * BK;
constexpr int W_BYTES = SUBS * BM * BK * 2;        // weight part of a stage: 32 KB, whatever a_box is
constexpr int MAX_PHASES = 7, MAX_STAGES = 6;
constexpr int HEAD_BYTES = 1024;
constexpr int SMEM_LIMIT = 225 * 1024;

enum Kind { K_GEMM = 0, K_CONVERT = 1 };
enum OutKind { OUT_ADD_F32 = 0, OUT_SILU_BF16 = 1, OUT_BF16 = 2 };
enum ErrorCode { ERR_WIDE_PRODUCER = 15, ERR_WIDE_MMA = 16, ERR_WIDE_EPILOGUE = 17, ERR_WIDE_GRID = 18 };

struct Phase {
    int kind;
    // product: out (+)= x W^T, x a bf16 matrix fetched by TMA
    int N, K, a_box, tiles, splits, per;
    int out_kind, ld_out;
    void* out;
    const float* rowsq;         // not null: the accumulator is scaled by rsqrt(rowsq[token] / K + eps)
    float eps;
    // conversion: xn = bf16(h * norm_w), rowsq[token] += sum h^2
    const float* h; int ld_h;
    const void* norm_w; int norm_w_bf16;
    bf16* xn; int ld_xn;
    float* rowsq_out;
};

struct Rope {
    int enabled;
    float* qkv; int ld;
    const int* positions; const float* cos_t; const float* sin_t; const int* slot_of_token;
    bf16* q_out; int ld_q;
    bf16* cache;
    int Hq, Hkv, hd, rot, page_size;
};

struct Params {
    int M, n_phases, stages, stage_bytes;
    Phase ph[MAX_PHASES];
    Rope rope;
    float* zero_a; float* zero_b;       // sums of squares to put back to zero at the end
    unsigned* grid_bar;
    int* error;
};

struct Maps { CUtensorMap w[MAX_PHASES]; CUtensorMap x[MAX_PHASES]; };

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool grid_wait(const unsigned* bar, unsigned target, int* error) {
#pragma unroll 1
    for (unsigned i = 0; i < SPIN_LIMIT; ++i) {
        if (ld_acquire(bar) >= target) return true;
        if (i > 64) __nanosleep(32);
    }
    atomicExch(error, ERR_WIDE_GRID);
    return false;
}
// Where a CTA is in its list of (product, item, stage): products only, conversions are skipped.
struct Cursor {
    int ph, item, i, n_kb, kb0, tile, a_box;
    bool done;
};
__device__ __forceinline__ void cursor_settle(Cursor& c, const Params& p, int G) {
    while (c.ph < p.n_phases) {
        const Phase& P = p.ph[c.ph];
        if (P.kind == K_GEMM && c.item < P.tiles * P.splits) {
            const int kblocks = (P.K + KSTEP - 1) / KSTEP;
            c.tile = c.item % P.tiles;
            c.kb0 = (c.item / P.tiles) * P.per;
            c.n_kb = min(P.per, kblocks - c.kb0);
            c.a_box = P.a_box;
            return;
        }
        ++c.ph;
        c.item = blockIdx.x;
    }
    c.done = true;
}
__device__ __forceinline__ void cursor_next(Cursor& c, const Params& p, int G) {
    if (++c.i < c.n_kb) return;
    c.i = 0;
    c.item += G;
    cursor_settle(c, p, G);
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
decode_chain_wide_kernel(const __grid_constant__ Maps maps, const __grid_constant__ Params p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(base);          // [MAX_STAGES]
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* acc_full = empty + MAX_STAGES;
    uint64_t* acc_empty = acc_full + 1;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 1);
    unsigned* go_slot = tmem_slot + 1;
    float* row_scale = reinterpret_cast<float*>(base + 512);     // [BN]
    unsigned char* ring = base + HEAD_BYTES;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr int X_BYTES = SUBS * BN * BK * 2;                  // activation part of a stage

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, STAGES = p.stages, STAGE_BYTES = p.stage_bytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 4);
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
        // cw: the next stage whose weights go out (as soon as its slot in the ring is free);
        // cx: the next stage whose activations go out (once the barrier before its product
        // has been passed, since another product wrote them)
        pdl_trigger();
        pdl_wait();                                       // the first product's activations come from the kernel before
        Cursor cw = {0, (int)blockIdx.x, 0, 0, 0, 0, 0, false}, cx = cw;
        cursor_settle(cw, p, G);
        cursor_settle(cx, p, G);
        int wn = 0, xn = 0;
        unsigned passed = 0, idle = 0;                    // phases whose input is complete on all CTAs
        while (!cx.done) {
            bool did = false;
            if (!cw.done) {
                const int s = wn % STAGES, round = wn / STAGES;
                if (round == 0 || mbar_try_wait(&empty[s], (round - 1) & 1)) {
                    mbar_expect_tx(&full[s], (unsigned)(cw.a_box * BK * 2 * SUBS + X_BYTES));
#pragma unroll
                    for (int h = 0; h < SUBS; ++h)
                        tma_load_2d(ring + (size_t)s * STAGE_BYTES + h * (BM * BK * 2), &maps.w[cw.ph], &full[s],
                                    (cw.kb0 + cw.i) * KSTEP + h * BK, cw.tile * cw.a_box);
                    ++wn;
                    cursor_next(cw, p, G);
                    did = true;
                }
            }
            if (xn < wn) {
                if ((unsigned)cx.ph <= passed) {
                    const int s = xn % STAGES;
#pragma unroll
                    for (int h = 0; h < SUBS; ++h)
                        tma_load_2d(ring + (size_t)s * STAGE_BYTES + W_BYTES + h * (BN * BK * 2), &maps.x[cx.ph], &full[s],
                                    (cx.kb0 + cx.i) * KSTEP + h * BK, 0);
                    ++xn;
                    cursor_next(cx, p, G);
                    did = true;
                } else {
                    passed = ld_acquire(p.grid_bar) / (unsigned)G;
                }
            }
            if (did) idle = 0;
            else if (++idle > SPIN_LIMIT) { atomicExch(p.error, ERR_WIDE_PRODUCER); break; }
            else if (idle > 64) __nanosleep(32);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
        const uint64_t desc_ring = smem_desc(smem_u32(ring));
        const unsigned stage_step = (unsigned)STAGE_BYTES >> 4;
        Cursor c = {0, (int)blockIdx.x, 0, 0, 0, 0, 0, false};
        cursor_settle(c, p, G);
        bool ok = true;
        int s = 0, n = 0;
        unsigned par = 0;
        while (!c.done && ok) {
            // the epilogue has read the accumulator of the item before
            if (n > 0 && !mbar_wait(acc_empty, (n - 1) & 1, p.error, ERR_WIDE_MMA)) { ok = false; break; }
            tc_fence_after();
            const int n_kb = c.n_kb;
            for (int i = 0; i < n_kb; ++i) {
                if (!mbar_try_wait(&full[s], par) && !mbar_wait(&full[s], par, p.error, ERR_WIDE_MMA)) { ok = false; break; }
                tc_fence_after();
                const uint64_t da = desc_ring + (uint64_t)(s * stage_step), db = da + (uint64_t)(W_BYTES >> 4);
#pragma unroll
                for (int h = 0; h < SUBS; ++h)
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        mma_bf16_ss(tmem_base, da + (uint64_t)(h * ((BM * BK * 2) >> 4) + k * 2),
                                    db + (uint64_t)(h * ((BN * BK * 2) >> 4) + k * 2), idesc, (i > 0 || h > 0 || k > 0) ? 1u : 0u);
                tc_commit(&empty[s]);
                if (++s == STAGES) { s = 0; par ^= 1u; }
                cursor_next(c, p, G);
            }
            if (ok) tc_commit(acc_full);
            ++n;
        }
        if (!ok) {
            for (int st = 0; st < STAGES; ++st)
                for (int q = 0; q < 2; ++q)
                    if (mbar_try_wait(&full[st], q)) break;
#pragma unroll 1
            for (unsigned spin = 0; spin < 4096; ++spin) __nanosleep(256);
        }
    } else if (warp >= 2) {
        // ----------------------------------------- conversions, epilogues, grid barrier
        const int quarter = warp & 3;
        const int te = threadIdx.x - 64, M = p.M;
        const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16);
        bool ok = true;
        int n = 0;
        pdl_wait();
        for (int ph = 0; ph < p.n_phases; ++ph) {
            const Phase& P = p.ph[ph];
            if (ph > 0) {
                if (threadIdx.x == 64 && *go_slot && !grid_wait(p.grid_bar, (unsigned)G * ph, p.error)) *go_slot = 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                ok = ok && *go_slot;
            }
            if (P.kind == K_CONVERT) {
                // stream times norm weight to bf16, 8 columns a thread; a warp's 32 units lie in one
                // row when a row has a multiple of 32 units, and then add their squares up first
                const int upr = P.K >> 3, total = M * upr;
                const bool rowwise = (upr & 31) == 0;
                for (int unit = blockIdx.x * 128 + te; unit < ((total + 31) & ~31) && ok; unit += G * 128) {
                    float ss = 0.f;
                    int r = 0;
                    if (unit < total) {
                        r = unit / upr;
                        const int k = (unit - r * upr) * 8;
                        const float* hr = P.h + (size_t)r * P.ld_h + k;
                        const float4 a = __ldcg(reinterpret_cast<const float4*>(hr));
                        const float4 b = __ldcg(reinterpret_cast<const float4*>(hr + 4));
                        float w[8];
                        if (P.norm_w_bf16) {
                            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(P.norm_w) + k));
                            const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 f = __bfloat1622float2(wp[e]);
                                w[2 * e] = f.x; w[2 * e + 1] = f.y;
                            }
                        } else {
                            const float* wf = reinterpret_cast<const float*>(P.norm_w) + k;
                            const float4 wa = __ldg(reinterpret_cast<const float4*>(wf));
                            const float4 wb = __ldg(reinterpret_cast<const float4*>(wf + 4));
                            w[0] = wa.x; w[1] = wa.y; w[2] = wa.z; w[3] = wa.w; w[4] = wb.x; w[5] = wb.y; w[6] = wb.z; w[7] = wb.w;
                        }
                        float x[8];
                        x[0] = a.x * w[0]; x[1] = a.y * w[1]; x[2] = a.z * w[2]; x[3] = a.w * w[3];
                        x[4] = b.x * w[4]; x[5] = b.y * w[5]; x[6] = b.z * w[6]; x[7] = b.w * w[7];
                        *reinterpret_cast<uint4*>(P.xn + (size_t)r * P.ld_xn + k) = pack8(x);
                        ss = (a.x * a.x + a.y * a.y) + (a.z * a.z + a.w * a.w) + (b.x * b.x + b.y * b.y) + (b.z * b.z + b.w * b.w);
                    }
                    if (rowwise) {
                        ss = warp_sum(ss);
                        if (lane == 0 && unit < total) atomicAdd(P.rowsq_out + r, ss);
                    } else if (unit < total) {
                        atomicAdd(P.rowsq_out + r, ss);
                    }
                }
            } else {
                if (P.rowsq) {
                    if (te < BN) row_scale[te] = te < M ? 1.0f / sqrtf(__ldcg(P.rowsq + te) / (float)P.K + P.eps) : 0.f;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
                for (int item = blockIdx.x; item < P.tiles * P.splits; item += G, ++n) {
                    const int tile = item % P.tiles;
                    if (!ok) continue;
                    ok = mbar_wait(acc_full, n & 1, p.error, ERR_WIDE_EPILOGUE);
                    tc_fence_after();
                    const int fl = quarter * 32 + lane;
                    const int feat = fl < P.a_box ? tile * P.a_box + fl : 0x3fffffff;
                    // The lane's whole row (one feature, every token) comes out of tensor memory in one
                    // round trip, and the accumulator is given back before anything is stored: eight
                    // round trips of eight tokens each were most of a 3 us epilogue.  The product's
                    // numbers go into registers first (read through `P` they are fetched from the
                    // parameter bank again after every asm statement).
                    const int out_kind = P.out_kind, ld_out = P.ld_out, n_feat = P.N;
                    const bool scaled = P.rowsq != nullptr, live = feat < n_feat;
                    void* const out = P.out;
                    float v[BN];
                    if (ok) tmem_ld_row<BN>(taddr, v);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0 && ok) mbar_arrive(acc_empty);
                    if (!ok) continue;
                    if (scaled) {
#pragma unroll
                        for (int j = 0; j < BN; ++j) v[j] *= row_scale[j];
                    }
                    if (out_kind == OUT_ADD_F32) {
                        float* o = reinterpret_cast<float*>(out) + (live ? feat : 0);
#pragma unroll
                        for (int j = 0; j < BN; ++j)
                            if (j < M && live) atomicAdd(o + (size_t)j * ld_out, v[j]);
                    } else if (out_kind == OUT_BF16) {
                        bf16* o = reinterpret_cast<bf16*>(out) + (live ? feat : 0);
#pragma unroll
                        for (int j = 0; j < BN; ++j)
                            if (j < M && live) o[(size_t)j * ld_out] = __float2bfloat16_rn(v[j]);
                    } else {
                        // rows of the weight alternate gate_j, up_j: an even lane holds the gate and its
                        // neighbour the up value of the same feature.  Of two tokens the even lane
                        // finishes the first and the odd lane the second, so every lane does one
                        // SiLU and one store per pair after one exchange.
                        bf16* o = reinterpret_cast<bf16*>(out) + (live ? (feat >> 1) : 0);
                        const bool odd = (lane & 1) != 0;
#pragma unroll
                        for (int j = 0; j < BN; j += 2) {
                            const float got = __shfl_xor_sync(0xffffffffu, odd ? v[j] : v[j + 1], 1);
                            const float g = odd ? got : v[j], u = odd ? v[j + 1] : got;
                            const int tok = j + (odd ? 1 : 0);
                            if (tok < M && live) o[(size_t)tok * ld_out] = __float2bfloat16_rn(silu_mul(g, u));
                        }
                    }
                }
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) atomicAdd(p.grid_bar, 1u);
        }
        if (p.rope.enabled) {
            const Rope& R = p.rope;
            if (threadIdx.x == 64 && *go_slot && !grid_wait(p.grid_bar, (unsigned)G * p.n_phases, p.error)) *go_slot = 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            ok = ok && *go_slot;
            // A warp takes a run of consecutive (token, head) rows, four at a time: first the
            // positions of all four, then their angles and values (loads that do not wait for one
            // another), then the arithmetic and the stores.  One row at a time the three dependent
            // round trips of each row added up to 6 us at 64 tokens.
            const int heads = R.Hq + 2 * R.Hkv, half = R.rot >> 1;
            const size_t head_step = (size_t)R.page_size * R.hd;
            const int rows = M * heads, warps = G * 4, per = (rows + warps - 1) / warps;
            const int first = (blockIdx.x * 4 + quarter) * per, last = min(first + per, rows);
            constexpr int RB = 4, JMAX = 4;                       // rows at a time; 32-lane strides of half a head
            if (half > 32 * JMAX && ok) { atomicExch(p.error, ERR_WIDE_EPILOGUE); ok = false; }
            for (int r0 = first; r0 < last && ok; r0 += RB) {
                int tok[RB], hh[RB], pos[RB];
#pragma unroll
                for (int b = 0; b < RB; ++b) {
                    const int wi = min(r0 + b, last - 1);
                    tok[b] = wi / heads;
                    hh[b] = wi - tok[b] * heads;
                    pos[b] = hh[b] < R.Hq + R.Hkv ? R.positions[tok[b]] : 0;
                }
                float x1[RB][JMAX], x2[RB][JMAX], cs[RB][JMAX], sn[RB][JMAX];
#pragma unroll
                for (int b = 0; b < RB; ++b) {
                    const float* src = R.qkv + (size_t)tok[b] * R.ld + (size_t)hh[b] * R.hd;
                    const bool rotated = hh[b] < R.Hq + R.Hkv;
                    const float* ct = R.cos_t + (size_t)pos[b] * half;
                    const float* st = R.sin_t + (size_t)pos[b] * half;
#pragma unroll
                    for (int jj = 0; jj < JMAX; ++jj) {
                        const int j = jj * 32 + lane;
                        const bool in = j < half;
                        x1[b][jj] = in ? __ldcg(src + j) : 0.f;
                        x2[b][jj] = in ? __ldcg(src + j + half) : 0.f;
                        cs[b][jj] = in && rotated ? ct[j] : 1.f;
                        sn[b][jj] = in && rotated ? st[j] : 0.f;
                    }
                }
#pragma unroll
                for (int b = 0; b < RB; ++b) {
                    if (r0 + b >= last) continue;
                    float* src = R.qkv + (size_t)tok[b] * R.ld + (size_t)hh[b] * R.hd;
                    const int slot = R.slot_of_token ? R.slot_of_token[tok[b]] : -1;
                    bf16* dst = nullptr;
                    if (hh[b] < R.Hq) {
                        dst = R.q_out + (size_t)tok[b] * R.ld_q + (size_t)hh[b] * R.hd;
                    } else if (slot >= 0 && R.cache) {
                        const int page = slot / R.page_size, off = slot - page * R.page_size;
                        const int kv = hh[b] < R.Hq + R.Hkv ? 0 : 1, g = hh[b] - R.Hq - kv * R.Hkv;
                        dst = R.cache + ((size_t)(page * 2 + kv) * R.Hkv * R.page_size + off) * R.hd + (size_t)g * head_step;
                    }
                    // values (cos 1, sin 0) and the columns beyond the rotated ones pass unchanged
                    for (int j = R.rot + lane; j < R.hd; j += 32)
                        if (dst) dst[j] = __float2bfloat16_rn(__ldcg(src + j));
#pragma unroll
                    for (int jj = 0; jj < JMAX; ++jj) {
                        const int j = jj * 32 + lane;
                        if (j < half && dst) {
                            dst[j] = __float2bfloat16_rn(x1[b][jj] * cs[b][jj] - x2[b][jj] * sn[b][jj]);
                            dst[j + half] = __float2bfloat16_rn(x1[b][jj] * sn[b][jj] + x2[b][jj] * cs[b][jj]);
                        }
                    }
                    __syncwarp();
                    for (int j = lane; j < R.hd; j += 32) src[j] = 0.f;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x < 64) {
        // the last CTA to leave puts the barrier and the sums of squares back to zero
        __shared__ int last;
        if (threadIdx.x == 0) {
            __threadfence();
            last = atomicAdd(p.grid_bar + 1, 1u) == (unsigned)G - 1;
        }
        asm volatile("bar.sync 3, 64;" ::: "memory");
        if (last) {
            if (p.zero_a) p.zero_a[threadIdx.x] = 0.f;
            if (p.zero_b) p.zero_b[threadIdx.x] = 0.f;
            if (threadIdx.x == 0) { p.grid_bar[0] = 0u; p.grid_bar[1] = 0u; }
            __threadfence();
        }
    }
}

int round_up(int a, int b) { return (a + b - 1) / b * b; }

bool plan_product(const RiChainPhase& f, int sms, Phase* P) {
    if (f.N < 1 || f.K < 8 || f.K % 8) return false;
    const int kblocks = (f.K + KSTEP - 1) / KSTEP, tiles128 = (f.N + BM - 1) / BM;
    P->N = f.N; P->K = f.K;
    if (f.out_kind == OUT_ADD_F32) {
        P->a_box = BM; P->tiles = tiles128;
        const int want = max(1, min(kblocks, sms / tiles128));
        P->per = (kblocks + want - 1) / want;
        P->splits = (kblocks + P->per - 1) / P->per;
    } else {
        const int waves = (tiles128 + sms - 1) / sms;
        P->a_box = min(BM, round_up((f.N + waves * sms - 1) / (waves * sms), 16));
        P->tiles = (f.N + P->a_box - 1) / P->a_box;
        P->splits = 1; P->per = kblocks;
    }
    return true;
}

template <int BN>
int launch_wide(const Maps& maps, const Params& p, int grid, size_t smem, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_chain_wide_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // the grid barrier needs all CTAs resident together
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, decode_chain_wide_kernel<BN>, maps, p);
}
}  // namespace

int ri_decode_chain_wide_fits(const RiChainPhase* phases, int n_phases, int M, int sms) {
    if (!phases || n_phases < 1 || M < 17 || M > 64 || sms < 1) return 0;
    int total = 0;
    for (int i = 0; i < n_phases; ++i) {
        Phase P;
        if (!plan_product(phases[i], sms, &P)) return 0;
        if (phases[i].x_kind == 2) return 0;               // unmerged key ranges: the chain for up to 16 tokens alone takes them
        if (phases[i].x_kind == 1 && (!phases[i].xn || !phases[i].rowsq)) return 0;
        total += phases[i].x_kind == 1 ? 2 : 1;
    }
    return total <= MAX_PHASES ? 1 : 0;
}

int ri_decode_chain_wide(const RiChainPhase* phases, int n_phases, const RiChainRope* rope, int M,
                         unsigned* grid_bar, int* error, int sms, void* stream) {
    if (!grid_bar || !error || !ri_decode_chain_wide_fits(phases, n_phases, M, sms)) return (int)cudaErrorInvalidValue;
    const int bn = M <= 32 ? 32 : 64;
    Maps maps;
    Params p = {};
    p.M = M; p.grid_bar = grid_bar; p.error = error;
    int n = 0;
    for (int i = 0; i < n_phases; ++i) {
        const RiChainPhase& f = phases[i];
        if (!f.w || !f.x || !f.out || (reinterpret_cast<uintptr_t>(f.w) & 15) || (reinterpret_cast<uintptr_t>(f.x) & 15) ||
            f.out_kind < 0 || f.out_kind > 2 || f.x_kind < 0 || f.x_kind > 1 || (f.out_kind == OUT_SILU_BF16 && f.N % 2))
            return (int)cudaErrorInvalidValue;
        const void* x = f.x;
        int x_rows = f.x_rows;
        const float* rowsq = nullptr;
        if (f.x_kind == 1) {
            if (f.ld_x % 4 || !f.norm_w || (reinterpret_cast<uintptr_t>(f.norm_w) & 15) || (reinterpret_cast<uintptr_t>(f.xn) & 15))
                return (int)cudaErrorInvalidValue;
            Phase& C = p.ph[n];
            C = Phase{};
            C.kind = K_CONVERT; C.K = f.K;
            C.h = reinterpret_cast<const float*>(f.x); C.ld_h = f.ld_x;
            C.norm_w = f.norm_w; C.norm_w_bf16 = f.norm_w_dtype == RI_BF16 ? 1 : 0;
            C.xn = reinterpret_cast<bf16*>(f.xn); C.ld_xn = f.K; C.rowsq_out = f.rowsq;
            maps.w[n] = CUtensorMap{}; maps.x[n] = CUtensorMap{};
            ++n;
            x = f.xn; x_rows = 64; rowsq = f.rowsq;
            if (!p.zero_a) p.zero_a = f.rowsq;
            else if (!p.zero_b && f.rowsq != p.zero_a) p.zero_b = f.rowsq;
            else if (f.rowsq != p.zero_a && f.rowsq != p.zero_b) return (int)cudaErrorInvalidValue;
        } else if (f.ld_x != f.K || f.x_rows < bn) {
            return (int)cudaErrorInvalidValue;              // the TMA map sees x as [x_rows][K]
        }
        Phase& P = p.ph[n];
        P = Phase{};
        P.kind = K_GEMM;
        plan_product(f, sms, &P);
        P.out_kind = f.out_kind; P.ld_out = f.ld_out; P.out = f.out; P.rowsq = rowsq; P.eps = f.eps;
        RI_CHECKED(ri_tc_weight_map(f.w, f.N, f.K, P.a_box, &maps.w[n]));
        RI_CHECKED(ri_tc_weight_map(x, x_rows, f.K, bn, &maps.x[n]));
        ++n;
    }
    p.n_phases = n;
    p.stage_bytes = W_BYTES + SUBS * bn * BK * 2;
    p.stages = min(MAX_STAGES, (SMEM_LIMIT - 1024 - HEAD_BYTES) / p.stage_bytes);
    if (p.stages < 2) return (int)cudaErrorInvalidValue;
    if (rope) {
        Rope& R = p.rope;
        R.enabled = 1; R.qkv = rope->qkv; R.ld = rope->ld; R.positions = rope->positions; R.cos_t = rope->cos_t;
        R.sin_t = rope->sin_t; R.slot_of_token = rope->slot_of_token; R.q_out = reinterpret_cast<bf16*>(rope->q_out);
        R.ld_q = rope->ld_q; R.cache = reinterpret_cast<bf16*>(rope->cache); R.Hq = rope->Hq; R.Hkv = rope->Hkv;
        R.hd = rope->hd; R.rot = rope->rot; R.page_size = rope->page_size;
        if (!R.qkv || !R.positions || !R.cos_t || !R.sin_t || !R.q_out || R.rot > R.hd || R.rot % 2 || R.page_size < 1)
            return (int)cudaErrorInvalidValue;
    }
    const size_t smem = 1024 + HEAD_BYTES + (size_t)p.stages * p.stage_bytes;
    cudaStream_t s = (cudaStream_t)stream;
    return bn == 32 ? launch_wide<32>(maps, p, sms, smem, s) : launch_wide<64>(maps, p, sms, smem, s);
}
