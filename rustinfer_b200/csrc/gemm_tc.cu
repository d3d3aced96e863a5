// C[M,N] = X[M,K] * W[N,K]^T in bf16 on the 5th-generation tensor cores: tcgen05.mma with
// both operands staged in shared memory by TMA (128-byte swizzle) and the fp32 accumulator
// in tensor memory, read back with tcgen05.ld for a fused epilogue.
//
// RustInfer sends these products to cuBLASLt, with a SIMT GEMV for one row
// (crates/infer-backend-cuda/src/kernels/matmul/matmul.cu:131-650,870-934) and separate
// kernels for SwiGLU and the residual add; it has no sm_100 path.  This kernel is the
// engine's own: one CTA computes a 128 x BN tile (or a K-slice of it).
//
//   warp 0      TMA producer: one thread arms the stage's mbarrier and issues two loads
//   warp 1      allocates tensor memory; one thread issues the MMAs and commits
//   warps 2-5   epilogue: tcgen05.ld of their 32 lanes, then the fused store
//
// Orientation.  The 128-row operand of the MMA ("A") is the weight when few tokens are in
// flight (decode: the weights stream through once, tokens are the narrow N of the MMA) and
// the activations otherwise (prefill).  Split-K: grid.z CTAs take slices of K, park fp32
// partial tiles in a workspace, and the CTA whose ticket is last adds them in slice order
// (so the result does not depend on which CTA came last) and runs the epilogue.
//
// Epilogues: store bf16 / store fp32 / SiLU(gate)*up for a weight whose rows alternate
// gate_j, up_j / add into the fp32 residual stream.
//
// Every wait on an mbarrier is bounded; on a time-out the kernel records a code in
// *error, waits (bounded) for the copies it still has in flight, frees its tensor
// memory and returns.
#include "common.cuh"
#include "tc_primitives.cuh"
#include <cuda.h>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace {
using namespace ri_tc;
constexpr int BM = 128;                 // rows of the A operand per tile (MMA M)
constexpr int BK = 64;                  // 64 bf16 = one 128-byte swizzle row
constexpr int THREADS = 192;

enum Epilogue { EPI_BF16 = 0, EPI_F32 = 1, EPI_SILU = 2, EPI_RESIDUAL = 3, EPI_ROPE = 4 };
enum ErrorCode { ERR_PRODUCER_WAIT = 1, ERR_MMA_WAIT = 2, ERR_EPILOGUE_WAIT = 3, ERR_DRAIN_WAIT = 4 };


constexpr int MAX_STAGES = 32;
// bytes of operand stages per CTA: few tokens (a pure weight stream) take half an SM's
// shared memory, so that the next product's CTAs can move in and prefetch beside them
constexpr int SMEM_BUDGET = 200 * 1024;
constexpr int SMEM_BUDGET_STREAM = 96 * 1024;
constexpr int SMEM_BUDGET_LONG = 160 * 1024;
int g_stream_budget = SMEM_BUDGET_STREAM;
// The MMA always reads 128 rows of A; when a tile loads fewer, the rows past them are
// whatever follows in shared memory, and the lanes they feed are never stored.  The slack
// keeps that read inside the allocation.
constexpr int SMEM_TAIL = BM * BK * 2;
constexpr size_t SMEM_EXTRA = SMEM_TAIL + 1024 /*alignment*/ + 1024 /*barriers*/;
constexpr size_t SMEM_TOTAL = (size_t)SMEM_BUDGET + SMEM_EXTRA;

template <int BN> struct Cfg {
    static constexpr int ACC_COLS = BN < 32 ? 32 : BN;      // columns of one accumulator
    static constexpr int TMEM_COLS = 2 * ACC_COLS;          // two accumulators: epilogue and MMA overlap
};

struct Params {
    int a_rows, b_rows;                  // valid rows of the A and B operands
    int K;
    int swap;                            // 1: A = weight (lanes = features), B = activations (columns = tokens)
    int epilogue;
    void* out;                           // bf16 or fp32 [tokens][ld_out]; fp32 residual stream for EPI_RESIDUAL
    int ld_out;
    int vec;                             // rows of out start on 16-byte boundaries: vector stores allowed
    int splits;
    float* workspace;                    // [tiles][splits][BN][128] fp32
    int* counters;                       // [tiles], zero between calls
    int* error;
    int tiles_a, n_tiles;
    int a_box;                           // rows of A per tile actually loaded (<= 128, a multiple of 8)
    int stages, stage_bytes;             // ring of operand stages: (a_box + BN) * 128 bytes each
    int budget;                          // bytes of the ring
    int pair_bn;                         // width of a CTA pair's tile (256 or 192)
    // CTA pairs, the tiles of the last, partly filled wave: their k-blocks are dealt out evenly
    // over all pairs (each pair a run of k-blocks that meets one or two of those tiles); the
    // parts of a tile are added up in `sk_acc` and the pair that adds last finishes the tile
    int sk_tiles;                        // tiles dealt out that way (0: none), the last of n_tiles
    int sk_pairs, sk_q, sk_extra;        // pairs that take part; k-blocks of each: sk_q, the first sk_extra one more
    float* sk_acc;                       // [pair][first or second tile of its run][2 CTAs][4 warps][width/4][32 lanes][4] fp32
    // EPI_ROPE (CTA pairs only): the product is q, k, v of many tokens; q and k heads are rotated
    // straight from the accumulator, q goes to `out` (bf16 [tokens][ld_out]), k and v into their pages
    const int* rope_positions;           // [tokens]
    const float* rope_cos;               // [positions][head_dim / 2]
    const float* rope_sin;
    const int* rope_slot;                // [tokens] slot of the token's key in the cache, < 0: none; null: no keys
    bf16* rope_cache;                    // [page][K|V][kv head][slot][head_dim]
    int rope_hq, rope_hkv, rope_hd, rope_page;
};


// one accumulator value: token `tok`, feature `feat` (neighbour: the value of feature feat + 1)
__device__ __forceinline__ void store_one(const Params& p, int n_tok, int n_feat, int tok, int feat,
                                          float acc, float neighbour) {
    if (feat >= n_feat || tok >= n_tok) return;
    const size_t row = (size_t)tok * p.ld_out;
    switch (p.epilogue) {
        case EPI_BF16: reinterpret_cast<bf16*>(p.out)[row + feat] = __float2bfloat16_rn(acc); break;
        case EPI_F32: reinterpret_cast<float*>(p.out)[row + feat] = acc; break;
        case EPI_RESIDUAL: atomicAdd(reinterpret_cast<float*>(p.out) + row + feat, acc); break;   // parts of one sum may come from several CTAs
        case EPI_SILU:                                   // even feature = gate_j, odd = up_j
            if ((feat & 1) == 0)
                reinterpret_cast<bf16*>(p.out)[row + (feat >> 1)] = __float2bfloat16_rn(silu_mul(acc, neighbour));
            break;
    }
}


// 16 consecutive features of one token (activations on the 128-row side)
__device__ __forceinline__ void store_row16(const Params& p, int tok, int feat0, const float (&v)[16]) {
    if (tok >= p.a_rows) return;
    if (!p.vec || feat0 + 16 > p.b_rows) {
#pragma unroll
        for (int j = 0; j < 16; ++j) store_one(p, p.a_rows, p.b_rows, tok, feat0 + j, v[j], j < 15 ? v[j + 1] : 0.f);
        return;
    }
    const size_t row = (size_t)tok * p.ld_out;
    switch (p.epilogue) {
        case EPI_BF16: {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + row + feat0);
            dst[0] = pack8(v);
            dst[1] = pack8(v + 8);
            break;
        }
        case EPI_F32: {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + row + feat0);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            break;
        }
        case EPI_RESIDUAL: {
            // a reduction at the memory side instead of load, add, store: nothing comes back, so
            // the thread does not sit out a trip to L2 per 16 columns (each element is added
            // once, so the result does not depend on any order)
            float* dst = reinterpret_cast<float*>(p.out) + row + feat0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                             ::"l"(dst + 4 * j), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3]) : "memory");
            break;
        }
        case EPI_SILU: {
            float m[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) m[j] = silu_mul(v[2 * j], v[2 * j + 1]);
            *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + row + (feat0 >> 1)) = pack8(m);
            break;
        }
    }
}


// 64 consecutive features of one token, all inside the matrix and with rows that allow vector
// stores (the caller has checked both for the whole warp)
__device__ __forceinline__ void store_row64(const Params& p, int tok, int feat0, const float (&v)[64]) {
    if (tok >= p.a_rows) return;
    const size_t row = (size_t)tok * p.ld_out;
    switch (p.epilogue) {
        case EPI_BF16: {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + row + feat0);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = pack8(v + 8 * j);
            break;
        }
        case EPI_F32: {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + row + feat0);
#pragma unroll
            for (int j = 0; j < 16; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            break;
        }
        case EPI_RESIDUAL: {
            float* dst = reinterpret_cast<float*>(p.out) + row + feat0;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                             ::"l"(dst + 4 * j), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3]) : "memory");
            break;
        }
        case EPI_SILU: {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.out) + row + (feat0 >> 1));
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float m[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) m[j] = silu_mul(v[16 * q + 2 * j], v[16 * q + 2 * j + 1]);
                dst[q] = pack8(m);
            }
            break;
        }
    }
}

// Persistent over tiles: CTA x takes tiles x, x + gridDim.x, ...; blockIdx.z is the K slice.
template <int BN>
__global__ void __launch_bounds__(THREADS, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const Params p) {
    using C = Cfg<BN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);      // swizzle atoms are 1 KiB
    const int STAGES = p.stages, STAGE_BYTES = p.stage_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + p.budget + SMEM_TAIL);
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* acc_full = empty + MAX_STAGES;             // [2] accumulator written, epilogue may read
    uint64_t* acc_empty = acc_full + 2;                  // [2] accumulator read, MMA may overwrite
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);
    int* ticket_slot = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (p.K + BK - 1) / BK;
    const int per = (kblocks + p.splits - 1) / p.splits;
    const int kb_begin = blockIdx.z * per;
    const int kb_end = min(kb_begin + per, kblocks);
    const int n_kb = max(kb_end - kb_begin, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((unsigned)C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        // The weight tiles of the first stages are fetched before the dependency wait: no
        // earlier kernel writes weights, so they stream in while the predecessor drains.
        const CUtensorMap* wmap = p.swap ? &map_a : &map_b;
        const CUtensorMap* xmap = p.swap ? &map_b : &map_a;
        const int woff = p.swap ? 0 : p.a_box * BK * 2, xoff = p.swap ? p.a_box * BK * 2 : 0;
        const unsigned stage_tx = (unsigned)(p.a_box + BN) * BK * 2;   // bytes the two boxes of a stage bring
        pdl_trigger();
        const int pre = blockIdx.x < p.n_tiles ? min(n_kb, STAGES) : 0;
        {
            const int tile = blockIdx.x;
            const int w0 = p.swap ? (tile % p.tiles_a) * p.a_box : (tile / p.tiles_a) * BN;
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(&full[i], stage_tx);
                tma_load_2d(tiles + (size_t)i * STAGE_BYTES + woff, wmap, &full[i], (kb_begin + i) * BK, w0);
            }
        }
        pdl_wait();
        // Stages are given back in pairs (the MMA thread commits once per two k-blocks, which
        // halves its fixed cost per k-block), so the producer asks for a pair when it reaches
        // the even stage and then fills both.
        bool ok = true;
        int it = 0, s = 0;                                // k-blocks loaded so far, over all tiles; ring position
        unsigned par = 1;                                 // parity of the release the current lap of the ring waits for
        for (int tile = blockIdx.x; tile < p.n_tiles && ok; tile += gridDim.x) {
            const int a0 = (tile % p.tiles_a) * p.a_box, b0 = (tile / p.tiles_a) * BN;
            const int w0 = p.swap ? a0 : b0, x0 = p.swap ? b0 : a0;
            for (int i = 0; i < n_kb; ++i, ++it) {
                unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                if (it >= pre) {
                    if (it >= STAGES && (s & 1) == 0 &&
                        !mbar_try_wait(&empty[s >> 1], par) && !mbar_wait(&empty[s >> 1], par, p.error, ERR_PRODUCER_WAIT)) { ok = false; break; }
                    mbar_expect_tx(&full[s], stage_tx);
                    tma_load_2d(st + woff, wmap, &full[s], (kb_begin + i) * BK, w0);
                }
                tma_load_2d(st + xoff, xmap, &full[s], (kb_begin + i) * BK, x0);
                if (++s == STAGES) { s = 0; par ^= 1u; }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        // instruction descriptor: D fp32, A and B bf16, both K-major, N = BN, M = 128
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
        // One scalar thread feeds the tensor core, and its own instruction stream is what
        // limits the rate (measured: a wait, four MMAs and a commit with descriptors rebuilt
        // and the ring position divided out cost 870 cycles a k-block against 512 of tensor
        // work at N = 256).  So: descriptors are made once and stepped by adds, the ring
        // position is counted, the wait tries once before it loops, and one commit frees two
        // stages.
        const uint64_t desc0 = smem_desc(smem_u32(tiles));
        const unsigned stage_step = (unsigned)STAGE_BYTES >> 4, b_step = (unsigned)(p.a_box * BK * 2) >> 4;
        bool ok = true;
        int s = 0, t = 0;
        unsigned par = 0;
        for (int tile = blockIdx.x; tile < p.n_tiles && ok; tile += gridDim.x, ++t) {
            const int buf = t & 1, use = t >> 1;
            // the epilogue has emptied this accumulator (first use of a buffer passes at once)
            if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, p.error, ERR_MMA_WAIT)) { ok = false; break; }
            tc_fence_after();
            const unsigned tmem_d = tmem_base + buf * C::ACC_COLS;
            for (int i = 0; i < n_kb; ++i) {
                if (!mbar_try_wait(&full[s], par) && !mbar_wait(&full[s], par, p.error, ERR_MMA_WAIT)) { ok = false; break; }
                tc_fence_after();
                const uint64_t da = desc0 + (uint64_t)(s * stage_step), db = da + (uint64_t)b_step;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    mma_bf16_ss(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                if (s & 1) tc_commit(&empty[s >> 1]);     // the pair is free once these MMAs have read it
                if (++s == STAGES) { s = 0; par ^= 1u; }
            }
            tc_commit(&acc_full[buf]);                    // the accumulator is complete
        }
        if (!ok) {
            // whatever was loaded last must have landed before shared memory is given up
            for (int s = 0; s < STAGES; ++s)
                for (int par = 0; par < 2; ++par)
                    if (mbar_try_wait(&full[s], par)) break;
#pragma unroll 1
            for (unsigned spin = 0; spin < 4096; ++spin) __nanosleep(256);
        }
    } else if (warp >= 2) {
        // -------------------------------------------------------------------- epilogue
        const int quarter = warp & 3;                     // the 32 TMEM lanes this warp may read
        bool ok = true;
        int t = 0;
        pdl_wait();                                       // out, workspace and counters belong to earlier kernels till now
        const bool atomic_out = p.splits > 1 && p.epilogue == EPI_RESIDUAL;
        for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++t) {
            const int a0 = (tile % p.tiles_a) * p.a_box, b0 = (tile / p.tiles_a) * BN;
            // lanes beyond the rows this tile loaded hold nothing of this tile
            const int ra = quarter * 32 + lane < p.a_box ? a0 + quarter * 32 + lane : 0x3fffffff;
            const int buf = t & 1, use = t >> 1;
            // (also for a K slice that got no k-block: the MMA thread commits at once, but it must
            // have passed its own wait on `acc_empty` before these warps arrive there, or it would
            // wait for a phase that never comes)
            if (ok) ok = mbar_wait(&acc_full[buf], use & 1, p.error, ERR_EPILOGUE_WAIT);
            tc_fence_after();
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + buf * C::ACC_COLS;
            const bool have = ok && n_kb > 0;
            bool last = true;
            if (atomic_out) {
                // K slices of a product that is added into the fp32 stream: every slice adds
                // its own part, no meeting point needed (the order of the adds is not fixed)
                last = false;
                float* h = reinterpret_cast<float*>(p.out);
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    float v[16];
                    if (!have) break;
                    tmem_ld16(taddr + c0, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = p.swap ? b0 + c0 + j : ra, feat = p.swap ? ra : b0 + c0 + j;
                        const int n_tok = p.swap ? p.b_rows : p.a_rows, n_feat = p.swap ? p.a_rows : p.b_rows;
                        if (tok < n_tok && feat < n_feat) atomicAdd(h + (size_t)tok * p.ld_out + feat, v[j]);
                    }
                }
            } else if (p.splits > 1) {
                // park this slice's partial tile, then find out whether we are the last slice
                float* mine = p.workspace + ((size_t)tile * p.splits + blockIdx.z) * (BN * 128);
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    float v[16];
                    if (have) tmem_ld16(taddr + c0, v);
                    else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) mine[(size_t)(c0 + j) * 128 + quarter * 32 + lane] = v[j];
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) *ticket_slot = atomicAdd(&p.counters[tile], 1);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                last = *ticket_slot == p.splits - 1;
                if (last) {
                    __threadfence();
                    if (threadIdx.x == 64) p.counters[tile] = 0;
                }
            }
            if (last) {
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    float v[16];
                    if (p.splits > 1) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
                        const float* base = p.workspace + (size_t)tile * p.splits * (BN * 128) + quarter * 32 + lane;
                        for (int s = 0; s < p.splits; ++s)
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                v[j] += __ldcg(base + (size_t)s * (BN * 128) + (size_t)(c0 + j) * 128);
                    } else if (have) {
                        tmem_ld16(taddr + c0, v);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
                    }
                    if (!p.swap) {
                        store_row16(p, ra, b0 + c0, v);
                    } else if (p.epilogue == EPI_SILU) {
                        // lanes alternate gate, up: the even lane needs its odd neighbour's value
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
                            store_one(p, p.b_rows, p.a_rows, b0 + c0 + j, ra, v[j], other);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) store_one(p, p.b_rows, p.a_rows, b0 + c0 + j, ra, v[j], 0.f);
                    }
                }
            }
            // this accumulator may be overwritten by the tile after next
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)C::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host: tensor maps
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(sym);
    }
    return fn;
}

struct MapKey {
    const void* ptr; int rows, cols, box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        h ^= ((size_t)k.rows * 0x9E3779B97F4A7C15ull) ^ ((size_t)k.cols << 21) ^ ((size_t)k.box_rows << 43);
        return h;
    }
};

// A row-major bf16 matrix [rows][cols] seen as tiles of box_rows x 64 elements with the
// 128-byte swizzle; rows and columns outside the matrix read as zero.
int make_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    std::lock_guard<std::mutex> lock(mu);
    const MapKey key{ptr, rows, cols, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiled fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}


// ------------------------------------------------------------ a 256 x 256 tile on a CTA pair
// Many tokens (prefill): what limits the one-CTA kernel is operand traffic, 48 KB from L2 per
// 128 x 256 x 64 block and SM.  Here two CTAs of a cluster share a 256 x 256 tile: each loads
// its own 128 rows of activations and HALF of the 256 weight rows (32 KB per block), and one
// thread of the even CTA issues tcgen05.mma.cta_group::2, which reads A from each CTA's own
// shared memory, the two halves of B from both, and writes each CTA's 128 x 256 accumulator into
// its own tensor memory.  Barriers: TMA copies of both CTAs complete on the even CTA's `full`
// (its address with the peer bit cleared); tcgen05.commit with a two-CTA multicast frees the
// stages and publishes the accumulator in both; the odd CTA's epilogue warps arrive on the even
// CTA's `acc_empty` through its cluster address.  Every wait on an mbarrier is bounded.
constexpr int PAIR_BN = 256;
constexpr unsigned PEER_BIT_MASK = 0xFEFFFFFFu;          // shared::cluster address of the even CTA's copy

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar) & PEER_BIT_MASK), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void mma_bf16_ss_pair(unsigned tmem_d, uint64_t a, uint64_t b, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}
// arrive on the barrier at the same offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, unsigned rank) {
    asm volatile("{\n\t.reg .b32 ra;\n\t"
                 "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
                 "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
                 ::"r"(smem_u32(bar)), "r"(rank) : "memory");
}

// The rotary epilogue of one warp's 32 token rows of a tile, columns [b0, b0 + width): whole heads
// (the width and b0 are multiples of the head size).  A thread owns a token's row; the halves of a
// head that the rotation pairs up, (i, i + head_dim / 2), both lie in its accumulator row.  32
// columns of each half at a time: RustInfer rotates q and k in place after the product has
// rounded them to bf16 (crates/infer-backend-cuda/src/kernels/rope/rope.cu:107-132); here the fp32
// accumulator is rotated and rounded once, as in the few-token chain.
struct RopeRow {                    // what a thread needs of its token before the accumulator is there
    bool live;
    int slot;
    const float* ct;
    const float* st;
    float c[32], s[32];             // cos and sin of the first 32 pairs of a head at the token's position
};
__device__ __forceinline__ void rope_row_begin(const Params& p, int tok, RopeRow& r) {
    const int half = p.rope_hd >> 1;
    r.live = tok < p.a_rows;
    const int pos = r.live ? p.rope_positions[tok] : 0;
    r.slot = (r.live && p.rope_slot) ? p.rope_slot[tok] : -1;
    r.ct = p.rope_cos + (size_t)pos * half;
    r.st = p.rope_sin + (size_t)pos * half;
#pragma unroll
    for (int k = 0; k < 32; k += 4) {
        *reinterpret_cast<float4*>(r.c + k) = *reinterpret_cast<const float4*>(r.ct + k);
        *reinterpret_cast<float4*>(r.s + k) = *reinterpret_cast<const float4*>(r.st + k);
    }
}
__device__ __forceinline__ void rope_rows(const Params& p, unsigned taddr, int tok, int b0, int width, RopeRow& r) {
    const int hd = p.rope_hd, half = hd >> 1;
    const bool live = r.live;
    bf16* kdst = nullptr;
    bf16* vdst = nullptr;
    if (r.slot >= 0) {
        const int page = r.slot / p.rope_page, off = r.slot - page * p.rope_page;
        kdst = p.rope_cache + ((size_t)(page * 2 + 0) * p.rope_hkv * p.rope_page + off) * hd;
        vdst = p.rope_cache + ((size_t)(page * 2 + 1) * p.rope_hkv * p.rope_page + off) * hd;
    }
    const size_t head_step = (size_t)p.rope_page * hd;
    bf16* qrow = reinterpret_cast<bf16*>(p.out) + (size_t)tok * p.ld_out;
    // 32 pairs at a time over all heads of the tile: their cos and sin are the same for every head
#pragma unroll 1
    for (int i0 = 0; i0 < half; i0 += 32) {
        if (i0 > 0) {
#pragma unroll
            for (int k = 0; k < 32; k += 4) {
                *reinterpret_cast<float4*>(r.c + k) = *reinterpret_cast<const float4*>(r.ct + i0 + k);
                *reinterpret_cast<float4*>(r.s + k) = *reinterpret_cast<const float4*>(r.st + i0 + k);
            }
        }
#pragma unroll 1
        for (int c0 = 0; c0 < width && b0 + c0 < p.b_rows; c0 += hd) {
            const int head = (b0 + c0) / hd;
            if (head < p.rope_hq + p.rope_hkv) {
                bf16* dst = head < p.rope_hq ? qrow + (size_t)head * hd
                                             : (kdst ? kdst + (size_t)(head - p.rope_hq) * head_step : nullptr);
                float lo[32], hi[32];
                tmem_ld_row<32>(taddr + c0 + i0, lo);                 // every lane of the warp takes part
                tmem_ld_row<32>(taddr + c0 + half + i0, hi);
                if (live && dst) {
#pragma unroll
                    for (int k = 0; k < 32; ++k) {
                        const float y1 = lo[k] * r.c[k] - hi[k] * r.s[k];
                        hi[k] = lo[k] * r.s[k] + hi[k] * r.c[k];
                        lo[k] = y1;
                    }
#pragma unroll
                    for (int k = 0; k < 32; k += 8) {
                        *reinterpret_cast<uint4*>(dst + i0 + k) = pack8(lo + k);
                        *reinterpret_cast<uint4*>(dst + half + i0 + k) = pack8(hi + k);
                    }
                }
            } else if (i0 == 0) {
                bf16* dst = vdst ? vdst + (size_t)(head - p.rope_hq - p.rope_hkv) * head_step : nullptr;
#pragma unroll 1
                for (int j0 = 0; j0 < hd; j0 += 32) {
                    float v[32];
                    tmem_ld_row<32>(taddr + c0 + j0, v);
                    if (live && dst) {
#pragma unroll
                        for (int k = 0; k < 32; k += 8) *reinterpret_cast<uint4*>(dst + j0 + k) = pack8(v + k);
                    }
                }
            }
        }
    }
}

// What a pair works on next: a whole tile, or a run of k-blocks of one of the dealt-out tiles.
struct PairItem { int tile, kb0, kb1, part; };
// first k-block (counted through the dealt-out tiles) of a pair's run
__device__ __forceinline__ int sk_start(const Params& p, int pair) {
    return pair * p.sk_q + min(pair, p.sk_extra);
}
// the pair whose run holds k-block `step`
__device__ __forceinline__ int sk_pair_of(const Params& p, int step) {
    const int wide = p.sk_extra * (p.sk_q + 1);
    return step < wide ? step / (p.sk_q + 1) : p.sk_extra + (step - wide) / p.sk_q;
}
// Item `idx` of a pair: first its share of the dealt-out tiles (their sums are finished by
// whichever pair comes last, behind the whole tiles that follow), then whole tiles pair, pair + pairs, ...
__device__ __forceinline__ bool pair_item(const Params& p, int pair, int pairs, int n_kb, int idx, PairItem& it) {
    const int whole = p.n_tiles - p.sk_tiles;
    int n_seg = 0;
    if (p.sk_tiles > 0 && pair < p.sk_pairs) {
        const int s0 = sk_start(p, pair), s1 = sk_start(p, pair + 1);
        const int r = s0 / n_kb, k0 = s0 - r * n_kb;
        const int len0 = min(s1 - s0, n_kb - k0);
        n_seg = len0 < s1 - s0 ? 2 : 1;
        if (idx == 0) { it.tile = whole + r; it.kb0 = k0; it.kb1 = k0 + len0; it.part = 1; return true; }
        if (idx == 1 && n_seg == 2) { it.tile = whole + r + 1; it.kb0 = 0; it.kb1 = s1 - s0 - len0; it.part = 1; return true; }
    }
    const int tile = pair + (idx - n_seg) * pairs;
    if (tile >= whole) return false;
    it.tile = tile; it.kb0 = 0; it.kb1 = n_kb; it.part = 0;
    return true;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const Params p) {
    constexpr int ACC_COLS = 256, TMEM_COLS = 512;
    const int BN = p.pair_bn, HALF_BN = BN >> 1;                  // 128 to 256, whichever evens out the waves
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int STAGES = p.stages, STAGE_BYTES = p.stage_bytes;       // A 128 x 64 and half of B, up to 128 x 64: 32 KB
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + p.budget + SMEM_TAIL);
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* acc_full = empty + MAX_STAGES;
    uint64_t* acc_empty = acc_full + 2;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int n_kb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((unsigned)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        const unsigned pair_tx = 2u * (unsigned)STAGE_BYTES;          // both CTAs' copies land on the even CTA's barrier
        pdl_trigger();
        pdl_wait();
        bool ok = true;
        int it = 0, s = 0;
        unsigned par = 1;
        PairItem item;
        for (int idx = 0; ok && pair_item(p, pair, pairs, n_kb, idx, item); ++idx) {
            const int tile = item.tile;
            const int a0 = (tile % p.tiles_a) * 256 + (int)rank * BM, b0 = (tile / p.tiles_a) * BN + (int)rank * HALF_BN;
            for (int i = item.kb0; i < item.kb1; ++i, ++it) {
                unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                if (it >= STAGES && (s & 1) == 0 &&
                    !mbar_try_wait(&empty[s >> 1], par) && !mbar_wait(&empty[s >> 1], par, p.error, ERR_PRODUCER_WAIT)) { ok = false; break; }
                if (rank == 0) mbar_expect_tx(&full[s], pair_tx);
                tma_load_2d_pair(st, &map_a, &full[s], i * BK, a0);
                tma_load_2d_pair(st + BM * BK * 2, &map_b, &full[s], i * BK, b0);
                if (++s == STAGES) { s = 0; par ^= 1u; }
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ------------------------------------------------------------ MMA issuer (even CTA only)
        // D fp32, A and B bf16, both K-major, N = the tile's width, M = 256 over the two CTAs
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(256 >> 4) << 24);
        const uint64_t desc0 = smem_desc(smem_u32(tiles));
        const unsigned stage_step = (unsigned)STAGE_BYTES >> 4, b_step = (unsigned)(BM * BK * 2) >> 4;
        bool ok = true;
        int s = 0, t = 0;
        unsigned par = 0;
        PairItem item;
        for (int idx = 0; ok && pair_item(p, pair, pairs, n_kb, idx, item); ++idx, ++t) {
            const int buf = t & 1, use = t >> 1;
            if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, p.error, ERR_MMA_WAIT)) { ok = false; break; }
            tc_fence_after();
            const unsigned tmem_d = tmem_base + buf * ACC_COLS;
            for (int i = item.kb0; i < item.kb1; ++i) {
                if (!mbar_try_wait(&full[s], par) && !mbar_wait(&full[s], par, p.error, ERR_MMA_WAIT)) { ok = false; break; }
                tc_fence_after();
                const uint64_t da = desc0 + (uint64_t)(s * stage_step), db = da + (uint64_t)b_step;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    mma_bf16_ss_pair(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > item.kb0 || k > 0) ? 1u : 0u);
                if (s & 1) tc_commit_pair(&empty[s >> 1]);
                if (++s == STAGES) { s = 0; par ^= 1u; }
            }
            tc_commit_pair(&acc_full[buf]);
        }
        if (!ok) {
            for (int st = 0; st < STAGES; ++st)
                for (int q = 0; q < 2; ++q)
                    if (mbar_try_wait(&full[st], q)) break;
#pragma unroll 1
            for (unsigned spin = 0; spin < 4096; ++spin) __nanosleep(256);
        }
    } else if (warp >= 2) {
        // -------------------------------------------------------------------- epilogue (both CTAs)
        const int quarter = warp & 3;
        bool ok = true;
        int t = 0;
        pdl_wait();
        PairItem item;
        for (int idx = 0; pair_item(p, pair, pairs, n_kb, idx, item); ++idx, ++t) {
            const int tile = item.tile;
            const int a0 = (tile % p.tiles_a) * 256 + (int)rank * BM, b0 = (tile / p.tiles_a) * BN;
            const int ra = a0 + quarter * 32 + lane;
            const int buf = t & 1, use = t >> 1;
            RopeRow rr;
            if (p.epilogue == EPI_ROPE) rope_row_begin(p, ra, rr);      // the table's rows come while the tile is computed
            if (ok) ok = mbar_wait(&acc_full[buf], use & 1, p.error, ERR_EPILOGUE_WAIT);
            tc_fence_after();
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + buf * ACC_COLS;
            // Part of a tile's sum over K.  Added into the fp32 stream it needs no meeting point
            // (the stores below are reductions at the memory side).  Otherwise the part goes to
            // this pair's slot of the meeting buffer, and the warp that comes last (a ticket per
            // tile, CTA and warp: the same rows come from the same warp of every pair) adds the
            // parts in the order of the pairs, so the sum does not depend on who came last.  The
            // accumulator in tensor memory is given back before that: the whole tiles that follow
            // hide the meeting.
            const bool meet = item.part && p.epilogue != EPI_RESIDUAL;
            const int sk_tile = tile - (p.n_tiles - p.sk_tiles);
            const size_t warp_floats = (size_t)BN * 32, slot_floats = warp_floats * 8;
            const size_t warp_off = (size_t)((int)rank * 4 + quarter) * warp_floats + lane * 4;
            bool finish = ok;
            int first_pair = 0, parts = 0;
            if (meet && ok) {
                const int seg = sk_start(p, pair) < sk_tile * n_kb ? 1 : 0;      // this tile is the second one of the run
                float* mine = p.sk_acc + (size_t)(pair * 2 + seg) * slot_floats + warp_off;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    float v[64];
                    tmem_ld_row<64>(taddr + c0, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        __stcg(reinterpret_cast<float4*>(mine + (size_t)(c0 / 4 + j) * 128),
                               make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
                }
                // (the accumulator is free as soon as it is in registers; the fence below waits
                // for the stores, and the MMA thread should not wait with it)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(&acc_empty[buf], 0);
                __threadfence();
                __syncwarp();
                first_pair = sk_pair_of(p, sk_tile * n_kb);
                parts = sk_pair_of(p, sk_tile * n_kb + n_kb - 1) - first_pair + 1;
                const int slot = (sk_tile * 2 + (int)rank) * 4 + quarter;
                int ticket = 0;
                if (lane == 0) ticket = atomicAdd(&p.counters[slot], 1);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                finish = ticket == parts - 1;
                if (finish) {
                    __threadfence();
                    if (lane == 0) p.counters[slot] = 0;
                }
            }
            if (finish && p.epilogue == EPI_ROPE) {
                rope_rows(p, taddr, ra, b0, BN, rr);
            } else if (finish) {
                // 64 columns a round trip to tensor memory where the tile lies inside the matrix:
                // the epilogue of a pair's last tile has no MMA to hide behind.  At the ragged
                // edge 16 at a time, element by element.
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    float v[64];
                    if (meet) {
#pragma unroll
                        for (int j = 0; j < 64; ++j) v[j] = 0.f;
#pragma unroll 1
                        for (int pr = first_pair; pr < first_pair + parts; ++pr) {
                            const int seg = sk_start(p, pr) < sk_tile * n_kb ? 1 : 0;
                            const float* src = p.sk_acc + (size_t)(pr * 2 + seg) * slot_floats + warp_off;
                            float4 x[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) x[j] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(c0 / 4 + j) * 128));
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                v[4 * j] += x[j].x; v[4 * j + 1] += x[j].y; v[4 * j + 2] += x[j].z; v[4 * j + 3] += x[j].w;
                            }
                        }
                    } else {
                        tmem_ld_row<64>(taddr + c0, v);
                    }
                    if (p.vec && b0 + c0 + 64 <= p.b_rows) {
                        store_row64(p, ra, b0 + c0, v);
                    } else {
#pragma unroll
                        for (int c1 = 0; c1 < 64; c1 += 16) {
                            float w[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) w[j] = v[c1 + j];
                            store_row16(p, ra, b0 + c0 + c1, w);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0 && !(meet && ok)) mbar_arrive_remote(&acc_empty[buf], 0);   // the even CTA's MMA thread counts all eight warps
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // neither CTA leaves while the other may still touch it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)TMEM_COLS) : "memory");
    }
}

int device_sms() { return ri_device_sms(); }

int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int sms = device_sms();
    const int pairs = (p.sk_tiles == 0 && p.n_tiles < sms / 2) ? p.n_tiles : sms / 2;
    RI_CHECKED(ri_launch(gemm_tc_pair_kernel, dim3(2 * pairs), dim3(THREADS), (size_t)p.budget + SMEM_EXTRA, s, ma, mb, p));
    return ri_launch_status();
}
}  // namespace

int ri_tc_weight_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out) {
    return make_map(ptr, rows, cols, box_rows, out);
}

namespace {
template <int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, int tiles, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)SMEM_TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int sms = device_sms();
    // one CTA per SM walks the tiles; with K slices every CTA has exactly one tile
    const int ctas = (p.splits > 1 || tiles < sms) ? tiles : sms;
    RI_CHECKED(ri_launch(gemm_tc_kernel<BN>, dim3(ctas, 1, p.splits), dim3(THREADS), (size_t)p.budget + SMEM_EXTRA, s, ma, mb, p));
    return ri_launch_status();
}
}  // namespace

// Floats of workspace a call may need: tiles * splits * BN * 128 (0 when splits == 1).
RI_API long long ri_gemm_tc_workspace_floats(int M, int N, int splits, int swap, int bn) {
    if (splits <= 1) return 0;
    const int a_rows = swap ? N : M, b_rows = swap ? M : N;
    const long long tiles = (long long)((a_rows + BM - 1) / BM) * ((b_rows + bn - 1) / bn);
    return tiles * splits * bn * 128;
}

// X [M][K] bf16 (row pitch K), W [N][K] bf16; out per `epilogue`:
//   0 bf16 [M][ld_out], 1 fp32 [M][ld_out], 2 bf16 [M][ld_out] = silu(gate)*up with W's rows
//   alternating gate_j, up_j (N = 2 * features of out), 3 fp32 [M][ld_out] += result.
// swap: 1 puts the weight on the 128-row side of the MMA (few tokens), 0 the activations.
// bn: rows of the other operand per tile (16, 32, 64, 128 or 256).  counters: one int per
// tile, zero before the first call (the kernel leaves them zero).  error: one int that a
// timed-out wait sets; zero it before use and read it when in doubt.
RI_API void ri_set_pdl(int on) { ri_pdl_flag() = on ? 1 : 0; }

// Bytes of operand stages a CTA keeps when few tokens stream the weights (16 KiB to 200 KiB).
RI_API void ri_gemm_tc_set_stream_budget(int bytes) {
    if (bytes >= 16 * 1024 && bytes <= SMEM_BUDGET) g_stream_budget = bytes & ~1023;
}

// a_box: rows of the 128-row operand a tile really covers (a multiple of 8 from 8 to 128;
// fewer than 128 evens out the last wave of tiles over the SMs).
// sk_acc: SMs x 65536 floats where the parts of tiles that several CTA pairs share meet (two
// 256 x 256 fp32 tiles a pair); null: every tile stays with one pair.
namespace {
int gemm_tc_impl(const void* X, const void* W, int M, int N, int K, void* out, int ld_out, int epilogue,
                 int swap, int bn, int splits, int a_box, float* workspace, int* counters, int* error,
                 float* sk_acc, const Params* rope, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || splits < 1 || (splits > 1 && (!workspace || !counters)) || !error ||
        a_box < 8 || a_box > BM || a_box % 8 != 0)
        return (int)cudaErrorInvalidValue;
    const void* A = swap ? W : X;
    const void* B = swap ? X : W;
    Params p;
    p.pair_bn = 0;
    p.sk_tiles = p.sk_pairs = p.sk_q = p.sk_extra = 0; p.sk_acc = nullptr;
    p.rope_positions = nullptr; p.rope_cos = p.rope_sin = nullptr; p.rope_slot = nullptr; p.rope_cache = nullptr;
    p.rope_hq = p.rope_hkv = p.rope_hd = p.rope_page = 0;
    if (rope) {
        p.rope_positions = rope->rope_positions; p.rope_cos = rope->rope_cos; p.rope_sin = rope->rope_sin;
        p.rope_slot = rope->rope_slot; p.rope_cache = rope->rope_cache;
        p.rope_hq = rope->rope_hq; p.rope_hkv = rope->rope_hkv; p.rope_hd = rope->rope_hd; p.rope_page = rope->rope_page;
        sk_acc = nullptr;                                  // whole heads stay with one pair
    }
    p.a_rows = swap ? N : M;
    p.b_rows = swap ? M : N;
    p.K = K; p.swap = swap; p.epilogue = epilogue; p.out = out; p.ld_out = ld_out; p.splits = splits;
    p.workspace = workspace; p.counters = counters; p.error = error;
    p.tiles_a = (p.a_rows + BM - 1) / BM;
    const int tiles_b = (p.b_rows + bn - 1) / bn;
    p.n_tiles = p.tiles_a * tiles_b;
    const int esize = (epilogue == EPI_BF16 || epilogue == EPI_SILU) ? 2 : 4;
    p.vec = ((reinterpret_cast<uintptr_t>(out) & 15) == 0 && ((size_t)ld_out * esize) % 16 == 0) ? 1 : 0;
    CUtensorMap ma, mb;
    p.a_box = a_box;
    p.stage_bytes = (a_box + bn) * BK * 2;
    p.budget = (swap && bn <= 64) ? g_stream_budget : SMEM_BUDGET;
    // a long weight stream per CTA (the head over a large vocabulary) is worth a deeper ring than
    // the half-SM one that lets the next product move in early: 525 MB at batch 8 took 98 us with
    // 96 KB and 85.7 us (6.1 TB/s) with 160 KB
    if (swap && bn <= 64 && g_stream_budget < SMEM_BUDGET_LONG &&
        (double)p.a_rows * K * 2 / (double)device_sms() > 1048576.0) p.budget = SMEM_BUDGET_LONG;
    p.stages = p.budget / p.stage_bytes;
    if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
    p.stages &= ~1;                                       // stages are released in pairs
    if (p.stages < 2) return (int)cudaErrorInvalidValue;
    p.tiles_a = (p.a_rows + a_box - 1) / a_box;
    p.n_tiles = p.tiles_a * tiles_b;
    // many tokens: a 256 x 256 tile on a CTA pair (less operand traffic per flop)
    static const bool pair_off = getenv("RUSTINFER_B200_GEMM_PAIR") && atoi(getenv("RUSTINFER_B200_GEMM_PAIR")) == 0;
    if (!swap && bn == PAIR_BN && splits == 1 && a_box == BM && !pair_off && p.a_rows >= 512) {
        // A tile is 256 rows by 256 columns, or by 192 where that fills the waves better.  The
        // k-blocks of a last wave that would leave pairs idle can be dealt out over all pairs
        // (3072 features of 2048 tokens, K = 8192: 96 tiles of 256 on 74 pairs are two waves,
        // 256 k-blocks a pair; dealt out, 74 whole tiles and 22 x 128 / 74 = 38 k-blocks each).
        // A k-block costs a pair about the same time at both widths, so the count decides.
        // Dealing is not free: every part is a whole 256 x 256 fp32 tile that has to go
        // somewhere.  A product that is added into the fp32 stream adds its parts where the
        // whole would go (reductions at the memory side, measured to cost about 24 k-blocks);
        // any other one leaves them in the buffer, and the pairs that finish a tile read four or
        // five parts back from L2 under the operands' traffic (about 40 k-blocks).  So only a
        // long K with a short last wave is dealt: the 3B shape's down projection, 97 -> 79 us.
        p.tiles_a = (p.a_rows + 255) / 256;
        const int pairs = device_sms() / 2;
        const int n_kb = (K + BK - 1) / BK;
        const int meeting = epilogue == EPI_RESIDUAL ? 24 : 40;
        static const bool deal_off = getenv("RUSTINFER_B200_GEMM_DEAL") && atoi(getenv("RUSTINFER_B200_GEMM_DEAL")) == 0;
        if (deal_off) sk_acc = nullptr;
        long long best = -1;
        for (int w : {256, 192}) {
            if (rope && w % p.rope_hd != 0) continue;      // a tile holds whole heads
            const int tiles = p.tiles_a * ((p.b_rows + w - 1) / w);
            const int waves = tiles / pairs, rest = tiles % pairs;
            for (int deal = 0; deal < 2; ++deal) {
                // (a run of k-blocks meets two tiles at most)
                if (deal && (rest == 0 || !sk_acc || n_kb < 8 || waves == 0)) continue;
                long long cost;
                int q = 0, extra = 0, takers = 0;
                if (!deal) {
                    cost = (long long)(waves + (rest ? 1 : 0)) * n_kb * 16;
                } else {
                    const int steps = rest * n_kb;
                    takers = steps / 4 < pairs ? steps / 4 : pairs;       // at least four k-blocks a pair
                    if (takers < 1) continue;
                    q = steps / takers; extra = steps % takers;
                    cost = ((long long)waves * n_kb + q + (extra ? 1 : 0) + meeting) * 16;
                }
                cost += w == 192 ? 1 : 0;                                  // equal counts: the wider tile
                if (best < 0 || cost < best) {
                    best = cost; p.pair_bn = w;
                    p.sk_tiles = deal ? rest : 0; p.sk_pairs = takers; p.sk_q = q; p.sk_extra = extra;
                }
            }
        }
        p.sk_acc = sk_acc;
        p.stage_bytes = (BM + p.pair_bn / 2) * BK * 2;
        p.stages = (p.budget / p.stage_bytes) & ~1;
        if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
        p.n_tiles = p.tiles_a * ((p.b_rows + p.pair_bn - 1) / p.pair_bn);
        int stp = make_map(A, p.a_rows, K, BM, &ma);
        if (stp != 0) return stp;
        stp = make_map(B, p.b_rows, K, p.pair_bn / 2, &mb);
        if (stp != 0) return stp;
        return launch_pair(ma, mb, p, (cudaStream_t)stream);
    }
    if (rope) return (int)cudaErrorNotSupported;           // only the CTA-pair kernel has that epilogue
    int st = make_map(A, p.a_rows, K, a_box, &ma);
    if (st != 0) return st;
    st = make_map(B, p.b_rows, K, bn, &mb);
    if (st != 0) return st;
    cudaStream_t s = (cudaStream_t)stream;
    const int tiles = p.n_tiles;
    switch (bn) {
        case 16: return launch<16>(ma, mb, p, tiles, s);
        case 32: return launch<32>(ma, mb, p, tiles, s);
        case 64: return launch<64>(ma, mb, p, tiles, s);
        case 128: return launch<128>(ma, mb, p, tiles, s);
        case 256: return launch<256>(ma, mb, p, tiles, s);
    }
    return (int)cudaErrorInvalidValue;
}
}  // namespace

RI_API int ri_gemm_tc(const void* X, const void* W, int M, int N, int K, void* out, int ld_out, int epilogue,
                      int swap, int bn, int splits, int a_box, float* workspace, int* counters, int* error,
                      float* sk_acc, void* stream) {
    if (epilogue == EPI_ROPE) return (int)cudaErrorInvalidValue;       // has an entry of its own
    return gemm_tc_impl(X, W, M, N, K, out, ld_out, epilogue, swap, bn, splits, a_box, workspace, counters, error,
                        sk_acc, nullptr, stream);
}

// q, k, v of many tokens with the rotary encoding and the cache write in the product's epilogue
// (CTA pairs: 512 tokens or more).  X [M][K] bf16, W [N][K] bf16 with N = (Hq + 2 Hkv) head_dim
// rows, or Hq head_dim when the layer keeps no keys (slot_of_token and cache null, Hkv 0).  q_out
// bf16 [M][ld_q] gets the rotated q heads; k (rotated) and v go to the token's slot of the cache
// [page][K|V][kv head][slot][head_dim] (slot < 0: not written).  cos, sin: fp32 [positions][head_dim / 2].
// Head sizes 64 and 128, the whole head rotated.  cudaErrorNotSupported (801) where the pair kernel does
// not take the product: the caller then runs the product and the rotary kernel one after the other.
RI_API int ri_gemm_tc_rope(const void* X, const void* W, int M, int N, int K, void* q_out, int ld_q,
                           const int* positions, const float* cos_t, const float* sin_t, const int* slot_of_token,
                           void* cache, int Hq, int Hkv, int head_dim, int page_size, int* counters, int* error,
                           void* stream) {
    if (M <= 0) return 0;
    if ((head_dim != 64 && head_dim != 128) || Hq <= 0 || Hkv < 0 || N != (Hq + 2 * Hkv) * head_dim || !positions ||
        !cos_t || !sin_t || (Hkv > 0 && (!slot_of_token || !cache || page_size <= 0)) || ld_q % 8 != 0 ||
        (reinterpret_cast<uintptr_t>(q_out) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
        (reinterpret_cast<uintptr_t>(cos_t) & 15) || (reinterpret_cast<uintptr_t>(sin_t) & 15))
        return (int)cudaErrorInvalidValue;
    if (M < 512 || N < PAIR_BN) return (int)cudaErrorNotSupported;
    Params r;
    r.rope_positions = positions; r.rope_cos = cos_t; r.rope_sin = sin_t;
    r.rope_slot = Hkv > 0 ? slot_of_token : nullptr; r.rope_cache = (bf16*)cache;
    r.rope_hq = Hq; r.rope_hkv = Hkv; r.rope_hd = head_dim; r.rope_page = page_size;
    return gemm_tc_impl(X, W, M, N, K, q_out, ld_q, EPI_ROPE, 0, PAIR_BN, 1, BM, nullptr, counters, error, nullptr, &r, stream);
}
