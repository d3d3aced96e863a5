// Paged causal GQA attention for prompt portions on the 5th-generation tensor cores:
// S = Q K^T and O_tile = P V are tcgen05.mma instructions with fp32 accumulators in tensor
// memory; K and V tiles are fetched page by page with TMA straight from the paged cache
// (a box per page and kv head); the softmax runs in registers, one thread per query row.
// Compiled for one RI_HEAD_DIM (64 or 128).
//
// RustInfer's ragged attention is an mma.sync kernel with one CTA per q head that gathers
// keys token by token (crates/infer-backend-cuda/src/kernels/flash_attn_gqa/
// flash_attn_paged_prefill.cu:316-520) or, on Hopper, vendored FlashAttention-3 (wgmma);
// neither exists for sm_100.  What is computed is the same: row (token, q head) sees keys
// 0..position (or a window), scores scaled by 1/sqrt(head_dim) in base 2, probabilities
// rounded to bf16 for P V, fp32 sums.
//
// One CTA = 128 rows x one kv head; a row is (query token, q head of the kv head's group),
// so the group's heads share every K/V tile.  192 threads:
//   warp 0      TMA producer (one thread): K and V boxes of each 64-key tile, 3 stages each
//   warp 1      tensor memory allocation; one thread issues the MMAs, S of tile j+1 before
//               P V of tile j, so the tensor core computes scores while the softmax of the
//               tile before is still running
//   warps 2-5   softmax: thread = row; tcgen05.ld of the row's 64 scores, online softmax,
//               P (bf16) written to swizzled shared memory as the A operand of P V.  The
//               output accumulates in tensor memory across tiles; it is rescaled (load,
//               multiply, store) only when a row's maximum has grown by more than 2^8 since
//               the reference it was scaled to, which after the first tiles is rare
// Every wait on an mbarrier is bounded; a time-out leaves a code in *error and the kernel
// winds down (tensor memory freed, copies in flight drained).
#include "common.cuh"
#include "tc_primitives.cuh"
#include <cuda.h>
#include <mutex>
#include <type_traits>
#include <unordered_map>

#ifndef RI_HEAD_DIM
#error "compile with -DRI_HEAD_DIM=<head size>"
#endif
#ifndef RI_ATTN_POLY_OF
#define RI_ATTN_POLY_OF (RI_HEAD_DIM == 64 ? 3 : 0)
#endif

namespace {
using namespace ri_tc;                    // mbarriers with bounded waits, TMA loads, tcgen05 fences, commit, MMA
constexpr int HD = RI_HEAD_DIM;
static_assert(HD == 64 || HD == 128, "tcgen05 attention: head size 64 or 128");
constexpr int BM = 128;                   // rows per CTA (MMA M)
constexpr int BN = 64;                    // keys per tile
constexpr int KB = HD / 64;               // 64-wide column blocks of a head (one 128-byte swizzle row each)
constexpr int NS = 2;                     // stages of K and of V
constexpr int THREADS = 192;
constexpr int TMEM_COLS = HD == 64 ? 128 : 256;   // S: 64 columns, O: HD columns
constexpr int COL_S = 0, COL_O = BN;
constexpr float RESCALE_STEP = 8.0f;              // log2 of the growth of a row's maximum that forces a rescale

constexpr int Q_BYTES = BM * 128 * KB;            // [KB][128 rows][128 B]
constexpr int KV_STAGE = BN * 128 * KB;           // [KB][64 keys][128 B]
constexpr int P_BYTES = BM * 128;                 // [128 rows][64 keys] bf16
constexpr int OFF_Q = 0, OFF_K = OFF_Q + Q_BYTES, OFF_V = OFF_K + NS * KV_STAGE, OFF_P = OFF_V + NS * KV_STAGE;
constexpr int OFF_BAR = OFF_P + P_BYTES;
// No slack for rounding the base up: with heads of 128 two CTAs fit an SM only without it
// (2 x (112 KB + barriers + 1 KB the system keeps per CTA) of 228 KB).  A kernel without static
// shared memory gets its dynamic part on a 1024-byte boundary; the kernel checks that and refuses
// to run otherwise.
constexpr size_t SMEM = (size_t)OFF_BAR + 128;

enum { ERR_PRODUCER = 11, ERR_MMA = 12, ERR_SOFTMAX = 13, ERR_ALIGNMENT = 14 };

__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory descriptors, 128-byte swizzle, 8-row groups 1024 bytes apart.
//  K-major (rows of 64 contraction elements): Q, K and P.
__device__ __forceinline__ uint64_t desc_kmajor(unsigned addr) {
    return (uint64_t)((addr & 0x3ffff) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
//  MN-major (rows are keys = the contraction, 64 head dims contiguous): V as loaded from the
//  cache.  Leading offset: between 64-dim column blocks; stride offset: between 8-key groups.
__device__ __forceinline__ uint64_t desc_mnmajor(unsigned addr) {
    return (uint64_t)((addr & 0x3ffff) >> 4) | ((uint64_t)((BN * 128) >> 4) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void mma_ss(unsigned tmem_d, uint64_t a, uint64_t b, unsigned idesc, unsigned accumulate) {
    mma_bf16_ss(tmem_d, a, b, idesc, accumulate);
}
// 16 consecutive fp32 columns of this thread's lane into r[0..15] (complete after tmem_ld_wait)
__device__ __forceinline__ void tmem_ld16_issue(unsigned addr, float* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
                   "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
                 : "r"(addr));
}
// 64 consecutive fp32 columns in one instruction
__device__ __forceinline__ void tmem_ld64_issue(unsigned addr, float* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
        : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]),
          "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]),
          "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]),
          "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31]),
          "=f"(r[32]), "=f"(r[33]), "=f"(r[34]), "=f"(r[35]), "=f"(r[36]), "=f"(r[37]), "=f"(r[38]), "=f"(r[39]),
          "=f"(r[40]), "=f"(r[41]), "=f"(r[42]), "=f"(r[43]), "=f"(r[44]), "=f"(r[45]), "=f"(r[46]), "=f"(r[47]),
          "=f"(r[48]), "=f"(r[49]), "=f"(r[50]), "=f"(r[51]), "=f"(r[52]), "=f"(r[53]), "=f"(r[54]), "=f"(r[55]),
          "=f"(r[56]), "=f"(r[57]), "=f"(r[58]), "=f"(r[59]), "=f"(r[60]), "=f"(r[61]), "=f"(r[62]), "=f"(r[63])
        : "r"(addr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16(unsigned addr, const float* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(addr), "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]),
                   "f"(r[8]), "f"(r[9]), "f"(r[10]), "f"(r[11]), "f"(r[12]), "f"(r[13]), "f"(r[14]), "f"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 2^x on the special-function unit, one instruction (inputs here are <= 0 or -inf)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x for a pair of x <= 0 without the special-function unit: x = n + f with n the nearest
// integer, 2^f for f in [-0.5, 0.5] by a polynomial of degree 4 (relative error 2.7e-6, far
// inside the rounding of a probability to bf16), n added to the exponent.  The unit computes
// 16 exponentials a clock and SM; a third of a tile's go this way, on the fma pipe, beside it.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
    const float magic = 12582912.f;                            // 1.5 * 2^23: adding it rounds to an integer
    x.x = fmaxf(x.x, -126.f); x.y = fmaxf(x.y, -126.f);
    const float2 m2 = make_float2(magic, magic);
    const float2 xr = __fadd2_rn(x, m2);
    const float2 n = __fadd2_rn(xr, make_float2(-magic, -magic));
    const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
    float2 r = make_float2(0.009570098482072353f, 0.009570098482072353f);
    r = __ffma2_rn(r, f, make_float2(0.05591785907745361f, 0.05591785907745361f));
    r = __ffma2_rn(r, f, make_float2(0.240247443318367f, 0.240247443318367f));
    r = __ffma2_rn(r, f, make_float2(0.6931217908859253f, 0.6931217908859253f));
    r = __ffma2_rn(r, f, make_float2(0.9999992847442627f, 0.9999992847442627f));
    r.x = __int_as_float(__float_as_int(r.x) + (__float_as_int(xr.x) << 23));
    r.y = __int_as_float(__float_as_int(r.y) + (__float_as_int(xr.y) << 23));
    return r;
}
constexpr int POLY_OF = RI_ATTN_POLY_OF;   // one pair of every POLY_OF goes to the polynomial (0: none)

// the larger of three in one instruction
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

struct Params {
    const bf16* q; int q_stride;
    bf16* out; int out_stride;
    const int* block_table; int table_stride;
    const int* cu_q; const int* kv_len; const int* tile_entry; const int* tile_tok0;
    int Hq, Hkv, G, tpt, page_size, box_rows;
    float scale_log2; int window;
    int* error;
};

// three CTAs per SM for heads of 64, two for 128 (tensor memory, shared memory and registers
// allow it): the other CTAs' softmax fills the issue slots one leaves while it waits on its chain
__global__ void __launch_bounds__(THREADS, HD == 64 ? 3 : 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap cache_map, const Params p) {
    extern __shared__ __align__(1024) unsigned char sm[];
    if ((smem_u32(sm) & 1023u) != 0) {                         // the 128-byte swizzle wants 1024-byte tiles
        if (threadIdx.x == 0) atomicCAS(p.error, 0, ERR_ALIGNMENT);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + OFF_BAR);
    uint64_t* k_full = bars;              // [NS]
    uint64_t* k_empty = k_full + NS;      // [NS]
    uint64_t* v_full = k_empty + NS;      // [NS]
    uint64_t* v_empty = v_full + NS;      // [NS]
    uint64_t* s_full = v_empty + NS;      // scores of a tile are in tensor memory
    uint64_t* s_empty = s_full + 1;       // ... and have been read into registers
    uint64_t* p_full = s_empty + 1;       // probabilities of a tile are in shared memory
    uint64_t* p_empty = p_full + 1;       // ... and P V has read them
    uint64_t* o_done = p_empty + 1;       // P V of a tile has been added to the output
    uint64_t* q_ready = o_done + 1;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(q_ready + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTAs start in the order x fastest: all kv heads of the last tile first, the first tile
    // last.  In a causal prompt the late tiles see the most keys, so the long CTAs start
    // early and the short ones fill the end of the last wave.
    const int tile = gridDim.y - 1 - blockIdx.y;
    const int b = p.tile_entry[tile];
    const int tok0 = p.tile_tok0[tile];
    const int g = blockIdx.x;                                  // kv head
    const int q_begin = b >= 0 ? p.cu_q[b] : 0, q_len = b >= 0 ? p.cu_q[b + 1] - q_begin : 0;
    const int kvl = b >= 0 ? p.kv_len[b] : 0;
    const int pos0 = kvl - q_len;
    const int ntok = min(p.tpt, q_len - tok0);
    const int p_first = pos0 + tok0, p_last = p_first + ntok - 1;
    const int lo_tile = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
    const int t_begin = lo_tile / BN, t_end = p_last / BN + 1;
    const int n_tiles = (b >= 0 && ntok > 0) ? t_end - t_begin : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
        }
        mbar_init(s_full, 1); mbar_init(s_empty, 4);
        mbar_init(p_full, 4); mbar_init(p_empty, 1);
        mbar_init(o_done, 1);
        mbar_init(q_ready, 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((unsigned)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // The whole warp: lane 0 waits for a free stage and announces the bytes, then every box
        // of the tile goes out from a lane of its own.  A box is one page's keys (or values) of
        // one 64-column block, 2 KB with pages of 16; one thread sends a box every 74 ns, and 8 to
        // 16 boxes a tile from one thread were the period of the whole kernel (1.2 to 2.4 us a
        // tile against 0.2 to 0.4 us of tensor-core work).
        pdl_wait();                                            // the cache was written by the kernel before
        const int* bt = p.block_table + (size_t)b * p.table_stride;
        const int boxes = BN / p.box_rows;                     // at most 8 pages meet a tile
        bool ok = true;
        // Pages are smaller than a tile (a box per page, from its first key) or whole multiples
        // of it (one box, block and offset counted along).  Pages past the request's last one
        // are never allocated: its first page is read instead (those keys are masked, and their
        // V rows are zeroed before use).
        const bool small_pages = p.page_size < BN;
        int blk = (t_begin * BN) / p.page_size, off = small_pages ? 0 : (t_begin * BN) % p.page_size;
        const int kv_step = p.Hkv * p.page_size;               // rows between a page's keys and its values
        // this lane's box of a tile: page c of the tile, 64-column block kb.  The page number of the
        // next tile's box is read one tile ahead, so that no box waits for a look-up.
        const int c = lane / KB, kb = lane - c * KB;
        const bool mine = c < boxes;
        auto page_of = [&](int key0, int blk0) -> int {
            if (!mine) return 0;
            const bool live = key0 + c * p.box_rows < kvl;
            return bt[live ? blk0 + (small_pages ? c : 0) : 0];
        };
        int page = n_tiles > 0 ? page_of(t_begin * BN, blk) : 0;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int s = j % NS, u = j / NS;
            const int key0 = (t_begin + j) * BN;
            int blk_n = blk, off_n = off;
            if (small_pages) blk_n += boxes;
            else if ((off_n += BN) >= p.page_size) { off_n = 0; ++blk_n; }
            const int page_next = j + 1 < n_tiles ? page_of(key0 + BN, blk_n) : 0;
            const int row = (page * 2 * p.Hkv + g) * p.page_size + (key0 + c * p.box_rows < kvl ? off : 0);
            for (int kv = 0; kv < 2 && ok; ++kv) {
                uint64_t* full = kv ? &v_full[s] : &k_full[s];
                uint64_t* empty = kv ? &v_empty[s] : &k_empty[s];
                int good = 1;
                if (lane == 0) {
                    if (u > 0 && !mbar_wait(empty, (u - 1) & 1, p.error, ERR_PRODUCER)) good = 0;
                    if (good) mbar_expect_tx(full, KV_STAGE);
                }
                good = __shfl_sync(0xffffffffu, good, 0);
                if (!good) { ok = false; break; }
                if (mine)
                    tma_load_2d(sm + (kv ? OFF_V : OFF_K) + s * KV_STAGE + kb * (BN * 128) + c * p.box_rows * 128,
                                &cache_map, full, kb * 64, row + kv * kv_step);
            }
            page = page_next; blk = blk_n; off = off_n;
        }
    } else if (warp == 1 && lane == 0) {
        // -------------------------------------------------------------------- MMA issuer
        // D fp32, A and B bf16; S: both K-major, N = 64; P V: B is MN-major, N = HD
        const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
        const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
        const unsigned q_addr = smem_u32(sm + OFF_Q);
        bool ok = n_tiles > 0 && mbar_wait(q_ready, 0, p.error, ERR_MMA);
        auto issue_s = [&](int j) -> bool {
            const int s = j % NS, u = j / NS;
            if (!mbar_wait(&k_full[s], u & 1, p.error, ERR_MMA)) return false;
            if (!mbar_wait(s_empty, (j & 1) ^ 1, p.error, ERR_MMA)) return false;   // scores of tile j-1 were read
            tc_fence_after();
            const unsigned k_addr = smem_u32(sm + OFF_K + s * KV_STAGE);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    mma_ss(tmem_base + COL_S, desc_kmajor(q_addr + kb * (BM * 128) + k * 32),
                           desc_kmajor(k_addr + kb * (BN * 128) + k * 32), idesc_s, (kb > 0 || k > 0) ? 1u : 0u);
            tc_commit(&k_empty[s]);
            tc_commit(s_full);
            return true;
        };
        if (ok) ok = issue_s(0);
        for (int j = 0; j < n_tiles && ok; ++j) {
            if (j + 1 < n_tiles) ok = issue_s(j + 1);
            if (!ok) break;
            const int s = j % NS, u = j / NS;
            if (!mbar_wait(p_full, j & 1, p.error, ERR_MMA) ||
                !mbar_wait(&v_full[s], u & 1, p.error, ERR_MMA)) { ok = false; break; }
            tc_fence_after();
            const unsigned p_addr = smem_u32(sm + OFF_P);
            const unsigned v_addr = smem_u32(sm + OFF_V + s * KV_STAGE);
#pragma unroll
            for (int k = 0; k < BN / 16; ++k)                  // 16 keys per MMA: two 8-key groups of V
                mma_ss(tmem_base + COL_O, desc_kmajor(p_addr + k * 32), desc_mnmajor(v_addr + k * 2048),
                       idesc_o, (j > 0 || k > 0) ? 1u : 0u);
            tc_commit(&v_empty[s]);
            tc_commit(p_empty);
            tc_commit(o_done);
        }
    } else if (warp >= 2) {
        // ----------------------------------------------------------------------- softmax
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                     // this thread's row = its TMEM lane
        const int jj = r / p.G, hh = r - jj * p.G;
        const bool row_ok = n_tiles > 0 && jj < ntok;
        const int p_row = p_first + jj;
        const int lo_row = p.window > 0 ? max(0, p_row - p.window + 1) : 0;
        const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
        pdl_wait();
        // Q row into swizzled shared memory (chunk c of row r sits at chunk c ^ (r & 7))
        {
            const bf16* src = p.q + (size_t)(q_begin + tok0 + jj) * p.q_stride + (size_t)(g * p.G + hh) * HD;
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (row_ok) v = *reinterpret_cast<const uint4*>(src + kb * 64 + c * 8);
                    *reinterpret_cast<uint4*>(sm + OFF_Q + kb * (BM * 128) + r * 128 + ((c ^ (r & 7)) << 4)) = v;
                }
            proxy_fence();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready);
        }
        float m = -INFINITY, l = 0.f;                          // m: the maximum the output is scaled to
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int t = t_begin + j;
            if (!mbar_wait(s_full, j & 1, p.error, ERR_SOFTMAX)) { ok = false; break; }
            tc_fence_after();
            float s[BN];
            tmem_ld64_issue(lane_addr + COL_S, s);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty);                // the tensor core may write the next tile's scores
            const bool masked = p.window > 0 || t * BN + BN - 1 > p_row || !row_ok;
            if (masked) {
#pragma unroll
                for (int i = 0; i < BN; ++i) {
                    const int key = t * BN + i;
                    s[i] = (row_ok && key <= p_row && key >= lo_row) ? s[i] : -INFINITY;
                }
            }
            // four independent chains each for the maximum and the sum: one thread owns the whole
            // row, and a single chain of 64 dependent operations would leave the scheduler idle
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < BN; i += 8) {
                mx4[0] = max3(mx4[0], s[i], s[i + 1]); mx4[1] = max3(mx4[1], s[i + 2], s[i + 3]);
                mx4[2] = max3(mx4[2], s[i + 4], s[i + 5]); mx4[3] = max3(mx4[3], s[i + 6], s[i + 7]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            // The reference maximum moves only when the row's maximum has outgrown it by 2^8
            // (probabilities up to 256 are exact enough in bf16 and harmless in fp32 sums);
            // then the output in tensor memory and the sum are brought to the new reference.
            float factor = 1.f;
            if (mx > m + RESCALE_STEP || (m == -INFINITY && mx != -INFINITY)) {
                factor = m == -INFINITY ? 0.f : ex2(m - mx);
                m = mx;
            }
            const bool rescale = factor != 1.f && j > 0;
            if (__any_sync(0xffffffffu, rescale)) {
                if (!mbar_wait(o_done, (j - 1) & 1, p.error, ERR_SOFTMAX)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 16) {
                    float v[16];
                    tmem_ld16_issue(lane_addr + COL_O + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] *= factor;
                    tmem_st16(lane_addr + COL_O + c0, v);
                }
                tmem_st_wait();
                tc_fence_before();
            }
            l *= factor;
            const float m_use = m == -INFINITY ? 0.f : m;
            // two scores an instruction where the hardware has one (fma and add on pairs of fp32).
            // A warp with a masked row in this tile (the diagonal, a window's edge, rows past the
            // portion) computes every exponential on the special-function unit, which gives an
            // exact zero for a masked score; the polynomial gives 2^-126 there.
            const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(-m_use, -m_use);
            float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            auto exponentials = [&](auto with_poly) {
#pragma unroll
                for (int i = 0; i < BN; i += 4) {
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const float2 x = __ffma2_rn(make_float2(s[i + 2 * k], s[i + 2 * k + 1]), scale2, shift2);
                        if (decltype(with_poly)::value && POLY_OF > 0 && ((i / 2 + k) % POLY_OF) == POLY_OF - 1) {
                            const float2 e = ex2_poly2(x);
                            s[i + 2 * k] = e.x;
                            s[i + 2 * k + 1] = e.y;
                        } else {
                            s[i + 2 * k] = ex2(x.x);
                            s[i + 2 * k + 1] = ex2(x.y);
                        }
                        sum2[k] = __fadd2_rn(sum2[k], make_float2(s[i + 2 * k], s[i + 2 * k + 1]));
                    }
                }
            };
            if (__any_sync(0xffffffffu, masked)) exponentials(std::false_type{});
            else exponentials(std::true_type{});
            l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
            // P row (bf16) into the A operand of P V
            if (!mbar_wait(p_empty, (j & 1) ^ 1, p.error, ERR_SOFTMAX)) { ok = false; break; }
            {
                unsigned char* prow = sm + OFF_P + r * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint4 w;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(s[c * 8 + 2 * i], s[c * 8 + 2 * i + 1]);
                    *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = w;
                }
            }
            // keys no row of the tile sees (past the last position, or before the window): whatever
            // the cache holds there must not reach P V, not even times zero; their V rows are
            // cleared (threads r < 64 each take one key row of the tile)
            if (t * BN + BN - 1 > p_last || t * BN < lo_tile) {
                const int st = j % NS, u = j / NS;
                if (!mbar_wait(&v_full[st], u & 1, p.error, ERR_SOFTMAX)) { ok = false; break; }
                if (r < BN && (t * BN + r > p_last || t * BN + r < lo_tile)) {
#pragma unroll
                    for (int kb = 0; kb < KB; ++kb) {
                        uint4* vrow = reinterpret_cast<uint4*>(sm + OFF_V + st * KV_STAGE + kb * (BN * 128) + r * 128);
#pragma unroll
                        for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            proxy_fence();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        // the output of the last tile's P V, scaled by 1 / sum
        if (ok && n_tiles > 0) ok = mbar_wait(o_done, (n_tiles - 1) & 1, p.error, ERR_SOFTMAX);
        if (ok && n_tiles > 0) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = p.out + (size_t)(q_begin + tok0 + jj) * p.out_stride + (size_t)(g * p.G + hh) * HD;
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 16) {
                float v[16];
                tmem_ld16_issue(lane_addr + COL_O + c0, v);       // every lane of the warp takes part
                tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint4 w;
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            h[i] = __floats2bfloat162_rn(v[c * 8 + 2 * i] * inv, v[c * 8 + 2 * i + 1] * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c * 8) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host: tensor map
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
    const void* ptr; long long rows; int box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && box_rows == o.box_rows; }
};
struct MapHash {
    size_t operator()(const MapKey& k) const {
        return reinterpret_cast<size_t>(k.ptr) ^ ((size_t)k.rows * 0x9E3779B97F4A7C15ull) ^ ((size_t)k.box_rows << 50);
    }
};
// One layer of the cache, [page][K|V][kv head][slot][HD], seen as a matrix of HD-wide rows.
int cache_map(const void* ptr, long long rows, int box_rows, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    std::lock_guard<std::mutex> lock(mu);
    const MapKey key{ptr, rows, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiled fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    if (cache.size() > 1024) cache.clear();
    cache.emplace(key, *out);
    return 0;
}
}  // namespace

RI_API void ri_set_pdl(int on) { ri_pdl_flag() = on ? 1 : 0; }
RI_API int ri_attention_tc_head_dim() { return HD; }

// 1 if this kernel takes the grouping and page size, else 0 (the caller then uses the
// mma.sync kernel): a group of at most 128 heads, pages of 8, 16, 32 or a multiple of 64 keys.
// A tile holds floor(128 / group) tokens; with a group that does not divide 128 the last
// rows of the tile are padding (a group of 3: 42 tokens, 126 rows), computed and dropped.
RI_API int ri_attention_tc_supports(int Hq, int Hkv, int page_size) {
    if (Hkv <= 0 || Hq % Hkv != 0) return 0;
    const int G = Hq / Hkv;
    if (G > BM) return 0;
    return (page_size == 8 || page_size == 16 || page_size == 32 || (page_size > 0 && page_size % 64 == 0)) ? 1 : 0;
}
RI_API int ri_attention_tc_tokens_per_tile(int Hq, int Hkv) { return BM / (Hq / Hkv); }

// Tiles are (entry, first token) pairs of 128 / (Hq/Hkv) tokens.  error: one int that a
// timed-out wait sets (zero it before use).
RI_API int ri_attention_prefill_tc(const void* q, int q_stride, void* out, int out_stride, const void* cache,
                                   long long n_pages, const int* block_table, int table_stride, const int* cu_q,
                                   const int* kv_len, const int* tile_entry, const int* tile_tok0, int n_tiles,
                                   int Hq, int Hkv, int page_size, float scale, int window, int* error,
                                   void* stream) {
    if (n_tiles <= 0) return 0;
    if (!ri_attention_tc_supports(Hq, Hkv, page_size) || !error) return (int)cudaErrorInvalidValue;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    Params p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.out_stride = out_stride;
    p.block_table = block_table; p.table_stride = table_stride; p.cu_q = cu_q; p.kv_len = kv_len;
    p.tile_entry = tile_entry; p.tile_tok0 = tile_tok0;
    p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.tpt = BM / p.G; p.page_size = page_size;
    p.box_rows = page_size < BN ? page_size : BN;
    p.scale_log2 = scale * 1.4426950408889634f; p.window = window; p.error = error;
    CUtensorMap map;
    int st = cache_map(cache, n_pages * 2 * Hkv * page_size, p.box_rows, &map);
    if (st != 0) return st;
    RI_CHECKED(ri_launch(attention_tc_kernel, dim3(Hkv, n_tiles), dim3(THREADS), SMEM, (cudaStream_t)stream, map, p));
    return ri_launch_status();
}
