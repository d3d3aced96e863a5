// What a caller hands to the decode chain kernels (decode_chain.cu: up to 16 tokens, the
// activation operand resident in shared memory; decode_chain_wide.cu: 17 to 64 tokens, the
// operand streamed with the weights).
#pragma once

// One product of a chain, as the caller describes it.
struct RiChainPhase {
    const void* w;              // bf16 [N][K], K a multiple of 8, 16-byte aligned
    int N, K;
    int x_kind;                 // 0: x is bf16 [M][ld_x]; 1: x is the fp32 stream [M][ld_x] and the
    int ld_x;                   //    operand is x * norm_w * rsqrt(mean(x^2) + eps); 2: see `part_o`
    int x_rows;                 // rows the matrix x really has (a TMA box reads 8, 16 or 32 of them)
    const void* x;
    const void* norm_w;
    int norm_w_dtype;
    float eps;
    int out_kind;               // 0: fp32 out += product; 1: bf16 out[M][N/2] = silu(gate) * up over
    int ld_out;                 //    alternating weight rows; 2: bf16 out = product
    void* out;
    // steps of 17 to 64 tokens only, where x_kind is 1: room for the normed operand (bf16
    // [64][K], unscaled) and for the rows' sums of squares (64 floats, zero between launches)
    void* xn;
    float* rowsq;
    // x_kind 2 (steps of up to 16 tokens): the operand is the attention output of M single-token
    // entries whose key ranges have not been merged yet; x points at the partial outputs, fp32
    // [M][part_heads][part_splits][part_head_dim] (K = part_heads * part_head_dim), part_lse at
    // their base-2 log-sum-exps [M][part_heads][part_splits]; the merge happens while the operand
    // is laid out in shared memory
    const float* part_lse;
    int part_splits, part_heads, part_head_dim;
};

struct RiChainRope {
    float* qkv; int ld;
    const int* positions; const float* cos_t; const float* sin_t; const int* slot_of_token;
    void* q_out; int ld_q;
    void* cache;
    int Hq, Hkv, hd, rot, page_size;
};


// the chain for 17 to 64 tokens (decode_chain_wide.cu)
int ri_decode_chain_wide(const RiChainPhase* phases, int n_phases, const RiChainRope* rope, int M,
                         unsigned* grid_bar, int* error, int sms, void* stream);
int ri_decode_chain_wide_fits(const RiChainPhase* phases, int n_phases, int M, int sms);
