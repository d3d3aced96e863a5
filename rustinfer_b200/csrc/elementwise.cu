// Row-wise kernels of the decoder: embedding gather, residual add + RMSNorm, rotary
// position encoding fused with the write of keys and values into cache pages, and
// SiLU-multiply.  All arithmetic is fp32; storage is fp32 or bf16 by template.
//
// What they compute follows RustInfer's kernels: embedding
// (crates/infer-backend-cuda/src/kernels/embedding/emb.cu:9-38), fused add + RMSNorm
// (crates/infer-backend-cuda/src/kernels/fused_add_rmsnorm/fused_add_rmsnorm.cu:16-97),
// rotate-half RoPE (crates/infer-backend-cuda/src/kernels/rope/rope.cu:84-133), paged
// scatter (crates/infer-backend-cuda/src/kernels/kv_cache/scatter_kv_batch.cu:236-300)
// and SwiGLU (crates/infer-backend-cuda/src/kernels/swiglu/swiglu.cu:294-343).  Unlike
// them the residual stream stays fp32, the norm's scale is never rounded to bf16, and
// RoPE and the scatter are one kernel.
#include "common.cuh"

RI_API const char* ri_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

// ---------------------------------------------------------------- embedding gather
template <typename TW>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                    float* __restrict__ out, int d, int vocab) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * d;
    if (id < 0 || id >= vocab) {            // ids are validated on the host; never read outside
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32<TW>(src[i]);
}

RI_API int ri_embed_gather(const int* ids, const void* table, int table_dtype, float* out,
                           int tokens, int d, int vocab, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == RI_BF16)
        RI_CHECKED(ri_launch(embed_gather_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, ids, (const bf16*)table, out, d, vocab));
    else
        RI_CHECKED(ri_launch(embed_gather_kernel<float>, dim3(tokens), dim3(threads), 0, s, ids, (const float*)table, out, d, vocab));
    return ri_launch_status();
}

// ------------------------------------------------------- residual add + RMSNorm
// h (fp32 residual stream) += delta, then out = h * rsqrt(mean(h^2) + eps) * w.
// With `rows` the kernel reads rows[r] of h and delta, writes row r of out and leaves h
// alone (the final norm over the rows whose logits are wanted).
template <typename TA, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TA* __restrict__ delta,
                                   const TW* __restrict__ w, float eps, TA* __restrict__ out,
                                   const int* __restrict__ rows, int d) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hp = h + (size_t)src * d;
    const TA* dp = delta ? delta + (size_t)src * d : nullptr;
    const bool write_back = (rows == nullptr) && (dp != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = hp[i];
        if (dp) v += to_f32<TA>(dp[i]);
        if (write_back) hp[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    TA* op = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = hp[i];
        if (dp && !write_back) v += to_f32<TA>(dp[i]);
        op[i] = from_f32<TA>(v * inv * to_f32<TW>(w[i]));
    }
}

// bf16 activations, width a multiple of 8 and at most 8 * 1024: every thread keeps its 8
// elements in registers between the sum of squares and the scaling, and moves 16 or 32
// bytes per access.
__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 float_to_bf16x8(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

template <typename TW>
__global__ void add_rmsnorm_bf16x8_kernel(float* __restrict__ h, const bf16* __restrict__ delta,
                                          const TW* __restrict__ w, float eps, bf16* __restrict__ out,
                                          const int* __restrict__ rows, int d) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const int i0 = threadIdx.x * 8;
    const bool active = i0 < d;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    float ss = 0.f;
    if (active) {
        float* hp = h + (size_t)src * d + i0;
        const float4 a = *reinterpret_cast<const float4*>(hp);
        const float4 b = *reinterpret_cast<const float4*>(hp + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        if (delta) {
            float dv[8];
            bf16x8_to_float(*reinterpret_cast<const uint4*>(delta + (size_t)src * d + i0), dv);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] += dv[i];
            if (!rows) {
                *reinterpret_cast<float4*>(hp) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(hp + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    }
    ss = block_sum(ss, red);
    if (!active) return;
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    float wv[8];
    if (sizeof(TW) == 2) {
        bf16x8_to_float(*reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(w) + i0), wv);
    } else {
        const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i0);
        const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i0 + 4);
        wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * wv[i];
    *reinterpret_cast<uint4*>(out + (size_t)r * d + i0) = float_to_bf16x8(v);
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

RI_API int ri_add_rmsnorm(float* h, const void* delta, const void* w, int w_dtype, float eps,
                          void* out, int act_dtype, const int* rows, int n_rows, int d,
                          void* stream) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == RI_BF16 && d % 8 == 0 && d <= 8192 && aligned16(h) && aligned16(out) && aligned16(w) &&
        (!delta || aligned16(delta))) {
        const int vt = ((d / 8 + 31) / 32) * 32;
        if (w_dtype == RI_BF16)
            RI_CHECKED(ri_launch(add_rmsnorm_bf16x8_kernel<bf16>, dim3(n_rows), dim3(vt), 0, s, h, (const bf16*)delta, (const bf16*)w, eps,
                                                                  (bf16*)out, rows, d));
        else
            RI_CHECKED(ri_launch(add_rmsnorm_bf16x8_kernel<float>, dim3(n_rows), dim3(vt), 0, s, h, (const bf16*)delta, (const float*)w, eps,
                                                                   (bf16*)out, rows, d));
        return ri_launch_status();
    }
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
#define RI_LAUNCH(TA, TW)                                                                  \
    RI_CHECKED(ri_launch(add_rmsnorm_kernel<TA, TW>, dim3(n_rows), dim3(threads), 0, s, h, (const TA*)delta, (const TW*)w, \
                                                          eps, (TA*)out, rows, d))
    if (act_dtype == RI_BF16) {
        if (w_dtype == RI_BF16) RI_LAUNCH(bf16, bf16); else RI_LAUNCH(bf16, float);
    } else {
        if (w_dtype == RI_BF16) RI_LAUNCH(float, bf16); else RI_LAUNCH(float, float);
    }
#undef RI_LAUNCH
    return ri_launch_status();
}

// h += delta on every row (flush of the last pending residual when the stream itself is wanted)
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ h, const TA* __restrict__ delta, size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) h[i] += to_f32<TA>(delta[i]);
}

RI_API int ri_residual_add(float* h, const void* delta, int act_dtype, long long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int blocks = (int)((n + 255) / 256);
    if (blocks > ri_device_sms() * 8) blocks = ri_device_sms() * 8;
    if (act_dtype == RI_BF16) RI_CHECKED(ri_launch(residual_add_kernel<bf16>, dim3(blocks), dim3(256), 0, s, h, (const bf16*)delta, (size_t)n));
    else RI_CHECKED(ri_launch(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, s, h, (const float*)delta, (size_t)n));
    return ri_launch_status();
}

// --------------------------------------------------- RoPE + write of K,V into pages
// qkv row t: [Hq heads of q | Hkv heads of k | Hkv heads of v], head_dim each.
// q is rotated in place; k is rotated and written to the page slot of token t; v is
// copied there.  The pair of element i is i + rotary_dim/2; elements at and beyond
// rotary_dim pass through.  cos/sin tables are fp32 [positions, rotary_dim/2].
// Cache layout of one layer: [page][K|V][kv head][slot in page][head_dim].
template <typename TA>
__global__ void rope_scatter_kernel(TA* __restrict__ qkv, int row_stride,
                                    const int* __restrict__ positions,
                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                    const int* __restrict__ slot_of_token, TA* __restrict__ cache,
                                    int Hq, int Hkv, int hd, int rot, int page_size) {
    // wait first, then let the next kernel start: the attention kernel that follows reads all
    // but this kernel's output before its own wait, so every earlier kernel must be complete by then
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const int pos = positions[t];
    TA* row = qkv + (size_t)t * row_stride;
    const float* ct = cos_t + (size_t)pos * half;
    const float* st = sin_t + (size_t)pos * half;
    const int slot = (slot_of_token && Hkv > 0) ? slot_of_token[t] : -1;
    TA* kdst = nullptr;
    TA* vdst = nullptr;
    if (slot >= 0) {
        const int page = slot / page_size, off = slot - page * page_size;
        kdst = cache + ((size_t)(page * 2 + 0) * Hkv * page_size + off) * hd;
        vdst = cache + ((size_t)(page * 2 + 1) * Hkv * page_size + off) * hd;
    }
    const size_t head_step = (size_t)page_size * hd;    // between kv heads inside a page
    const int n_rot = (Hq + Hkv) * half;
    for (int wi = threadIdx.x; wi < n_rot; wi += blockDim.x) {
        const int head = wi / half, i = wi - head * half;
        TA* p = row + (size_t)head * hd;
        const float x1 = to_f32<TA>(p[i]), x2 = to_f32<TA>(p[i + half]);
        const float c = ct[i], s = st[i];
        const TA y1 = from_f32<TA>(x1 * c - x2 * s);
        const TA y2 = from_f32<TA>(x1 * s + x2 * c);
        if (head < Hq) {
            p[i] = y1;
            p[i + half] = y2;
        } else if (kdst) {
            TA* kd = kdst + (size_t)(head - Hq) * head_step;
            kd[i] = y1;
            kd[i + half] = y2;
        }
    }
    if (kdst) {
        const int pass = hd - rot;                      // unrotated tail of each k head
        for (int wi = threadIdx.x; wi < Hkv * pass; wi += blockDim.x) {
            const int g = wi / pass, i = rot + (wi - g * pass);
            kdst[(size_t)g * head_step + i] = row[(size_t)(Hq + g) * hd + i];
        }
        const TA* vsrc = row + (size_t)(Hq + Hkv) * hd;
        for (int wi = threadIdx.x; wi < Hkv * hd; wi += blockDim.x) {
            const int g = wi / hd, i = wi - g * hd;
            vdst[(size_t)g * head_step + i] = vsrc[wi];
        }
    }
}

// bf16, head_dim and rotary_dim multiples of 16: one work item = 8 elements of the first
// half of a head and their 8 partners, or 8 elements that are only copied.
__global__ void rope_scatter_bf16x8_kernel(bf16* __restrict__ qkv, int row_stride,
                                           const int* __restrict__ positions,
                                           const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                           const int* __restrict__ slot_of_token, bf16* __restrict__ cache,
                                           int Hq, int Hkv, int hd, int rot, int page_size) {
    // wait first, then let the next kernel start: the attention kernel that follows reads all
    // but this kernel's output before its own wait, so every earlier kernel must be complete by then
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const int pos = positions[t];
    bf16* row = qkv + (size_t)t * row_stride;
    const float* ct = cos_t + (size_t)pos * half;
    const float* st = sin_t + (size_t)pos * half;
    const int slot = (slot_of_token && Hkv > 0) ? slot_of_token[t] : -1;
    bf16* kdst = nullptr;
    bf16* vdst = nullptr;
    if (slot >= 0) {
        const int page = slot / page_size, off = slot - page * page_size;
        kdst = cache + ((size_t)(page * 2 + 0) * Hkv * page_size + off) * hd;
        vdst = cache + ((size_t)(page * 2 + 1) * Hkv * page_size + off) * hd;
    }
    const size_t head_step = (size_t)page_size * hd;
    const int vph = half >> 3;                               // rotating vectors per head
    const int n_rot = (Hq + Hkv) * vph;
    for (int wi = threadIdx.x; wi < n_rot; wi += blockDim.x) {
        const int head = wi / vph, i = (wi - head * vph) * 8;
        if (head >= Hq && !kdst) continue;
        bf16* p = row + (size_t)head * hd;
        float x1[8], x2[8], c[8], s[8];
        bf16x8_to_float(*reinterpret_cast<const uint4*>(p + i), x1);
        bf16x8_to_float(*reinterpret_cast<const uint4*>(p + i + half), x2);
        *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(ct + i);
        *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(ct + i + 4);
        *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(st + i);
        *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(st + i + 4);
        float y1[8], y2[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            y1[k] = x1[k] * c[k] - x2[k] * s[k];
            y2[k] = x1[k] * s[k] + x2[k] * c[k];
        }
        bf16* dst = head < Hq ? p : kdst + (size_t)(head - Hq) * head_step;
        *reinterpret_cast<uint4*>(dst + i) = float_to_bf16x8(y1);
        *reinterpret_cast<uint4*>(dst + i + half) = float_to_bf16x8(y2);
    }
    if (kdst) {
        const int pass_v = (hd - rot) >> 3;                  // unrotated tail of each k head
        for (int wi = threadIdx.x; wi < Hkv * pass_v; wi += blockDim.x) {
            const int g = wi / pass_v, i = rot + (wi - g * pass_v) * 8;
            *reinterpret_cast<uint4*>(kdst + (size_t)g * head_step + i) =
                *reinterpret_cast<const uint4*>(row + (size_t)(Hq + g) * hd + i);
        }
        const bf16* vsrc = row + (size_t)(Hq + Hkv) * hd;
        const int vpv = hd >> 3;
        for (int wi = threadIdx.x; wi < Hkv * vpv; wi += blockDim.x) {
            const int g = wi / vpv, i = (wi - g * vpv) * 8;
            *reinterpret_cast<uint4*>(vdst + (size_t)g * head_step + i) =
                *reinterpret_cast<const uint4*>(vsrc + (size_t)g * hd + i);
        }
    }
}

RI_API int ri_rope_scatter(void* qkv, int act_dtype, int row_stride, const int* positions,
                           const float* cos_t, const float* sin_t, const int* slot_of_token,
                           void* cache, int tokens, int Hq, int Hkv, int hd, int rot,
                           int page_size, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int work = (Hq + 2 * Hkv) * hd / 2;
    const int threads = work >= 1024 ? 256 : 128;
    if (act_dtype == RI_BF16 && hd % 16 == 0 && rot % 16 == 0 && row_stride % 8 == 0 && aligned16(qkv) &&
        aligned16(cos_t) && aligned16(sin_t) && (!cache || aligned16(cache))) {
        const int vt = work / 8 >= 256 ? 256 : (work / 8 >= 128 ? 128 : 64);
        RI_CHECKED(ri_launch(rope_scatter_bf16x8_kernel, dim3(tokens), dim3(vt), 0, s, (bf16*)qkv, row_stride, positions, cos_t, sin_t,
                                                         slot_of_token, (bf16*)cache, Hq, Hkv, hd, rot, page_size));
        return ri_launch_status();
    }
    if (act_dtype == RI_BF16)
        RI_CHECKED(ri_launch(rope_scatter_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, (bf16*)qkv, row_stride, positions, cos_t,
            sin_t, slot_of_token, (bf16*)cache, Hq, Hkv, hd, rot, page_size));
    else
        RI_CHECKED(ri_launch(rope_scatter_kernel<float>, dim3(tokens), dim3(threads), 0, s, (float*)qkv, row_stride, positions, cos_t,
            sin_t, slot_of_token, (float*)cache, Hq, Hkv, hd, rot, page_size));
    return ri_launch_status();
}

// ------------------------------------------------------------------ SiLU(gate) * up
// gu row: [gate (I) | up (I)]; out[t, j] = gate / (1 + e^-gate) * up.
template <typename TA>
__global__ void silu_mul_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int inter) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= inter) return;
    const TA* row = gu + (size_t)t * 2 * inter;
    const float g = to_f32<TA>(row[j]), u = to_f32<TA>(row[inter + j]);
    out[(size_t)t * inter + j] = from_f32<TA>(g / (1.0f + expf(-g)) * u);
}

// bf16, width a multiple of 8: 16 bytes of gate and of up per thread
__global__ void silu_mul_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int inter,
                                       size_t n_vec) {
    pdl_trigger();
    pdl_wait();
    const int per_row = inter >> 3;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / per_row;
        const int j = (int)(i - t * per_row) * 8;
        const bf16* row = gu + t * 2 * (size_t)inter;
        float g[8], u[8];
        bf16x8_to_float(*reinterpret_cast<const uint4*>(row + j), g);
        bf16x8_to_float(*reinterpret_cast<const uint4*>(row + inter + j), u);
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] = g[k] / (1.0f + __expf(-g[k])) * u[k];
        *reinterpret_cast<uint4*>(out + t * (size_t)inter + j) = float_to_bf16x8(g);
    }
}

RI_API int ri_silu_mul(const void* gu, void* out, int act_dtype, int tokens, int inter, void* stream) {
    if (tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == RI_BF16 && inter % 8 == 0 && aligned16(gu) && aligned16(out)) {
        const size_t n_vec = (size_t)tokens * (inter / 8);
        size_t blocks = (n_vec + 255) / 256;
        if (blocks > (size_t)ri_device_sms() * 16) blocks = (size_t)ri_device_sms() * 16;
        RI_CHECKED(ri_launch(silu_mul_bf16x8_kernel, dim3((int)blocks), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, inter, n_vec));
        return ri_launch_status();
    }
    dim3 grid((inter + 255) / 256, tokens);
    if (act_dtype == RI_BF16) RI_CHECKED(ri_launch(silu_mul_kernel<bf16>, dim3(grid), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, inter));
    else RI_CHECKED(ri_launch(silu_mul_kernel<float>, dim3(grid), dim3(256), 0, s, (const float*)gu, (float*)out, inter));
    return ri_launch_status();
}

RI_API void ri_set_pdl(int on) { ri_pdl_flag() = on ? 1 : 0; }
