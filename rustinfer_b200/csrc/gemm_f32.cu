// C[M,N] = A[M,K] * W[N,K]^T in true fp32: FMA on CUDA cores, no tensor cores, no TF32.
//
// RustInfer's fp32 matrix product on CUDA is cublasGemmEx with
// CUBLAS_COMPUTE_32F_FAST_TF32 (crates/infer-backend-cuda/src/kernels/matmul/matmul.cu:1807-1834),
// which rounds the inputs to 10 mantissa bits; its exact path is the CPU back end
// (crates/infer-backend-cpu/src/lib.rs:377-430).  This kernel is the exact path on the
// GPU.  Every output element is summed over k in ascending order whatever M and N
// are, so a token's result does not depend on the batch it was computed in.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                float* __restrict__ C, int ldc, int M, int N, int K) {
    pdl_trigger();
    pdl_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tr = tid / 16, tc = tid % 16;          // 16 x 16 threads, 4 x 4 outputs each
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements of each operand, 256 threads: 4 elements per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BK, c = idx % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][tr * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tc * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + tr * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tc * TN + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
        }
    }
}
}  // namespace

RI_API int ri_gemm_f32(const float* A, int lda, const float* W, int ldw, float* C, int ldc,
                       int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    RI_CHECKED(ri_launch(gemm_f32_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, A, lda, W, ldw, C, ldc, M, N, K));
    return ri_launch_status();
}
