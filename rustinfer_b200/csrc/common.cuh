// Shared helpers of the sm_100a kernels: dtype conversion, warp and block reductions,
// launch checking.  Every exported function is plain C (called through ctypes), takes
// the CUDA stream as its last pointer argument and returns a cudaError_t as int.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define RI_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
#define RI_F32 0
#define RI_BF16 1

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order
// of additions is fixed by the thread layout, so equal inputs give equal bits.
__device__ __forceinline__ float block_sum(float v, float* red /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

static inline int ri_launch_status() { return (int)cudaGetLastError(); }

// Streaming multiprocessors of the current device (asked once per library and device change is
// not expected within a process: one process drives one GPU).
static inline int ri_device_sms() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            sms = n;
        else
            return 1;                                     // no device yet: ask again next time
    }
    return sms;
}

// ---- programmatic dependent launch -------------------------------------------------
// Kernels of one step run back to back on one stream.  Launched with the programmatic-
// serialization attribute, a kernel may begin (set up barriers, fetch weights that no
// earlier kernel writes) while its predecessor is still draining; it calls pdl_wait()
// before it touches anything the predecessor produced.  Every kernel launched this way
// calls pdl_wait(), so completion is transitive along the chain.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#define RI_CHECKED(expr) do { int ri_st_ = (expr); if (ri_st_ != 0) return ri_st_; } while (0)

// 1 (default): launch with the attribute; 0: plain launches.  One flag per library.
inline int& ri_pdl_flag() {
    static int on = 1;
    return on;
}

template <typename... KArgs, typename... Args>
static inline int ri_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ri_pdl_flag() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

RI_API const char* ri_error_string(int code);
