// An entry point for callers that cannot allocate device memory.
//
// This function has no counterpart in RustInfer; it exists for users of this library
// whose environment forbids cudaMalloc at the time they call: code that runs inside
// another framework's memory plan (a fixed arena handed out at start-up), callers in a
// stream-ordered or real-time section where an allocation would synchronise the device,
// and embedders that load the library through its C symbols and have no allocator of
// their own to lend.  ri_attention_decode_bf16 needs fp32 scratch for the partial results
// of its key splits and makes its caller bring it; this variant brings its own.
//
// The scratch is a file-scope __device__ array of RI_DECODE_STATIC_SCRATCH_FLOATS floats
// (4 MiB) inside the library, so every GPU on which the library is loaded holds 4 MiB
// until the process exits, whether or not this function is ever called.
//
// What the caller must know:
//  * Limit: entries * q_heads * splits * (head_dim + 1) must not exceed
//    RI_DECODE_STATIC_SCRATCH_FLOATS.  A larger request is refused with
//    cudaErrorInvalidValue and ri_attention_decode_static_error() tells why; nothing is
//    launched.
//  * The first call on a device looks up the array's device address and raises the
//    kernels' shared-memory limit.  Make that first call outside any stream capture.  The
//    look-up runs under a host lock, so host threads may race to be first.
//  * The function calls no cudaMalloc, cudaFree or allocating library routine, on any call.
//  * Every call uses the same array.  Two calls whose kernels may overlap on the GPU (other
//    streams, other host threads) race on it; keep calls on one stream or order them
//    yourself.  The array keeps the last call's contents; the kernels write every slot
//    they later read, so nothing has to be cleared between calls.
//  * Inputs and outputs are the caller's, exactly as for ri_attention_decode_bf16.
#pragma once

#define RI_DECODE_STATIC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as ri_attention_decode_bf16 without the two scratch pointers.
__attribute__((visibility("default")))
int ri_attention_decode_bf16_static(const void* q, int q_stride, void* out, int out_stride,
                                    const void* cache, const int* block_table, int table_stride,
                                    const int* cu_q, const int* kv_len, const int* entry_list,
                                    int n_entries, int Hq, int Hkv, int page_size, float scale,
                                    int window, int splits, void* stream);

// Why the last call of this thread was refused ("" if it was not).
__attribute__((visibility("default")))
const char* ri_attention_decode_static_error(void);

#ifdef __cplusplus
}
#endif
