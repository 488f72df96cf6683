// lb_gemm_tcgen05_static_scratch: the tensor-core matrix product for callers that cannot allocate
// device memory.
//
// This entry point has no counterpart in JunkuiZhang/lucciola (whose products never split K and so
// need no scratch); it exists for users of this library.
//
// Who needs it.  The ordinary entry point, lb_gemm_tcgen05, splits K across CTAs when few tokens meet
// a small weight matrix and then needs scratch memory for the partial sums and the tile counters; its
// caller has to provide that memory.  Some callers cannot: a host program that has already given all
// free device memory to its own pool (this engine itself hands 90 % of what is free to the cache pages,
// after which a cudaMalloc may simply fail); a loop that must not stall, since cudaMalloc and cudaFree
// synchronise the whole device; a program in C or another language that links this library without
// torch's allocator behind it.  For them the scratch lives inside the library: a file-scope
// `static __device__ __align__(256)` array of LB_STATIC_SCRATCH_BYTES bytes.  Every GPU on which the
// library's code is loaded holds that array from then until the process exits.
//
// What the caller passes: inputs and outputs only (x, w, y), their sizes and a stream.  The call makes
// no cudaMalloc, no cudaFree and calls no routine that allocates device memory; the tensor maps it
// needs are built on the stack for each call.
//
// Limits.  When the product is split (M <= 256 and fewer than 148 output tiles), the partial sums,
// splits * M * N floats, must fit LB_STATIC_SCRATCH_PARTIALS floats and the output tiles
// LB_STATIC_SCRATCH_COUNTERS counters; a larger request is refused with a message that names the
// limit, and nothing is launched.  Products that are not split use no scratch and have no such limit.
//
// Which kernel runs.  Every size goes to the few-token kernel (weight rows on the tensor core's 128 lanes,
// up to 256 tokens a tile).  The result is right for any M, but a product of many tokens (M > 256), which
// lb_gemm_tcgen05 sends to its persistent many-token kernel, runs slower here: this entry point is meant
// for the few-token products that need scratch at all.
//
// First call on a device.  The array's name is a host-side handle, not a device address.  The first
// call on each device, made with that device current, asks the runtime for the array's address on that
// device (cudaGetSymbolAddress) and keeps it; that first call should come before any stream capture
// begins.  Later calls on the device reuse the address.
//
// Sharing.  All calls on a device share the one array, and it keeps what the last call left.  The
// counters, which must start at zero, are cleared on the caller's stream before each launch; partial
// sums are overwritten before they are read.  Two calls that overlap on the GPU (different streams, no
// ordering between them) would use the same scratch at once and race: order such calls.
#pragma once

#include <cuda_runtime.h>

#define LB_STATIC_SCRATCH_COUNTERS 1024                 /* output tiles of a split product */
#define LB_STATIC_SCRATCH_PARTIALS (2 * 1024 * 1024)    /* float32 partial sums: 8 MB */
#define LB_STATIC_SCRATCH_BYTES (LB_STATIC_SCRATCH_COUNTERS * 4 + LB_STATIC_SCRATCH_PARTIALS * 4)

#ifdef __cplusplus
extern "C" {
#endif

// y[M,N] = x[M,K] . w[N,K]^T.  x: bfloat16, row stride ldx elements; w: bfloat16, contiguous;
// y: bfloat16 (y_dtype 1) or float32 (y_dtype 0), row stride ldy.  K and ldx multiples of 8, x and w
// 16-byte aligned.  Returns 0, or a non-zero code with the reason in lb_last_error().
int lb_gemm_tcgen05_static_scratch(void* y, int y_dtype, const void* x, const void* w, int M, int N, int K,
                                   long long ldx, long long ldy, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
