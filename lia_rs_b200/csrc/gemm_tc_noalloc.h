// lia_gemm_tc_noalloc: the tensor-core matrix product for callers that must not allocate.
//
// This entry point has no counterpart in the reference project; it exists for embedders of this library.
//
// Who needs it.  Some hosts of this library are not allowed to call cudaMalloc (or anything that calls
// it for them) at the moment they need a product: code that runs inside a region where the allocator is
// frozen (a memory pool handed out once at start-up, a real-time loop with a fixed footprint), a plug-in
// whose host owns all device memory, or a process that has already given the rest of the device to
// another library.  The ordinary entry point, lia_gemm_tc, leaves the split-K scratch to its caller, and
// the Python face gets it from torch's allocator.  This variant brings its own: a file-scope
// `static __device__` array of LIA_GEMM_NOALLOC_SCRATCH_BYTES (8 MiB) inside the library image.  Every
// GPU that loads the library holds these 8 MiB until the process exits, whether or not the entry point
// is ever called.
//
// Contract.
//  * Arguments are those of lia_gemm_tc without `scratch` and `scratch_floats`: the caller still passes
//    inputs and outputs (device pointers), sizes, strides, the SM count to fill and the stream.
//  * It calls no cudaMalloc, cudaFree, nor any allocating library routine.  The first call on a device
//    looks up the array's device address with cudaGetSymbolAddress while that device is current and keeps
//    it; make that first call before any stream capture begins, because the lookup may load the module.
//  * A product whose split-K partial sums would not fit the array is refused with LIA_ERR_SCRATCH (-6)
//    and nothing is launched.  The need is 4096 words of tile counters + splits * M * n_total floats,
//    n_total = N (2N for SWIGLU); lia_gemm_tc_noalloc_scratch_floats() returns it for given sizes so a
//    caller can ask beforehand.  Products that need no split (many tokens, or enough tiles to fill the
//    SMs) use no scratch.
//  * All calls share the one array of a device, and it keeps what the last call left there.  Partial
//    sums need no clearing: every one that is read was written by the same call first.  The tile
//    counters at the head of the array must be zero when a call starts: they are zero when the library
//    is loaded, and the kernel itself puts each one back to zero when the last K range of its tile has
//    arrived, so a call that ran to its end leaves them ready for the next.  Two calls that overlap on
//    one GPU (different streams, or different threads) race on counters and sums alike: keep calls to
//    this entry point on one device in one stream order.
//  * If a call's kernel gives up on one of its bounded waits it raises `*error_flag` to 3 and may leave tile
//    counters mid-count.  The caller cannot reach the array, so lia_gemm_tc_noalloc_reset(stream) zeroes the
//    counters for it (a cudaMemsetAsync in stream order, no allocation): call it after seeing that flag, before
//    the next product.
//  * Return codes are those of lia_gemm_tc (0 = launched) plus LIA_ERR_SCRATCH.  LIA_ERR_DRIVER (-4) from the
//    first call on a device means the address lookup failed, whatever the cause (a stream capture in progress
//    is one).
#pragma once
#include <cuda_runtime.h>

#define LIA_GEMM_NOALLOC_SCRATCH_BYTES (8u << 20)
#define LIA_ERR_SCRATCH (-6)     // the product needs more scratch than the built-in array holds

#ifdef __cplusplus
extern "C" {
#endif

int lia_gemm_tc_noalloc(int mode, const void* X, int ldx, const void* W, int ldw, void* out, int out_dtype,
                        int ldo, int M, int N, int K, float alpha, int sm_count, int* error_flag,
                        cudaStream_t stream);

// Floats of scratch the product of these sizes would use (0: it does not split K).
long long lia_gemm_tc_noalloc_scratch_floats(int mode, int M, int N, int K, int sm_count);

// Zero the tile counters at the head of the array, in stream order (after a call that raised error flag 3).
int lia_gemm_tc_noalloc_reset(cudaStream_t stream);

#ifdef __cplusplus
}
#endif
