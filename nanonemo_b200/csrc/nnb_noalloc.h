// Entry point of libnanonemo_b200.so that allocates nothing. It has no counterpart in the reference.
//
// Who needs it: code that runs where device memory cannot be requested — a host callback or a
// capture-time hook in which cudaMalloc is illegal, a service that was handed a fixed memory budget
// at start-up and runs with the allocator locked, or a C / ctypes caller that has no tensor library
// to allocate scratch space with. The ordinary entry point, nnb_sumsq_f32, needs a caller-provided
// scratch buffer for its per-block partial sums; this variant keeps that scratch in a file-scope
// device array inside the library, so the caller passes only the input and the output.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest input the no-allocation variant accepts, in elements (2^32 fp32 values = 16 GiB).
#define NNB_SUMSQ_NOALLOC_MAX_ELEMS (1LL << 32)
// Size of the built-in scratch array: partial sums of up to this many blocks + one ticket word.
// Every GPU that loads the library holds these 4100 bytes until the process exits.
#define NNB_SUMSQ_NOALLOC_MAX_BLOCKS 1024

// out[0] = sum(x[i]^2, i < n) for fp32 x (16-byte aligned device pointer), out a device fp32 scalar.
// Same kernel and same fixed summation order as nnb_sumsq_f32.
//  * Calls no cudaMalloc / cudaFree and no allocating library routine.
//  * n > NNB_SUMSQ_NOALLOC_MAX_ELEMS, n < 0, or a null / misaligned pointer: returns a negative code
//    and nnb_last_error() says why.
//  * The first call on each device looks up the device address of the built-in scratch array
//    (cudaGetSymbolAddress, with that device current); make that first call outside any stream capture.
//  * All calls on a device share the one scratch array. The ticket word is cleared on the stream before
//    every launch, so a call does not depend on what the previous one left behind; but two calls that
//    overlap on the GPU (different streams, no ordering between them) race on the array and both
//    results are then undefined. Order such calls yourself.
int nnb_sumsq_f32_noalloc(const void* x, long long n, void* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
