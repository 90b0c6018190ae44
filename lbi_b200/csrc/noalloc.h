// Allocation-free entry point.  It has no counterpart in the reference, which never exposes a C interface.
//
// Who needs it: code that is not allowed to allocate device memory at the moment of the call, for example a
// host that runs inside another framework's memory pool with the pool frozen, a real-time loop that must not hit
// cudaMalloc's implicit synchronisation, or a C/ctypes caller that has no allocator to hand over a workspace.
// The ordinary entry point lbi_rmsnorm_wgrad() makes its caller supply an (nblocks x dim) fp32 workspace; this
// variant keeps that workspace inside the library instead.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest feature dimension the built-in workspace covers, and the number of partial rows it holds.
#define LBI_NOALLOC_MAX_DIM 4096
#define LBI_NOALLOC_BLOCKS 148

// dw[d] = sum_r d_normed[r, d] * x[r, d] * rstd[r]   (weight gradient of RMSNorm, same result as lbi_rmsnorm_wgrad)
//
//   d_normed  bf16 [rows, dim]   x  fp32 [rows, dim]   rstd  fp32 [rows]   dw  fp32 [dim]   -- all device pointers
//
// * Calls no cudaMalloc / cudaFree and no allocating library routine.  Its workspace is a fixed array of
//   LBI_NOALLOC_BLOCKS * LBI_NOALLOC_MAX_DIM floats (about 2.4 MB) that every GPU holding this library keeps
//   resident until the process exits.
// * dim must be a multiple of 8 and at most LBI_NOALLOC_MAX_DIM; larger sizes are rejected with
//   cudaErrorInvalidValue (1) and nothing is launched.
// * The first call on each device looks up the device address of the workspace (cudaGetSymbolAddress, with that
//   device current).  Make that first call outside any stream capture.
// * All calls on one device share the workspace.  Each call overwrites every partial it later reads, so nothing
//   has to be cleared between calls; but two calls whose kernels overlap on the GPU (different streams without
//   an ordering between them) race on the workspace.  Order them on one stream or with events.
// Returns 0 on success, otherwise a cudaError_t.
int lbi_rmsnorm_wgrad_noalloc(const void* d_normed_bf16, const float* x_stream, const float* rstd, float* dw,
                              int64_t rows, int dim, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
