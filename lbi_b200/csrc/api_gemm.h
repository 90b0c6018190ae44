// C entry point of the tcgen05 GEMM (gemm_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// C[M, N] (+)= A[M, K] * B[N, K]^T with bf16 operands and fp32 accumulation.
//   a_mn_major = 0: A is row-major [M, K] with leading dimension lda;  1: A is stored row-major as [K, M] (M % 64 == 0).
//   b_mn_major likewise for B ([N, K] or [K, N], N % 64 == 0).
//   out_fp32 = 0: C is bf16 and is overwritten;  1: C is fp32, overwritten, or added to when accumulate != 0.
//   splits > 1 divides the K loop over gridDim.y CTAs that add into an fp32 C (which must then hold valid data).
//   status: device int, receives a non-zero site code if a bounded wait inside the kernel ran out.
// Requirements: all base pointers 16-byte aligned, lda/ldb multiples of 8 elements, ldc * sizeof(C element) a
// multiple of 16.  Returns 0 or a cudaError_t / 1000 + CUresult from the tensor-map encoder.
int lbi_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                  int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int splits, int* status, int sm_count,
                  cudaStream_t stream);

#ifdef __cplusplus
}
#endif
