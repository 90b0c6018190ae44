// C entry point of the tcgen05 attention input pullback (attn_pullback.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Causal attention, head_dim 64, seq_len a multiple of 128, equal numbers of query and key/value heads.
//   qkv    bf16 [B*T, 3*H*64]      packed q | k | v (rotary already applied)
//   d_o    bf16 [P*B*T, H*64]      P output cotangents, direction-major rows
//   o      bf16 [B*T, H*64]        forward output,  lse fp32 [B, H, T] natural-log sum-exp of the scaled scores
//   d_qkv  bf16 [P*B*T, 3*H*64]    result: dq | dk | dv per direction
//   delta  fp32 [P, B, H, T]       scratch supplied by the caller
//   rope_cos / rope_sin  fp32 [T, 32] or null: when given, dq and dk are rotated back (transpose of the rotary
//          embedding; pairs (i, i + 32), or (2i, 2i + 1) when rope_interleaved) before they are stored
//   status device int, set non-zero if a bounded wait inside the kernels ran out
// Launches three kernels on `stream` (row dots, dK/dV, dQ).  Returns 0 or a cudaError_t / 1000 + CUresult.
int lbi_attn_pullback(const void* qkv, const void* d_o, const void* o, const float* lse, void* d_qkv, float* delta,
                      int batch, int heads, int seq_len, int head_dim, int nbasis, float scale, const float* rope_cos,
                      const float* rope_sin, int rope_interleaved, int is_fp16, int* status, cudaStream_t stream);

// Causal flash-attention forward (attn_fwd.cu), same layout and limits as above:
//   out bf16 [B*T, H*64], lse fp32 [B, H, T].  One kernel on `stream`.
// is_fp16 (both entry points): the 16-bit tensors are fp16 instead of bf16 (the reference kernel's only dtype).
int lbi_attn_fwd(const void* qkv, void* out, float* lse, int batch, int heads, int seq_len, int head_dim, float scale,
                 int is_fp16, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
