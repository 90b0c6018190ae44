// C entry points of the peer-memory kernels (peer.cu): compute fused with the transfer over NVLink / NVSwitch.
// Every rank runs one process with one GPU; `*_ptrs` arguments are DEVICE arrays of `world` pointers into the peers'
// symmetric buffers (entry `rank` is this GPU's own buffer).  Cross-GPU ordering uses 32-bit sequence flags written
// with st.release.sys and polled with ld.acquire.sys; every poll is bounded (lbi_peer_set_wait_limit_ms) and reports
// through `status`.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Time limit (milliseconds, default 20000) of every flag wait of the kernels below, for the current device.
int lbi_peer_set_wait_limit_ms(int ms);

// All ranks write `seq` into slot [slot_base + rank] of every peer's flag array and wait until every peer's write has
// arrived in their own array.  Flags only ever grow, so no reset is needed.
int lbi_peer_barrier(uint32_t* const* flag_ptrs, int rank, int world, int slot_base, uint32_t seq, int* status,
                     cudaStream_t stream);

// Interface update fused with the hand-off of the new state:
//   delta = W2 act(W1 pooled + b1) + b2   (or W1 pooled + b1 when hidden == 0)
//   pre   = state_in + tanh(alpha) * delta ;  state_out = LayerNorm(pre) * ln_w + ln_b
// state_out is stored locally and, when peer_state is not null, into the next owner's mailbox, followed by a
// release-store of `seq` to peer_flag.  act: 0 = SiLU, 1 = GELU.  With a hidden layer, a scratch buffer hidden_buf
// [batch, hidden] and batch <= 8 the hidden units are spread over the grid (the first weight matrix is read once) and the CTA
// that finishes last runs the second layer, the LayerNorm and the peer store; otherwise one CTA per batch row does it all.
// done_counter: a zeroed device word, left zero.
int lbi_interface_update_handoff(const float* state_in, const float* pooled, const float* w1, const float* b1,
                                 const float* w2, const float* b2, const float* alpha, const float* ln_w,
                                 const float* ln_b, float ln_eps, int act, int batch, int dim, int hidden, int width,
                                 float* hidden_buf, float* delta_out, float* pre_out, float* state_out, float* peer_state,
                                 uint32_t* peer_flag, uint32_t seq, uint32_t* done_counter, cudaStream_t stream);

// Receiver side of the hand-off: wait until flag >= seq, then copy the mailbox into `out`.
int lbi_wait_state(const float* mailbox, const uint32_t* flag, uint32_t seq, float* out, int n, int* status,
                   cudaStream_t stream);

// Publish: make this rank's scan inputs (already written into its symmetric buffer) visible and raise its flag on
// every peer.  Runs after the kernels that wrote the buffer, on the same stream.
int lbi_peer_signal_all(uint32_t* const* flag_ptrs, int rank, int world, int slot_base, uint32_t seq,
                        cudaStream_t stream);

// Cross-GPU affine suffix scan  g_k = b_k + A_k^T g_{k+1},  g_K = 0  over K = world * k_local regions.  Region k lives
// in the buffer of rank k / k_local: mats [B, k_local, R, R] and offsets [B, k_local, R] (fp32).  Every rank waits for
// the flags of the ranks whose regions it reads, loads their matrices with plain peer loads and writes all g_k
// ([B, K, R]) into its own memory.  The Jacobian of the last region is never read.
int lbi_affine_scan_peer(const float* const* mats_ptrs, const float* const* offs_ptrs, const uint32_t* flags,
                         int slot_base, uint32_t seq, float* g, int batch, int world, int k_local, int r, int* status,
                         cudaStream_t stream);

// Basis-parallel form of the cross-GPU scan: every rank publishes partial rows [K, B, R, R] (rows[k][b][j][a] =
// d s_out[j] / d s_in[a], zero where another rank did the work) and partial offsets [K, B, R]; the kernel sums them over
// the ranks as it loads them and writes all g_k ([B, K, R]) on every rank.
int lbi_affine_scan_peer_sum(const float* const* rows_ptrs, const float* const* offs_ptrs, const uint32_t* flags, int slot_base,
                             uint32_t seq, float* g, int batch, int world, int k_total, int r, int flag_world, int* status,
                             cudaStream_t stream);
// Copy segments (offset, length in floats, multiples of 4) of src_a / src_b into the same offsets of every rank's buffer
// (dst_a[w], dst_b[w]: peer pointers, w < world, this rank included), then raise flag slot_base + rank on every peer to seq.
// done_counter: one zero-initialised uint32 owned by the caller (left at zero).
int lbi_peer_publish(const float* src_a, float* const* dst_a, const int64_t* segs_a, int n_a, const float* src_b,
                     float* const* dst_b, const int64_t* segs_b, int n_b, uint32_t* const* flag_ptrs, int rank, int world,
                     int slot_base, uint32_t seq, uint32_t* done_counter, cudaStream_t stream);

// Gradient reduce-scatter by peer loads: reduced[i] = sum_w grad_ptrs[w][lo + i] for this rank's shard, written back
// into this rank's own buffer at [lo, lo + n), with sum of squares of the reduced shard added to *sumsq.
// mc_grads: optional NVLS multicast address of the gradient buffer (multimem.ld_reduce); null selects peer loads.
int lbi_grad_reduce_scatter(float* const* grad_ptrs, const float* mc_grads, int rank, int world, int64_t lo, int64_t n,
                            float* sumsq, cudaStream_t stream);

// Exchange one float per rank (the shard's sum of squares): slot[rank] of every peer's `vals` array, then flags.
int lbi_exchange_scalar(float* const* val_ptrs, uint32_t* const* flag_ptrs, const float* mine, int rank, int world,
                        int slot_base, uint32_t seq, int* status, cudaStream_t stream);

// Clip + AdamW on this rank's shard, fused with the all-gather of the updated bf16 weights: the new weights are
// stored into every peer's shadow buffer at [lo, lo + n).  total_sumsq_parts: `world` floats (one per rank).
int lbi_adamw_allgather(float* param, const float* reduced_grad, float* exp_avg, float* exp_avg_sq,
                        void* const* shadow_ptrs, int world, int64_t lo, int64_t n, float lr, float beta1, float beta2,
                        float eps, float weight_decay, int step, const float* sumsq_parts, float clip_norm,
                        cudaStream_t stream);

#ifdef __cplusplus
}
#endif
