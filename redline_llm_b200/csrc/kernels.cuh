// Drop-in for the reference's src/kernels/kernels.cuh: the same host launchers,
// the same namespace, parameter lists and conventions, forwarded to the C ABI of
// the sm_100a library (include/redline_kernels.h, libredline_b200.so). A caller
// such as the reference's executor (src/core/model_executor.cpp:894-961,
// 1154-1217) or its kernel unit suite (tests/test_kernels.cu) compiles against
// this header unchanged and links the library instead of the reference's
// src/kernels/*.cu objects.
//
// Conventions are the reference's (src/kernels/kernels.cuh:12-32): device
// pointers, asynchronous on `stream`, explicit row strides in elements, FP16
// storage with FP32 accumulation, one layer's pool slice
// [num_blocks, 2, num_kv_heads, 16, head_dim], block tables padded with block 0.
// The launchers return void as the reference's do; a contract violation that the
// reference answers with fprintf + abort (src/kernels/paged_attention.cu:459-464)
// is answered the same way here, a launch error stays observable through
// cudaGetLastError() after the step's synchronisation
// (src/core/model_executor.cpp:711-712).
//
// All eleven launchers of the reference header are provided: the nine inside the
// captured decode graph (LaunchEmbedGather, LaunchRmsNorm, LaunchRmsNormResidual,
// LaunchRopeInplace, LaunchKvScatter, LaunchPagedAttentionDecode + the test-only
// cross-check launcher, LaunchSiluMul, LaunchGreedyArgmax) and the two prefill-only
// ones (LaunchKvGather, LaunchPrefillSoftmax).
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/redline_kernels.h"

namespace redline::kernels {

namespace detail {
// Contract violations (negative status) are programming errors: fail loudly, as
// the reference's RequireContract does. Positive statuses are CUDA launch errors
// and stay sticky in the runtime for the caller's cudaGetLastError().
inline void Check(int status, const char* launcher) {
  if (status < 0) {
    std::fprintf(stderr, "redline: %s: launch contract violated: %s\n", launcher, rl_last_error());
    std::abort();
  }
}
}  // namespace detail

inline void LaunchEmbedGather(half* out, std::int64_t out_row_stride, const half* embed,
                              const std::int32_t* input_ids, std::int32_t num_tokens,
                              std::int32_t hidden_size, cudaStream_t stream) {
  detail::Check(rl_launch_embed_gather(out, out_row_stride, embed, input_ids, num_tokens, hidden_size,
                                       stream),
                "LaunchEmbedGather");
}

inline void LaunchGreedyArgmax(std::int32_t* out_tokens, const half* logits, std::int32_t num_seqs,
                               std::int32_t vocab_size, cudaStream_t stream) {
  detail::Check(rl_launch_greedy_argmax(out_tokens, logits, num_seqs, vocab_size, stream),
                "LaunchGreedyArgmax");
}

inline void LaunchRmsNorm(half* out, const half* input, const half* weight, std::int32_t num_tokens,
                          std::int32_t hidden_size, float eps, cudaStream_t stream) {
  detail::Check(rl_launch_rmsnorm(out, input, weight, num_tokens, hidden_size, eps, stream),
                "LaunchRmsNorm");
}

inline void LaunchRmsNormResidual(half* out, half* residual, const half* input, const half* weight,
                                  std::int32_t num_tokens, std::int32_t hidden_size, float eps,
                                  cudaStream_t stream) {
  detail::Check(rl_launch_rmsnorm_residual(out, residual, input, weight, num_tokens, hidden_size, eps,
                                           stream),
                "LaunchRmsNormResidual");
}

inline void LaunchRopeInplace(half* q, half* k, std::int64_t q_row_stride, std::int64_t k_row_stride,
                              const std::int32_t* positions, std::int32_t num_tokens,
                              std::int32_t num_q_heads, std::int32_t num_kv_heads,
                              std::int32_t head_dim, float rope_theta, cudaStream_t stream) {
  // The reference skips silently on a bad head_dim / theta in release builds
  // (src/kernels/rope.cu:329-344); keep that behaviour for this launcher.
  (void)rl_launch_rope_inplace(q, k, q_row_stride, k_row_stride, positions, num_tokens, num_q_heads,
                               num_kv_heads, head_dim, rope_theta, stream);
}

inline void LaunchKvScatter(half* kv_pool_layer, const half* k, const half* v,
                            std::int64_t k_row_stride, std::int64_t v_row_stride,
                            const std::int32_t* block_tables, std::int64_t block_table_row_stride,
                            const std::int32_t* positions, std::int32_t num_tokens,
                            std::int32_t num_kv_heads, std::int32_t head_dim, cudaStream_t stream) {
  detail::Check(rl_launch_kv_scatter(kv_pool_layer, k, v, k_row_stride, v_row_stride, block_tables,
                                     block_table_row_stride, positions, num_tokens, num_kv_heads,
                                     head_dim, stream),
                "LaunchKvScatter");
}

inline void LaunchPagedAttentionDecode(half* out, std::int64_t out_row_stride, const half* q,
                                       std::int64_t q_row_stride, const half* kv_pool_layer,
                                       const std::int32_t* block_tables,
                                       const std::int32_t* seq_lens, std::int32_t num_seqs,
                                       std::int32_t max_blocks_per_seq, std::int32_t num_q_heads,
                                       std::int32_t num_kv_heads, std::int32_t head_dim, float scale,
                                       cudaStream_t stream) {
  detail::Check(rl_launch_paged_attention_decode(out, out_row_stride, q, q_row_stride, kv_pool_layer,
                                                 block_tables, seq_lens, num_seqs, max_blocks_per_seq,
                                                 num_q_heads, num_kv_heads, head_dim, scale, stream),
                "LaunchPagedAttentionDecode");
}

inline void LaunchPagedAttentionDecodeOracle(half* out, std::int64_t out_row_stride, const half* q,
                                             std::int64_t q_row_stride, const half* kv_pool_layer,
                                             const std::int32_t* block_tables,
                                             const std::int32_t* seq_lens, std::int32_t num_seqs,
                                             std::int32_t max_blocks_per_seq,
                                             std::int32_t num_q_heads, std::int32_t num_kv_heads,
                                             std::int32_t head_dim, float scale, cudaStream_t stream) {
  detail::Check(rl_launch_paged_attention_decode_check(out, out_row_stride, q, q_row_stride,
                                                       kv_pool_layer, block_tables, seq_lens, num_seqs,
                                                       max_blocks_per_seq, num_q_heads, num_kv_heads,
                                                       head_dim, scale, stream),
                "LaunchPagedAttentionDecodeOracle");
}

inline void LaunchKvGather(half* khat, half* vhat, std::int64_t khat_head_stride,
                           std::int64_t khat_row_stride, std::int64_t vhat_head_stride,
                           std::int64_t vhat_row_stride, const half* kv_pool_layer,
                           const std::int32_t* block_table_row, std::int32_t ctx_len,
                           std::int32_t num_kv_heads, std::int32_t head_dim, cudaStream_t stream) {
  detail::Check(rl_launch_kv_gather(khat, vhat, khat_head_stride, khat_row_stride, vhat_head_stride,
                                    vhat_row_stride, kv_pool_layer, block_table_row, ctx_len, num_kv_heads,
                                    head_dim, stream),
                "LaunchKvGather");
}

inline void LaunchPrefillSoftmax(half* probs, const float* scores, std::int32_t num_q_heads,
                                 std::int32_t chunk_len, std::int32_t kv_len, std::int32_t chunk_start,
                                 cudaStream_t stream) {
  detail::Check(rl_launch_prefill_softmax(probs, scores, num_q_heads, chunk_len, kv_len, chunk_start, stream),
                "LaunchPrefillSoftmax");
}

inline void LaunchSiluMul(half* out, const half* gate_up, std::int32_t num_tokens,
                          std::int32_t intermediate_size, cudaStream_t stream) {
  detail::Check(rl_launch_silu_mul(out, gate_up, num_tokens, intermediate_size, stream),
                "LaunchSiluMul");
}

// ---- beyond the reference header: the linear layers of the decode step (no counterpart in
// src/kernels/; an executor opts in where it calls its GEMM wrapper, src/core/model_executor.cpp:916-951).

// out[T, N] = x[T, K] . weight[N, K]^T (+ bias), T <= 64. silu_mul = true: weight is [2N, K] (gate rows, then
// up rows), bias must be null, out[T, N] = silu(gate) * up.
inline void LaunchDecodeLinear(half* out, std::int64_t out_row_stride, const half* x, std::int64_t x_row_stride,
                               const half* weight, std::int64_t weight_row_stride, const half* bias,
                               std::int32_t num_tokens, std::int32_t out_features, std::int32_t in_features,
                               bool silu_mul, cudaStream_t stream) {
  detail::Check(rl_launch_decode_linear(out, out_row_stride, x, x_row_stride, weight, weight_row_stride, bias,
                                        num_tokens, out_features, in_features, silu_mul ? 1 : 0, stream),
                "LaunchDecodeLinear");
}

// QKV projection + LaunchRopeInplace + LaunchKvScatter in one launch, same bits (head_dim 128).
inline void LaunchQkvRopeKvScatter(half* qkv, std::int64_t qkv_row_stride, const half* x, std::int64_t x_row_stride,
                                   const half* weight, std::int64_t weight_row_stride, const half* bias,
                                   std::int32_t num_tokens, std::int32_t in_features, half* kv_pool_layer,
                                   const std::int32_t* block_tables, std::int64_t block_table_row_stride,
                                   const std::int32_t* positions, std::int32_t num_q_heads,
                                   std::int32_t num_kv_heads, std::int32_t head_dim, float rope_theta,
                                   cudaStream_t stream) {
  detail::Check(rl_launch_qkv_rope_kv_scatter(qkv, qkv_row_stride, x, x_row_stride, weight, weight_row_stride, bias,
                                              num_tokens, in_features, kv_pool_layer, block_tables,
                                              block_table_row_stride, positions, num_q_heads, num_kv_heads,
                                              head_dim, rope_theta, stream),
                "LaunchQkvRopeKvScatter");
}

}  // namespace redline::kernels
