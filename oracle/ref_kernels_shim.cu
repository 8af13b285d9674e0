// ref_kernels_shim.cu - C-ABI doorway onto the reference's OWN CUDA kernels
// (src/kernels/*.cu of Kasamix/redline-llm), which the Makefile compiles for
// sm_100a from the sources where they lie in the mounted reference tree and
// links with this file into oracle/_ref/libredline_refkernels.so. Nothing of
// the reference is copied into this repository.
//
// TEST INFRASTRUCTURE: the GPU-side comparator. The tests run the reference's
// kernels on the same device buffers as this library's kernels, the benchmark
// times them beside its own (the `ref_us` column), and the free-running decode
// check drives a whole model through them. The shipped library never loads
// this file's output.
//
// Every entry point has the parameter list of the rl_launch_* function of the
// same launcher (include/redline_kernels.h), so one ctypes signature serves
// both libraries. The reference launchers return void; a launch error is
// reported from cudaPeekAtLastError (left sticky for the caller's own check).
#include <cstdint>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels/kernels.cuh"  // the reference's header, found through -I<reference>/src

namespace rk = redline::kernels;

namespace {
inline cudaStream_t S(void* stream) { return static_cast<cudaStream_t>(stream); }
inline int Status() { return static_cast<int>(cudaPeekAtLastError()); }
inline half* H(void* p) { return static_cast<half*>(p); }
inline const half* H(const void* p) { return static_cast<const half*>(p); }
}  // namespace

extern "C" {

int refk_launch_embed_gather(void* out, int64_t out_row_stride, const void* embed, const int32_t* input_ids,
                             int32_t num_tokens, int32_t hidden_size, void* stream) {
  rk::LaunchEmbedGather(H(out), out_row_stride, H(embed), input_ids, num_tokens, hidden_size, S(stream));
  return Status();
}

int refk_launch_rmsnorm(void* out, const void* input, const void* weight, int32_t num_tokens,
                        int32_t hidden_size, float eps, void* stream) {
  rk::LaunchRmsNorm(H(out), H(input), H(weight), num_tokens, hidden_size, eps, S(stream));
  return Status();
}

int refk_launch_rmsnorm_residual(void* out, void* residual, const void* input, const void* weight,
                                 int32_t num_tokens, int32_t hidden_size, float eps, void* stream) {
  rk::LaunchRmsNormResidual(H(out), H(residual), H(input), H(weight), num_tokens, hidden_size, eps, S(stream));
  return Status();
}

int refk_launch_rope_inplace(void* q, void* k, int64_t q_row_stride, int64_t k_row_stride,
                             const int32_t* positions, int32_t num_tokens, int32_t num_q_heads,
                             int32_t num_kv_heads, int32_t head_dim, float rope_theta, void* stream) {
  rk::LaunchRopeInplace(H(q), H(k), q_row_stride, k_row_stride, positions, num_tokens, num_q_heads, num_kv_heads,
                        head_dim, rope_theta, S(stream));
  return Status();
}

int refk_launch_kv_scatter(void* kv_pool_layer, const void* k, const void* v, int64_t k_row_stride,
                           int64_t v_row_stride, const int32_t* block_tables, int64_t block_table_row_stride,
                           const int32_t* positions, int32_t num_tokens, int32_t num_kv_heads,
                           int32_t head_dim, void* stream) {
  rk::LaunchKvScatter(H(kv_pool_layer), H(k), H(v), k_row_stride, v_row_stride, block_tables,
                      block_table_row_stride, positions, num_tokens, num_kv_heads, head_dim, S(stream));
  return Status();
}

int refk_launch_kv_gather(void* khat, void* vhat, int64_t khat_head_stride, int64_t khat_row_stride,
                          int64_t vhat_head_stride, int64_t vhat_row_stride, const void* kv_pool_layer,
                          const int32_t* block_table_row, int32_t ctx_len, int32_t num_kv_heads,
                          int32_t head_dim, void* stream) {
  rk::LaunchKvGather(H(khat), H(vhat), khat_head_stride, khat_row_stride, vhat_head_stride, vhat_row_stride,
                     H(kv_pool_layer), block_table_row, ctx_len, num_kv_heads, head_dim, S(stream));
  return Status();
}

int refk_launch_paged_attention_decode(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride,
                                       const void* kv_pool_layer, const int32_t* block_tables,
                                       const int32_t* seq_lens, int32_t num_seqs, int32_t max_blocks_per_seq,
                                       int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
                                       void* stream) {
  rk::LaunchPagedAttentionDecode(H(out), out_row_stride, H(q), q_row_stride, H(kv_pool_layer), block_tables,
                                 seq_lens, num_seqs, max_blocks_per_seq, num_q_heads, num_kv_heads, head_dim,
                                 scale, S(stream));
  return Status();
}

int refk_launch_paged_attention_decode_check(void* out, int64_t out_row_stride, const void* q,
                                             int64_t q_row_stride, const void* kv_pool_layer,
                                             const int32_t* block_tables, const int32_t* seq_lens,
                                             int32_t num_seqs, int32_t max_blocks_per_seq, int32_t num_q_heads,
                                             int32_t num_kv_heads, int32_t head_dim, float scale, void* stream) {
  rk::LaunchPagedAttentionDecodeOracle(H(out), out_row_stride, H(q), q_row_stride, H(kv_pool_layer), block_tables,
                                       seq_lens, num_seqs, max_blocks_per_seq, num_q_heads, num_kv_heads,
                                       head_dim, scale, S(stream));
  return Status();
}

int refk_launch_prefill_softmax(void* probs, const float* scores, int32_t num_q_heads, int32_t chunk_len,
                                int32_t kv_len, int32_t chunk_start, void* stream) {
  rk::LaunchPrefillSoftmax(H(probs), scores, num_q_heads, chunk_len, kv_len, chunk_start, S(stream));
  return Status();
}

int refk_launch_silu_mul(void* out, const void* gate_up, int32_t num_tokens, int32_t intermediate_size,
                         void* stream) {
  rk::LaunchSiluMul(H(out), H(gate_up), num_tokens, intermediate_size, S(stream));
  return Status();
}

int refk_launch_greedy_argmax(int32_t* out_tokens, const void* logits, int32_t num_seqs, int32_t vocab_size,
                              void* stream) {
  rk::LaunchGreedyArgmax(out_tokens, H(logits), num_seqs, vocab_size, S(stream));
  return Status();
}

}  // extern "C"
