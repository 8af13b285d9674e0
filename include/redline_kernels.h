/*
 * redline_kernels.h - C ABI of the B200 (sm_100a) non-GEMM decode kernels.
 *
 * One entry point per launcher of the reference's kernel contract
 * (Kasamix/redline-llm, src/kernels/kernels.cuh), with that launcher's
 * parameter list flattened to C types: FP16 tensors travel as void pointers to
 * device memory, strides are int64 element counts, counts are int32, the stream
 * is a cudaStream_t passed as void*. A C++ caller includes
 * redline_llm_b200/csrc/kernels.cuh instead, which restores the reference's
 * exact signatures in namespace redline::kernels and forwards here.
 *
 * Conventions (as src/kernels/kernels.cuh:12-32):
 *   - every pointer is a device pointer; every launch is asynchronous on
 *     `stream`; nothing synchronises internally;
 *   - FP16 storage, FP32 accumulation in every reduction;
 *   - one layer's KV pool slice is [num_blocks, 2 (0=K,1=V), num_kv_heads, 16,
 *     head_dim]; block-table rows are padded with block 0 (reserved);
 *   - zero extents return at once; odd shapes and 2-byte-aligned bases take a
 *     scalar kernel, never an error;
 *   - after the first call on a device (which may query device attributes and
 *     opt in to large dynamic shared memory) a launcher issues no CUDA API call
 *     but the launch, so it is legal inside CUDA-graph stream capture.
 *
 * Every function returns 0 on success, a positive cudaError_t when the launch
 * failed, or a negative RL_E_* code when the arguments break the contract;
 * rl_last_error() gives the text. There is no CPU fallback of any kind.
 */
#ifndef REDLINE_KERNELS_H_
#define REDLINE_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RL_OK 0
#define RL_E_NULL_POINTER (-1)
#define RL_E_BAD_SHAPE (-2)
#define RL_E_WORKSPACE (-3)
#define RL_E_TOO_LARGE (-4)

/* Library version string ("0.1.0"; mirrors redline.__version__, src/api/pybind.cpp:104-214). */
const char* rl_version(void);

/* Text of the last non-zero status returned on the calling thread. */
const char* rl_last_error(void);

/*
 * Optional warm-up for `device` (-1 = current): caches the SM count, opts the
 * attention kernel in to its dynamic shared memory and allocates the attention
 * workspace. The launchers do the same lazily on their first call; an engine
 * calls this (or performs one eager launch of each kernel, as the reference's
 * bucket warm-up does, src/core/model_executor.cpp:504-521) before capture.
 * No counterpart in the reference (its kernels keep no per-device state but
 * RoPE's constant table, src/kernels/rope.cu:123-176).
 */
int rl_kernels_init(int device);

/* out[t,:] = rmsnorm(input[t,:]) * weight.  Replaces LaunchRmsNorm,
 * src/kernels/kernels.cuh:54-55 (src/kernels/rmsnorm.cu:436-450). */
int rl_launch_rmsnorm(void* out, const void* input, const void* weight, int32_t num_tokens,
                      int32_t hidden_size, float eps, void* stream);

/* h = fp16(residual + input); residual <- h; out = fp16(fp16(h * rsqrt(mean(h^2) + eps)) * weight).
 * out, residual and input are pairwise distinct. Replaces LaunchRmsNormResidual,
 * src/kernels/kernels.cuh:66-68 (src/kernels/rmsnorm.cu:452-470). */
int rl_launch_rmsnorm_residual(void* out, void* residual, const void* input, const void* weight,
                               int32_t num_tokens, int32_t hidden_size, float eps, void* stream);

/* NeoX half-rotation in place on the Q and K views. Replaces LaunchRopeInplace,
 * src/kernels/kernels.cuh:78-81 (src/kernels/rope.cu:320-362). */
int rl_launch_rope_inplace(void* q, void* k, int64_t q_row_stride, int64_t k_row_stride,
                           const int32_t* positions, int32_t num_tokens, int32_t num_q_heads,
                           int32_t num_kv_heads, int32_t head_dim, float rope_theta, void* stream);

/* Bit-move of this step's K,V rows into the paged pool: p = positions[t],
 * block = block_tables[t*block_table_row_stride + (p >> 4)], slot = p & 15.
 * Replaces LaunchKvScatter, src/kernels/kernels.cuh:95-99 (src/kernels/kv_scatter.cu:146-176). */
int rl_launch_kv_scatter(void* kv_pool_layer, const void* k, const void* v, int64_t k_row_stride,
                         int64_t v_row_stride, const int32_t* block_tables,
                         int64_t block_table_row_stride, const int32_t* positions,
                         int32_t num_tokens, int32_t num_kv_heads, int32_t head_dim, void* stream);

/*
 * RoPE and KV scatter in ONE launch: exactly rl_launch_rope_inplace followed by
 * rl_launch_kv_scatter (same buffers, bit-identical results in the qkv buffer and in the pool),
 * saving a launch and a pass over K per layer. The reference runs the two launchers back to back
 * (src/core/model_executor.cpp:924-930) and has no fused form; an executor opts in by replacing
 * those two calls with this one.
 */
int rl_launch_rope_kv_scatter(void* q, void* k, const void* v, int64_t q_row_stride, int64_t k_row_stride,
                              int64_t v_row_stride, void* kv_pool_layer, const int32_t* block_tables,
                              int64_t block_table_row_stride, const int32_t* positions, int32_t num_tokens,
                              int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float rope_theta,
                              void* stream);

/*
 * Paged grouped-query decode attention, one query token per sequence, online
 * softmax with FP32 statistics and accumulation; rows with seq_len <= 0 are not
 * written. head_dim must be 128 and num_q_heads == 6 * num_kv_heads (as the
 * reference, src/kernels/paged_attention.cu:459-484,519-520). The KV axis is
 * split across the whole grid in balanced page ranges and merged in a fixed
 * order (the reference has no split variant: one CTA walks a whole (sequence, head) serially,
 * src/kernels/paged_attention.cu:176,214), so long and ragged contexts need no other entry point.
 * Uses the per-device workspace (see rl_kernels_init).
 * Replaces LaunchPagedAttentionDecode, src/kernels/kernels.cuh:141-146
 * (src/kernels/paged_attention.cu:507-532).
 */
int rl_launch_paged_attention_decode(void* out, int64_t out_row_stride, const void* q,
                                     int64_t q_row_stride, const void* kv_pool_layer,
                                     const int32_t* block_tables, const int32_t* seq_lens,
                                     int32_t num_seqs, int32_t max_blocks_per_seq,
                                     int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                     float scale, void* stream);

/*
 * Opt-in (default 0): launch the attention kernel with programmatic stream serialisation, so its
 * prologue - the page prefix over seq_lens and the first block-table reads - overlaps the tail of
 * the previous kernel of the stream (this library's KV-scatter / RoPE+scatter kernels and the
 * attention kernel itself release their dependents early), and so do the loads of its first K/V
 * pages other than each sequence's last page. The kernel waits for that previous kernel to complete
 * before it reads Q or any sequence's last page (the page this step's scatter writes) and before it
 * writes anything. Two rules for the caller: seq_lens and block_tables must not be produced by a
 * kernel still in flight when the attention launcher is called (in the reference's executor they are
 * uploaded once per step, src/core/model_executor.cpp:876-892); and such kernels may write the pool
 * only in each sequence's last page, as a decode step's scatter does (after a prefill that scattered
 * whole prompts, synchronise the stream or run one launch without the option). The option also makes
 * the norm / RoPE / scatter / linear launchers use dependent launch. Process-wide; set it before capture.
 * No counterpart in the reference.
 */
int rl_attention_set_prologue_overlap(int enable);

/*
 * The attention launcher for hosts that must not allocate: same arguments, same kernel and
 * bit-identical results as rl_launch_paged_attention_decode, but the split/merge scratch is a
 * ~1.6 MB device array built into the library image (held by every GPU that loads the library
 * until the process exits) instead of a cudaMalloc'd workspace. Meant for callers that cannot
 * call cudaMalloc - a process with a sealed device-memory budget, a plugin inside a host that
 * forbids allocation after start-up. It calls no cudaMalloc, cudaFree or allocating library
 * routine. Limits: at most 1024 sequences per call (RL_E_TOO_LARGE beyond that; the allocating
 * launcher walks larger batches in chunks) and a device of at most 256 SMs.
 * The first call on a device resolves the array's device address, opts the kernel in to its
 * shared memory and looks up the tensor-map encoder; make that first call before any stream
 * capture. Every call clears the array's counters in stream order and then reuses the same
 * array (it keeps the previous call's contents otherwise), so two calls of THIS entry point that
 * overlap on one GPU - issued on different streams, say - race on it; serialise them. The
 * allocating launcher has its own workspace and does not interfere. A bounded wait that gave up
 * sets a flag inside the array that stays set across calls until rl_attention_health - which
 * reports on this array as well as on the allocating launcher's workspace - has returned it.
 * This entry point has no counterpart in the reference.
 */
int rl_launch_paged_attention_decode_static(void* out, int64_t out_row_stride, const void* q,
                                            int64_t q_row_stride, const void* kv_pool_layer,
                                            const int32_t* block_tables, const int32_t* seq_lens,
                                            int32_t num_seqs, int32_t max_blocks_per_seq,
                                            int32_t num_q_heads, int32_t num_kv_heads,
                                            int32_t head_dim, float scale, void* stream);

/*
 * Fused paged prefill attention: the `chunk_len` query rows of one prompt chunk (absolute positions
 * chunk_start .. chunk_start + chunk_len - 1 of ONE sequence, already rotated by RoPE, rows q_row_stride
 * elements apart) attend causally to every key of that sequence up to their own position, read straight
 * from the paged pool through the sequence's block-table row (which must cover chunk_start + chunk_len
 * tokens; the chunk's own K/V must already have been scattered). Scores q.k * scale in FP32, masking by
 * SELECT (key position <= query position; slots and pages past the context never reach a result),
 * softmax with FP32 statistics, probabilities rounded to FP16 for P.V, FP32 accumulation, one FP16
 * rounding; out[row, head * 128 ..] is written for the chunk's rows only. head_dim must be 128,
 * num_q_heads a multiple of num_kv_heads (<= 8 KV heads); q, out and the pool slice 16-byte aligned, row
 * strides multiples of 8. One CTA per (128-row query tile, query head) or per run of key blocks of such a
 * pair: TMA page tiles, tcgen05 for Q.K^T and P.V with accumulators in tensor memory. The call enqueues one
 * kernel, or two when pairs were cut into runs (the second combines the runs' records in run order).
 * No single launcher of the reference corresponds: this replaces its prefill composite LaunchKvGather ->
 * cuBLASLt scores -> LaunchPrefillSoftmax -> cuBLASLt P.V (src/core/model_executor.cpp:1219-1290), the
 * fused kernel its design notes name as the follow-up (docs/DESIGN.md:872-876 of the reference).
 */
int rl_launch_paged_prefill_attention(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride,
                                      const void* kv_pool_layer, const int32_t* block_table_row,
                                      int32_t max_blocks_per_seq, int32_t chunk_start, int32_t chunk_len,
                                      int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
                                      void* stream);

/* Health of the prefill attention kernel's bounded waits on the current device (as rl_attention_health). */
int rl_prefill_attention_health(int* flag_out);

/*
 * Tuning knob of rl_launch_paged_prefill_attention: the longest run of 128-key blocks one CTA takes before a
 * (query tile, head) pair is cut across CTAs (their records are combined in run order by a second kernel of the
 * same launch call, so results do not depend on it beyond FP32 summation order). 0 (default) = chosen per launch from the
 * chunk's shape and the SM count. Process-wide. A launch that cuts pairs keeps a scratch area in device memory
 * (grown on demand outside stream capture, 66 KB per work item). No counterpart in the reference.
 */
int rl_prefill_attention_set_split_blocks(int blocks);

/*
 * The run length rl_launch_paged_prefill_attention would use for a chunk on a device of `sm_count` SMs: a
 * (query tile, head) pair with more 128-key blocks than this is cut into equal runs on separate CTAs. Host
 * arithmetic only (a replay of the launch: work items in grid order, each onto the SM that frees first); needs
 * no device. No counterpart in the reference.
 */
int rl_prefill_attention_run_length(int32_t chunk_start, int32_t chunk_len, int32_t num_q_heads, int32_t sm_count,
                                    int32_t* run_blocks_out);

/*
 * Decode input plumbing on the device: after a step's greedy argmax, prepare the next step's inputs in
 * place - input_ids[i] <- control[1 + i] if that is >= 0 (a scripted token), else sampled_tokens[i];
 * positions[i] <- seq_lens[i]; seq_lens[i] += 1 - for every row with seq_len > 0, when control[0] != 0
 * (control = int32[1 + num_rows] in device memory; control[0] == 0 leaves everything as it is). Placed at
 * the end of the captured decode sequence it lets an executor replay the graph of an unchanged batch
 * without reading the tokens back first; block tables must then already hold the page the next token
 * falls into. Replaces, on the device, the host loop of src/core/model_executor.cpp:784-874 for the
 * steady state (the reference rebuilds and uploads the three arrays every step, :876-892).
 */
int rl_launch_decode_advance(int32_t* input_ids, int32_t* positions, int32_t* seq_lens,
                             const int32_t* sampled_tokens, const int32_t* control, int32_t num_rows,
                             void* stream);

/*
 * Device-side health of the attention kernel on the current device: 0 when every
 * page load it waited for arrived, 1 when a bounded wait gave up (the output of
 * that launch is then undefined). Synchronises the device; meant for tests and
 * post-mortems, never for the step loop. Clears the flag. No counterpart in the
 * reference (its kernel has no asynchronous waits).
 */
int rl_attention_health(int* flag_out);

/*
 * Test hook for the give-up path of the attention kernel's bounded waits, for launches made after the call:
 * with drop_first_copy != 0 one warp of the first CTA never requests its first K/V page and so waits for a
 * copy that cannot arrive; wait_cycles > 0 replaces the limit of every wait (about a second by default) so
 * that the test takes a millisecond. The kernel then raises the health flag, lets its other copies land,
 * and returns normally with that launch's output undefined - nothing faults, traps or spins without bound,
 * and the context stays usable. (0, 0) restores normal operation. Process-wide; not for serving code.
 * No counterpart in the reference (its kernel has no asynchronous waits).
 */
int rl_attention_test_wait_expiry(int drop_first_copy, int64_t wait_cycles);

/* Same contract, one warp per (sequence, query head), two-pass softmax on CUDA
 * cores: a structurally independent cross-check for tests. Replaces
 * LaunchPagedAttentionDecodeOracle, src/kernels/kernels.cuh:152-158. */
int rl_launch_paged_attention_decode_check(void* out, int64_t out_row_stride, const void* q,
                                           int64_t q_row_stride, const void* kv_pool_layer,
                                           const int32_t* block_tables, const int32_t* seq_lens,
                                           int32_t num_seqs, int32_t max_blocks_per_seq,
                                           int32_t num_q_heads, int32_t num_kv_heads,
                                           int32_t head_dim, float scale, void* stream);

/* out[t,i] = fp16(silu(gate_up[t,i]) * gate_up[t,I+i]); out == gate_up writes in place over the
 * gate half (row stride 2I), any other out is dense [T,I]. Replaces LaunchSiluMul,
 * src/kernels/kernels.cuh:192-193 (src/kernels/silu_mul.cu:129-169). */
int rl_launch_silu_mul(void* out, const void* gate_up, int32_t num_tokens,
                       int32_t intermediate_size, void* stream);

/* out[t,:] = embed[input_ids[t],:], a bit move; the first launch of every decode step.
 * Replaces LaunchEmbedGather, src/kernels/kernels.cuh:48-50 (src/kernels/embed_gather.cu:121-156). */
int rl_launch_embed_gather(void* out, int64_t out_row_stride, const void* embed,
                           const int32_t* input_ids, int32_t num_tokens, int32_t hidden_size,
                           void* stream);

/* Per-row index of the largest logit: FP32 compares, ties to the lowest index, a NaN never wins,
 * an all-NaN row gives token 0. logits is dense [num_seqs, vocab_size]. Replaces
 * LaunchGreedyArgmax, src/kernels/kernels.cuh:198-199 (src/kernels/argmax.cu:228-252). */
int rl_launch_greedy_argmax(int32_t* out_tokens, const void* logits, int32_t num_seqs,
                            int32_t vocab_size, void* stream);

/* Prefill-only: one sequence's cached K/V from the paged pool into dense [kv_heads, ctx_len,
 * head_dim] staging views (position t <- block_table_row[t >> 4], slot t & 15), a bit move.
 * Replaces LaunchKvGather, src/kernels/kernels.cuh:119-123 (src/kernels/kv_gather.cu:136-168). */
int rl_launch_kv_gather(void* khat, void* vhat, int64_t khat_head_stride, int64_t khat_row_stride,
                        int64_t vhat_head_stride, int64_t vhat_row_stride, const void* kv_pool_layer,
                        const int32_t* block_table_row, int32_t ctx_len, int32_t num_kv_heads,
                        int32_t head_dim, void* stream);

/* Prefill-only: causal row softmax FP32 -> FP16 over dense [heads, chunk_len, kv_len]; row i sees
 * keys j <= chunk_start + i; masked entries become exact +0 and their scores are select-masked: whatever
 * they hold (NaN included) reaches no result; at most the rest of the 32-byte group that holds the last
 * live score is loaded, and discarded. Replaces
 * LaunchPrefillSoftmax, src/kernels/kernels.cuh:185-187 (src/kernels/prefill_attention.cu:166-192). */
int rl_launch_prefill_softmax(void* probs, const float* scores, int32_t num_q_heads, int32_t chunk_len,
                              int32_t kv_len, int32_t chunk_start, void* stream);

/*
 * Linear layer of the decode step for at most 64 token rows:
 *   out[t, n] = fp16( sum_k x[t, k] * weight[n, k]  (+ bias[n]) ),  FP16 in, FP32 accumulate, one rounding.
 * Replaces the cuBLASLt call behind CublasLtGemm::Run for the decode shapes
 * (src/gemm/cublaslt_gemm.cpp:569-598; call sites src/core/model_executor.cpp:916-951): with so few
 * rows the product is a stream over the weights, and this kernel (TMA + tcgen05, split along K where
 * the shape has few row tiles) is built to run it at HBM speed. Row strides are in elements; x and
 * weight rows must be 16-byte aligned and in_features a multiple of 8. More than 64 token rows
 * returns RL_E_TOO_LARGE: prefill-sized products stay with the library.
 *   epilogue 0: bias (may be NULL) added in FP32 before the rounding; out is [num_tokens, out_features].
 *   epilogue 1: the gated-MLP input. weight has 2*out_features rows, `gate` rows first, then `up` rows;
 *               out[t, c] = fp16( silu(fp16(gate_acc)) * fp16(up_acc) ), i.e. exactly rl_launch_silu_mul
 *               applied to the rounded GEMM output, without storing the [num_tokens, 2*out_features]
 *               intermediate. bias must be NULL.
 * Results do not depend on arrival order or on the ring depth (fixed summation order).
 * Outputs of at least three 128-row tiles per SM (a vocabulary projection) run with a 3-stage ring, several
 * CTAs per SM, and their weights at normal L2 priority; every other shape streams its weights evict-first.
 * First call per device must happen outside stream capture (it opts in to large shared memory and
 * allocates a 256-byte error flag).
 */
int rl_launch_decode_linear(void* out, int64_t out_row_stride, const void* x, int64_t x_row_stride,
                            const void* weight, int64_t weight_row_stride, const void* bias,
                            int32_t num_tokens, int32_t out_features, int32_t in_features,
                            int32_t epilogue, void* stream);

/*
 * The QKV projection of a decode step with RoPE and the KV scatter in its epilogue: exactly
 * rl_launch_decode_linear (epilogue 0, bias) into the fused qkv buffer (Q heads | K heads | V heads per row),
 * followed by rl_launch_rope_inplace on the Q and K views and rl_launch_kv_scatter of K and V - same bits in
 * the qkv buffer and in the pool, one launch instead of three (src/core/model_executor.cpp:916-930 runs the
 * GEMM and the two kernels back to back). head_dim must be 128 (a 128-row weight tile is one head, so the CTA
 * that finishes a token of a tile holds that token's whole head). weight is [(q_heads + 2 kv_heads) * 128,
 * in_features]. Shapes the kernel would not split along K take the three-launch route internally.
 * With dependent launch on (rl_attention_set_prologue_overlap) positions and block_tables are read before the
 * launch waits for the previous kernel, like seq_lens and block_tables in the attention launcher: they must
 * not be produced by a kernel still in flight (an executor uploads them at the start of the step).
 */
int rl_launch_qkv_rope_kv_scatter(void* qkv, int64_t qkv_row_stride, const void* x, int64_t x_row_stride,
                                  const void* weight, int64_t weight_row_stride, const void* bias,
                                  int32_t num_tokens, int32_t in_features, void* kv_pool_layer,
                                  const int32_t* block_tables, int64_t block_table_row_stride,
                                  const int32_t* positions, int32_t num_q_heads, int32_t num_kv_heads,
                                  int32_t head_dim, float rope_theta, void* stream);

/* Synchronises the device and reports (then clears) the error flag of rl_launch_decode_linear:
 * 0 = every bounded wait inside the kernel completed; 1..4 name the wait that gave up. */
int rl_decode_linear_health(int* flag_out);

/* Tuning: depth of the kernel's shared-memory ring, 2..8 stages of 24 KB (default 6; a launch never uses
 * more stages than its longest K split has k-blocks). Process-wide; affects later launches. */
int rl_decode_linear_set_stages(int stages);

/* Tuning: the largest number of CTAs a row tile may be split into along K (1, 2, 4 or 8; default 8).
 * The split count is a function of the shape and of this cap only, and the partial sums are added in a
 * fixed order, so a given (shape, cap) always gives the same bits; different caps may differ in the
 * last FP32 bit of the accumulated sum. Process-wide; affects later launches. */
int rl_decode_linear_set_max_splits(int max_splits);

#ifdef __cplusplus
}
#endif
#endif /* REDLINE_KERNELS_H_ */
