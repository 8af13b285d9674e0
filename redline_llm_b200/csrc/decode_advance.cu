// Decode input plumbing on the device, sm_100a: after a decode step has sampled its tokens, prepare the next
// step's inputs in place - token id <- the sampled token (or the caller's scripted token), position and
// seq_len advanced by one - so that the host need not read the tokens back before it launches the next step.
//
// The reference rebuilds these three arrays on the host every step and uploads them
// (src/core/model_executor.cpp:784-892): the step's critical path then holds a device -> host copy, the
// scheduler's bookkeeping and a host -> device copy between two graph replays. With this kernel at the end
// of the captured decode sequence, consecutive replays of an unchanged batch need no host round trip; the
// host reads each step's tokens one step late and uploads only the small control block.
//
// control[0]      != 0: advance; 0: leave the inputs as they are (replays over resident inputs)
// control[1 + i]  >= 0: the token to feed row i next (teacher forcing); < 0: feed the sampled token
// Rows with seq_len <= 0 are padding and stay untouched (src/core/model_executor.cpp:862-871).
#include "common.cuh"

namespace rl {
namespace {

__global__ void __launch_bounds__(128)
DecodeAdvanceKernel(int32_t* __restrict__ ids, int32_t* __restrict__ positions, int32_t* __restrict__ seq_lens,
                    const int32_t* __restrict__ tokens, const int32_t* __restrict__ control, int rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows || control[0] == 0) return;
  const int len = seq_lens[i];
  if (len <= 0) return;
  const int scripted = control[1 + i];
  ids[i] = scripted >= 0 ? scripted : tokens[i];
  positions[i] = len;       // the new token's position is the old length
  seq_lens[i] = len + 1;
}

}  // namespace
}  // namespace rl

extern "C" int rl_launch_decode_advance(int32_t* input_ids, int32_t* positions, int32_t* seq_lens,
                                        const int32_t* sampled_tokens, const int32_t* control, int32_t num_rows,
                                        void* stream) {
  using namespace rl;
  if (num_rows <= 0) return RL_OK;
  if (!input_ids || !positions || !seq_lens || !sampled_tokens || !control)
    return Fail(RL_E_NULL_POINTER, "decode_advance: null device pointer");
  DecodeAdvanceKernel<<<(num_rows + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      input_ids, positions, seq_lens, sampled_tokens, control, num_rows);
  return LaunchStatus("decode_advance");
}
