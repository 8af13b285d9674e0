// Token-embedding gather, sm_100a: out[t, :] = embed[input_ids[t], :], a pure
// bit move (src/kernels/kernels.cuh:36-50, src/kernels/embed_gather.cu:121-156).
// Padded batch slots carry token 0 and gather row 0; ids are range-checked at
// request admission, never here. One CTA per token row, 16-byte words when the
// row width and the bases allow it (hidden 1536 = 192 words), else halves.
#include "common.cuh"

namespace rl {
namespace {

template <typename Word>
__global__ void __launch_bounds__(256)
EmbedGatherKernel(half* __restrict__ out, int64_t out_row_stride, const half* __restrict__ embed,
                  const int32_t* __restrict__ ids, int hidden) {
  constexpr int kPer = sizeof(Word) / sizeof(half);
  const int64_t t = blockIdx.x;
  const Word* src = reinterpret_cast<const Word*>(embed + static_cast<int64_t>(ids[t]) * hidden);
  Word* dst = reinterpret_cast<Word*>(out + t * out_row_stride);
  for (int w = threadIdx.x; w < hidden / kPer; w += blockDim.x) dst[w] = src[w];
}

}  // namespace
}  // namespace rl

extern "C" int rl_launch_embed_gather(void* out, int64_t out_row_stride, const void* embed,
                                      const int32_t* input_ids, int32_t num_tokens,
                                      int32_t hidden_size, void* stream) {
  using namespace rl;
  if (num_tokens <= 0 || hidden_size <= 0) return RL_OK;
  if (!out || !embed || !input_ids) return Fail(RL_E_NULL_POINTER, "embed_gather: null device pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  half* o = static_cast<half*>(out);
  const half* e = static_cast<const half*>(embed);
  const bool vec = hidden_size % 8 == 0 && out_row_stride % 8 == 0 && Aligned16(out) && Aligned16(embed);
  if (vec) {
    const int threads = hidden_size / 8 >= 256 ? 256 : ((hidden_size / 8 + 31) / 32) * 32;
    EmbedGatherKernel<uint4><<<num_tokens, threads, 0, s>>>(o, out_row_stride, e, input_ids, hidden_size);
  } else {
    EmbedGatherKernel<half><<<num_tokens, 256, 0, s>>>(o, out_row_stride, e, input_ids, hidden_size);
  }
  return LaunchStatus("embed_gather");
}
