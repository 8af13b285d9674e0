// RMSNorm and fused residual-add + RMSNorm for sm_100a.
//
// Contract and rounding points follow the reference launchers
// (src/kernels/rmsnorm.cu:436-470 and the kernels at :159-254):
//   h   = fp16(residual + input)          rounding point 1 (a native half add)
//   residual <- h
//   ms  = mean(f32(h)^2), FP32             over the ROUNDED h
//   out = fp16( fp16(f32(h) * rsqrtf(ms + eps)) * weight )   rounding point 2 before the weight
//
// Mapping. Rows are cut into 16-byte chunks (8 halves). One CTA per row, one chunk per
// thread (thread = 32*i + lane): the row is read once and written once, the dependent
// instruction chain per thread is 8 elements long, and a decode batch of 64 rows still
// runs on 6 x 64 warps. The same shape is also the fastest at HBM-bound sizes (many
// small CTAs keep more loads in flight per SM than a warp per row with the row in
// registers: 32.0 against 34.0 us at 16384 x 1536, 5.6 against 8.0 us at 2048 x 1536).
// Summation order: per chunk left to right from zero, a lane-xor tree over the 32 chunks
// of each group i, then the groups in ascending i - a row gives the same bits whatever
// the batch size. A scalar block-per-row kernel covers odd widths and 2-byte-aligned bases.
#include "common.cuh"
#include "rmsnorm_math.cuh"

namespace rl {
namespace {

// One CTA of 32*CPL threads per row, one chunk per thread (thread = 32*i + lane).
template <int CPL, bool kResidual>
__global__ void __launch_bounds__(32 * CPL)
RmsNormBlockKernel(half* __restrict__ out, half* __restrict__ residual, const half* __restrict__ input,
                   const half* __restrict__ weight, int hidden, float eps) {
  __shared__ float group_sum[CPL];
  DependentLaunchGate();
  const int c = threadIdx.x;
  const int chunks = hidden >> 3;
  const size_t base = static_cast<size_t>(blockIdx.x) * hidden;
  const bool live = c < chunks;
  uint4 h = make_uint4(0, 0, 0, 0), w = h;
  float part = 0.0f;
  if (live) {
    h = LdgStream16(input + base + c * 8);
    w = Ldg16(weight + c * 8);
    if (kResidual) {
      h = AddChunk(Ldg16(residual + base + c * 8), h);
      Stg16(residual + base + c * 8, h);
    }
    part = ChunkSumSq(h);
  }
  part = WarpTreeSum(part);
  if ((c & 31) == 0) group_sum[c >> 5] = part;
  __syncthreads();
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < CPL; ++i) ss += group_sum[i];
  const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
  if (live) Stg16(out + base + c * 8, NormChunk(h, w, inv));
}

// Any width, any 2-byte alignment: one block per row, two passes over global
// memory (the second re-reads what the same thread wrote).
template <bool kResidual>
__global__ void __launch_bounds__(256)
RmsNormScalarKernel(half* out, half* residual, const half* input, const half* weight, int hidden,
                    float eps) {
  __shared__ float warp_sums[8];
  __shared__ float total_s;
  const size_t base = static_cast<size_t>(blockIdx.x) * hidden;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    half h = input[base + c];
    if (kResidual) {
      h = __hadd_rn(residual[base + c], h);
      residual[base + c] = h;
    }
    const float f = __half2float(h);
    ss = fmaf(f, f, ss);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) t += warp_sums[w];
    total_s = t;
  }
  __syncthreads();
  const float inv = rsqrtf(total_s / static_cast<float>(hidden) + eps);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const half h = kResidual ? residual[base + c] : input[base + c];
    const half normed = __float2half_rn(__half2float(h) * inv);
    out[base + c] = __hmul_rn(normed, weight[c]);
  }
}

template <bool kResidual>
int Launch(half* out, half* residual, const half* input, const half* weight, int num_tokens,
           int hidden, float eps, cudaStream_t stream) {
  if (num_tokens <= 0 || hidden <= 0) return RL_OK;
  if (!out || !input || !weight || (kResidual && !residual))
    return Fail(RL_E_NULL_POINTER, "rmsnorm: null device pointer");
  const bool vec = (hidden % 8 == 0) && (hidden / 8 <= 32 * kMaxChunksPerLane) && Aligned16(out) &&
                   Aligned16(input) && Aligned16(weight) && (!kResidual || Aligned16(residual));
  if (!vec) {
    RmsNormScalarKernel<kResidual><<<num_tokens, 256, 0, stream>>>(out, residual, input, weight,
                                                                   hidden, eps);
    return LaunchStatus("rmsnorm (scalar)");
  }
  const int cpl = (hidden / 8 + 31) / 32;
#define RL_NORM_CASE(N)                                                                           \
  case N:                                                                                         \
    LaunchOverlapped(RmsNormBlockKernel<N, kResidual>, dim3(num_tokens), dim3(32 * N), 0, stream, \
                     out, residual, input, weight, hidden, eps);                                  \
    break;
  switch (cpl) {
    RL_NORM_CASE(1) RL_NORM_CASE(2) RL_NORM_CASE(3) RL_NORM_CASE(4) RL_NORM_CASE(5)
    RL_NORM_CASE(6) RL_NORM_CASE(7) RL_NORM_CASE(8)
  }
#undef RL_NORM_CASE
  return LaunchStatus("rmsnorm");
}

}  // namespace
}  // namespace rl

extern "C" int rl_launch_rmsnorm(void* out, const void* input, const void* weight,
                                 int32_t num_tokens, int32_t hidden_size, float eps, void* stream) {
  return rl::Launch<false>(static_cast<half*>(out), nullptr, static_cast<const half*>(input),
                           static_cast<const half*>(weight), num_tokens, hidden_size, eps,
                           static_cast<cudaStream_t>(stream));
}

extern "C" int rl_launch_rmsnorm_residual(void* out, void* residual, const void* input,
                                          const void* weight, int32_t num_tokens,
                                          int32_t hidden_size, float eps, void* stream) {
  return rl::Launch<true>(static_cast<half*>(out), static_cast<half*>(residual),
                          static_cast<const half*>(input), static_cast<const half*>(weight),
                          num_tokens, hidden_size, eps, static_cast<cudaStream_t>(stream));
}
