// Arithmetic of RMSNorm / fused residual-add + RMSNorm on 16-byte chunks (8 halves), shared by the norm kernels and
// by the linear layer's add+norm epilogue so that both give the same bits: rounding points of
// src/kernels/rmsnorm.cu:125-148,204-254 (native half add; mean of squares of the ROUNDED sum in FP32;
// fp16(h * inv) before the weight product), and one summation order (per chunk left to right from zero, a
// lane-xor tree over the 32 chunks of a group, groups in ascending order).
#pragma once

#include "common.cuh"

#if defined(__USE_FAST_MATH__)
#error "the norm's rounding contract needs the precise math path"
#endif

namespace rl {

constexpr int kMaxChunksPerLane = 8;  // 8 chunks x 8 halves x 32 lanes = 2048 columns

// Sum of squares of one chunk, left to right from zero (the shared summation order).
__device__ __forceinline__ float ChunkSumSq(const uint4& x) {
  const uint32_t words[4] = {x.x, x.y, x.z, x.w};
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(AsHalf2(words[j]));
    ss = fmaf(f.x, f.x, ss);
    ss = fmaf(f.y, f.y, ss);
  }
  return ss;
}

__device__ __forceinline__ float WarpTreeSum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

__device__ __forceinline__ uint4 AddChunk(const uint4& r, const uint4& x) {
  return make_uint4(AsU32(__hadd2_rn(AsHalf2(r.x), AsHalf2(x.x))), AsU32(__hadd2_rn(AsHalf2(r.y), AsHalf2(x.y))),
                    AsU32(__hadd2_rn(AsHalf2(r.z), AsHalf2(x.z))), AsU32(__hadd2_rn(AsHalf2(r.w), AsHalf2(x.w))));
}

// out chunk = fp16(fp16(h * inv) * w); fp16 x fp16 is exact in FP32, so one half multiply equals
// fp16(f32(n) * f32(w)).
__device__ __forceinline__ uint4 NormChunk(const uint4& h, const uint4& w, float inv) {
  const uint32_t hw[4] = {h.x, h.y, h.z, h.w};
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(AsHalf2(hw[j]));
    o[j] = AsU32(__hmul2_rn(__floats2half2_rn(f.x * inv, f.y * inv), AsHalf2(ww[j])));
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace rl
