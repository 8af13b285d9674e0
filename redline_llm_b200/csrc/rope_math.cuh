// Rotary-embedding arithmetic shared by the RoPE kernels and by the linear layer's QKV epilogue, so that
// every path gives the same bits: NeoX half-rotation, FP16 cos/sin, each product and each sum rounded to
// FP16 (src/kernels/rope.cu:181-210), angles float(pos) * inv_freq[d] with the FP32 table computed on the
// host (src/kernels/rope.cu:150-176).
#pragma once

#include "common.cuh"

#if defined(__USE_FAST_MATH__)
#error "rope needs the precise sincosf"
#endif

namespace rl {

constexpr int kMaxPairs = 64;

struct InvFreq {
  float f[kMaxPairs];
};

// Host-side memo of the last table (pure host state; safe with any number of devices). Defined in rope.cu.
const InvFreq& RopeTableFor(float theta, int head_dim);

// Two rotation pairs at once: lo holds elements (d, d+1), hi holds (d + head_dim/2, d+1 + head_dim/2).
__device__ __forceinline__ void RotateWord(uint32_t& lo, uint32_t& hi, half2 c, half2 s) {
  const half2 x1 = AsHalf2(lo), x2 = AsHalf2(hi);
  const half2 a = __hsub2_rn(__hmul2_rn(x1, c), __hmul2_rn(x2, s));  // == x1*c + (-x2)*s, bit for bit
  const half2 b = __hadd2_rn(__hmul2_rn(x2, c), __hmul2_rn(x1, s));
  lo = AsU32(a);
  hi = AsU32(b);
}

// {cos, sin} of one rotation pair, already FP16 (the first rounding point).
__device__ __forceinline__ half2 RopeCosSin(float pos, float inv_freq) {
  float s32, c32;
  sincosf(pos * inv_freq, &s32, &c32);
  return __floats2half2_rn(c32, s32);
}

}  // namespace rl
