// Rotary position embedding applied in place to the Q and K views, sm_100a.
//
// NeoX half-rotation (element d pairs with d + head_dim/2), theta from the
// caller, the three FP16 rounding points of src/kernels/rope.cu:181-210,
// 231-257: cos/sin rounded to FP16; each of the four products rounded to FP16;
// each of the two sums rounded to FP16. Angles are one FP32 multiply
// float(pos) * inv_freq[d] with inv_freq[d] = 1.0f / powf(theta, 2d/head_dim)
// computed on the host in FP32 (src/kernels/rope.cu:150-176) and sincosf on the
// precise path, so results are bit-identical to the reference kernel and to the
// HF capture it is pinned to.
//
// The inverse-frequency table rides in the kernel's parameter space: there is
// no per-device constant table to upload, nothing to go stale with several GPUs
// in one process, and no CUDA call besides the launch on any call.
//
// Mapping: one block per token row. Threads d < head_dim/2 evaluate sincosf once
// for the row into shared memory; then each thread rotates one 8-element chunk
// of the low half against the matching chunk of the high half of one head with
// 16-byte loads and half2 arithmetic (fp16 x fp16 and fp16 + fp16 are each one
// correctly rounded half operation, equal to the FP32-then-round form; the _rn
// intrinsics forbid fusing them into an fma).
#include <cmath>
#include <mutex>

#include "rope_math.cuh"

namespace rl {

const InvFreq& RopeTableFor(float theta, int head_dim) {
  static std::mutex mu;
  static InvFreq table;
  static float cached_theta = 0.0f;
  static int cached_dim = 0;
  thread_local InvFreq local;
  std::lock_guard<std::mutex> lock(mu);
  if (cached_theta != theta || cached_dim != head_dim) {
    for (int d = 0; d < head_dim / 2; ++d) {
      const float exponent = static_cast<float>(2 * d) / static_cast<float>(head_dim);
      table.f[d] = 1.0f / std::pow(theta, exponent);
    }
    cached_theta = theta;
    cached_dim = head_dim;
  }
  local = table;
  return local;
}

namespace {

__device__ __forceinline__ half* HeadPtr(half* q, half* k, int64_t qs, int64_t ks, int row, int head,
                                         int num_q_heads, int head_dim) {
  return head < num_q_heads ? q + row * qs + head * head_dim
                            : k + row * ks + (head - num_q_heads) * head_dim;
}

// head_dim/2 a multiple of 8 and every head row 16-byte aligned.
__global__ void __launch_bounds__(128)
RopeVecKernel(half* q, half* k, int64_t q_row_stride, int64_t k_row_stride,
              const int32_t* __restrict__ positions, int num_q_heads, int total_heads, int head_dim,
              const __grid_constant__ InvFreq inv_freq) {
  __shared__ __align__(16) half2 cs[kMaxPairs];  // {cos, sin} per pair, already FP16
  const int row = blockIdx.x;
  const int half_dim = head_dim >> 1;
  const float pos = static_cast<float>(positions[row]);
  for (int d = threadIdx.x; d < half_dim; d += blockDim.x) {
    cs[d] = RopeCosSin(pos, inv_freq.f[d]);
  }
  __syncthreads();
  const int chunks = half_dim >> 3;
  for (int item = threadIdx.x; item < total_heads * chunks; item += blockDim.x) {
    const int head = item / chunks;
    const int d0 = (item - head * chunks) << 3;
    half* base = HeadPtr(q, k, q_row_stride, k_row_stride, row, head, num_q_heads, head_dim);
    uint4 lo = Ldg16(base + d0);
    uint4 hi = Ldg16(base + d0 + half_dim);
    uint32_t* l = &lo.x;
    uint32_t* h = &hi.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const half2 a = cs[d0 + 2 * j], b = cs[d0 + 2 * j + 1];
      RotateWord(l[j], h[j], __lows2half2(a, b), __highs2half2(a, b));
    }
    Stg16(base + d0, lo);
    Stg16(base + d0 + half_dim, hi);
  }
}

// Any even head_dim <= 128 and any 2-byte alignment: one thread per rotation pair.
__global__ void __launch_bounds__(128)
RopeScalarKernel(half* q, half* k, int64_t q_row_stride, int64_t k_row_stride,
                 const int32_t* __restrict__ positions, int num_q_heads, int total_heads,
                 int head_dim, const __grid_constant__ InvFreq inv_freq) {
  const int row = blockIdx.x;
  const int half_dim = head_dim >> 1;
  const float pos = static_cast<float>(positions[row]);
  for (int item = threadIdx.x; item < total_heads * half_dim; item += blockDim.x) {
    const int head = item / half_dim;
    const int d = item - head * half_dim;
    float s32, c32;
    sincosf(pos * inv_freq.f[d], &s32, &c32);
    const half c = __float2half_rn(c32), s = __float2half_rn(s32);
    half* base = HeadPtr(q, k, q_row_stride, k_row_stride, row, head, num_q_heads, head_dim);
    const half x1 = base[d], x2 = base[d + half_dim];
    base[d] = __hadd_rn(__hmul_rn(x1, c), __hmul_rn(__hneg(x2), s));
    base[d + half_dim] = __hadd_rn(__hmul_rn(x2, c), __hmul_rn(x1, s));
  }
}

// RoPE and KV scatter in one pass (decode shape: head_dim 128, 16-byte aligned views). One CTA per
// token: rotate Q and K in place exactly as RopeVecKernel does, and while the rotated K chunk is in
// registers also store it to its page slot; V chunks are copied to theirs. The qkv buffer ends up
// bit-identical to the two-launch sequence, and so does the pool.
__global__ void __launch_bounds__(128)
RopeScatterKernel(half* q, half* k, const half* __restrict__ v, int64_t q_row_stride, int64_t k_row_stride,
                  int64_t v_row_stride, half* __restrict__ pool, const int32_t* __restrict__ tables,
                  int64_t table_row_stride, const int32_t* __restrict__ positions, int num_q_heads,
                  int num_kv_heads, int head_dim, const __grid_constant__ InvFreq inv_freq) {
  __shared__ __align__(16) half2 cs[kMaxPairs];
  // the attention launch that follows may begin its table walk now (it waits for this grid to
  // complete before it reads the pool or Q); this grid itself waits for the QKV GEMM before it
  DependentLaunchGate();
  const int64_t row = blockIdx.x;
  const int half_dim = head_dim >> 1;
  const int p = positions[row];
  const int64_t block = tables[row * table_row_stride + (p >> kKvBlockShift)];
  const int slot = p & (kKvBlock - 1);
  const float pos = static_cast<float>(p);
  for (int d = threadIdx.x; d < half_dim; d += blockDim.x) {
    cs[d] = RopeCosSin(pos, inv_freq.f[d]);
  }
  __syncthreads();
  const int chunks = half_dim >> 3;
  const int total_heads = num_q_heads + num_kv_heads;
  const int rope_items = total_heads * chunks;
  const int v_items = num_kv_heads * (head_dim >> 3);
  for (int item = threadIdx.x; item < rope_items + v_items; item += blockDim.x) {
    if (item < rope_items) {
      const int head = item / chunks;
      const int d0 = (item - head * chunks) << 3;
      half* base = HeadPtr(q, k, q_row_stride, k_row_stride, static_cast<int>(row), head, num_q_heads, head_dim);
      uint4 lo = Ldg16(base + d0);
      uint4 hi = Ldg16(base + d0 + half_dim);
      uint32_t* l = &lo.x;
      uint32_t* h = &hi.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const half2 a = cs[d0 + 2 * j], b = cs[d0 + 2 * j + 1];
        RotateWord(l[j], h[j], __lows2half2(a, b), __highs2half2(a, b));
      }
      Stg16(base + d0, lo);
      Stg16(base + d0 + half_dim, hi);
      if (head >= num_q_heads) {
        half* dst = pool + (((block * 2 + 0) * num_kv_heads + (head - num_q_heads)) * kKvBlock + slot) *
                               static_cast<int64_t>(head_dim);
        Stg16(dst + d0, lo);
        Stg16(dst + d0 + half_dim, hi);
      }
    } else {
      const int w = item - rope_items;
      const int head = w / (head_dim >> 3);
      const int d0 = (w - head * (head_dim >> 3)) << 3;
      half* dst = pool + (((block * 2 + 1) * num_kv_heads + head) * kKvBlock + slot) * static_cast<int64_t>(head_dim);
      Stg16(dst + d0, Ldg16(v + row * v_row_stride + head * head_dim + d0));
    }
  }
}

}  // namespace
}  // namespace rl

extern "C" int rl_launch_rope_inplace(void* q, void* k, int64_t q_row_stride, int64_t k_row_stride,
                                      const int32_t* positions, int32_t num_tokens,
                                      int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                      float rope_theta, void* stream) {
  using namespace rl;
  const int total_heads = num_q_heads + num_kv_heads;
  if (num_tokens <= 0 || total_heads <= 0) return RL_OK;
  if (num_q_heads < 0 || num_kv_heads < 0 || head_dim <= 0 || head_dim % 2 != 0 ||
      head_dim / 2 > kMaxPairs || !(rope_theta > 0.0f))
    return Fail(RL_E_BAD_SHAPE, "rope: head_dim must be even and <= 128, theta > 0");
  if ((num_q_heads > 0 && !q) || (num_kv_heads > 0 && !k) || !positions)
    return Fail(RL_E_NULL_POINTER, "rope: null device pointer");
  const InvFreq& table = RopeTableFor(rope_theta, head_dim);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  half* qq = static_cast<half*>(q);
  half* kk = static_cast<half*>(k);
  const bool vec = (head_dim / 2) % 8 == 0 && q_row_stride % 8 == 0 && k_row_stride % 8 == 0 &&
                   Aligned16(q) && Aligned16(k);
  if (vec) {
    RopeVecKernel<<<num_tokens, 128, 0, s>>>(qq, kk, q_row_stride, k_row_stride, positions,
                                             num_q_heads, total_heads, head_dim, table);
  } else {
    RopeScalarKernel<<<num_tokens, 128, 0, s>>>(qq, kk, q_row_stride, k_row_stride, positions,
                                                num_q_heads, total_heads, head_dim, table);
  }
  return LaunchStatus("rope");
}

extern "C" int rl_launch_rope_kv_scatter(void* q, void* k, const void* v, int64_t q_row_stride,
                                         int64_t k_row_stride, int64_t v_row_stride, void* kv_pool_layer,
                                         const int32_t* block_tables, int64_t block_table_row_stride,
                                         const int32_t* positions, int32_t num_tokens, int32_t num_q_heads,
                                         int32_t num_kv_heads, int32_t head_dim, float rope_theta, void* stream) {
  using namespace rl;
  if (num_tokens <= 0 || num_q_heads + num_kv_heads <= 0) return RL_OK;
  if (!q || !k || !v || !kv_pool_layer || !block_tables || !positions)
    return Fail(RL_E_NULL_POINTER, "rope_kv_scatter: null device pointer");
  const bool vec = head_dim > 0 && head_dim % 16 == 0 && head_dim / 2 <= kMaxPairs && q_row_stride % 8 == 0 &&
                   k_row_stride % 8 == 0 && v_row_stride % 8 == 0 && Aligned16(q) && Aligned16(k) && Aligned16(v) &&
                   Aligned16(kv_pool_layer) && num_q_heads >= 0 && num_kv_heads > 0 && rope_theta > 0.0f;
  if (!vec) {  // odd shapes: the two separate launchers cover everything the contract admits
    const int rc = rl_launch_rope_inplace(q, k, q_row_stride, k_row_stride, positions, num_tokens, num_q_heads,
                                          num_kv_heads, head_dim, rope_theta, stream);
    if (rc != RL_OK) return rc;
    return rl_launch_kv_scatter(kv_pool_layer, k, v, k_row_stride, v_row_stride, block_tables,
                                block_table_row_stride, positions, num_tokens, num_kv_heads, head_dim, stream);
  }
  const InvFreq& table = RopeTableFor(rope_theta, head_dim);
  LaunchOverlapped(RopeScatterKernel, dim3(num_tokens), dim3(128), 0, static_cast<cudaStream_t>(stream),
                   static_cast<half*>(q), static_cast<half*>(k), static_cast<const half*>(v), q_row_stride,
                   k_row_stride, v_row_stride, static_cast<half*>(kv_pool_layer), block_tables,
                   block_table_row_stride, positions, num_q_heads, num_kv_heads, head_dim, table);
  return LaunchStatus("rope_kv_scatter");
}
