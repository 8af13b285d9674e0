// Greedy argmax over the vocabulary, sm_100a.
//
// Contract and ordering are the reference's (src/kernels/kernels.cuh:195-199,
// src/kernels/argmax.cu:228-252): per row, the int32 index of the largest
// logit; compares in FP32 (an exact, order-preserving widening of the stored
// FP16); a strictly greater value wins and equal values go to the LOWEST index
// (+0 and -0 compare equal); a NaN never displaces an incumbent, an all-NaN row
// yields token 0; an all -inf row yields token 0 through the index tie-break.
// The predicate is a total order over everything the reduction sees, so the
// winner does not depend on the reduction shape.
//
// Mapping. A decode batch is 64 rows x 151 936 logits = 19.4 MB: one CTA per row
// (the reference's shape) would use 64 of 148 SMs. Here every row is scanned by
// a thread-block CLUSTER of 8 CTAs, each taking a contiguous eighth of the row.
// A thread requests its whole share at once - ten 16-byte loads, all in flight
// before the first compare - and keeps it in registers. The maximum is found on
// packed halves (four max instructions per eight logits, no index arithmetic);
// only then is the lowest position of that value looked up, by equality, in the
// registers the data already sits in. CTA champions meet in the leader's shared
// memory through distributed shared memory and the leader writes the token - one
// launch, no scratch in global memory, no atomics.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace rl {
namespace {

constexpr int kClusterCtas = 8;
constexpr int kThreads = 256;
constexpr int kRegChunks = 10;  // 16-byte chunks a thread keeps in registers: 8 x 256 x 10 x 8 = 163 840 logits per row

struct Champion {
  float v;
  int i;
};

// Does candidate (v, i) beat the incumbent? Both arms are IEEE compares: false against NaN.
__device__ __forceinline__ bool Better(float v, int i, const Champion& b) {
  return (v > b.v) || (v == b.v && i < b.i);
}
__device__ __forceinline__ void Offer(Champion& b, float v, int i) {
  if (Better(v, i, b)) {
    b.v = v;
    b.i = i;
  }
}

__device__ __forceinline__ Champion WarpChampion(Champion c) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, c.v, off);
    const int oi = __shfl_xor_sync(0xffffffffu, c.i, off);
    Offer(c, ov, oi);
  }
  return c;
}

// kVec: rows are 16-byte aligned and vocab % 8 == 0.
template <bool kVec>
__global__ void __cluster_dims__(kClusterCtas, 1, 1) __launch_bounds__(kThreads)
ArgmaxClusterKernel(int32_t* __restrict__ out_tokens, const half* __restrict__ logits, int vocab) {
  __shared__ Champion warp_best[kThreads / 32];
  __shared__ Champion cta_best[kClusterCtas];  // used in the cluster leader only
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());
  const int row = blockIdx.x / kClusterCtas;
  const half* x = logits + static_cast<int64_t>(row) * vocab;

  Champion best{-INFINITY, vocab};  // the sentinel index sorts after every real column
  if (kVec) {
    const int chunks = vocab >> 3;
    const int per = (chunks + kClusterCtas - 1) / kClusterCtas;
    const int begin = rank * per, end = min(chunks, (rank + 1) * per);
    __shared__ float warp_max[kThreads / 32];
    __shared__ float cta_max;
    // The largest value, on packed halves. __hmax2 returns the other operand when one is NaN, so NaN never
    // displaces the incumbent; the incumbent starts at -inf.
    const half2 ninf = __float2half2_rn(-INFINITY);
    half2 mx = ninf;
    if (per <= kRegChunks * kThreads) {
      // the whole share of this thread in registers, every load in flight before the first use
      uint4 w[kRegChunks];
#pragma unroll
      for (int k = 0; k < kRegChunks; ++k) {
        const int c = begin + threadIdx.x + k * kThreads;
        w[k] = c < end ? LdgStream16(x + c * 8) : make_uint4(0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u);  // -inf
      }
#pragma unroll
      for (int k = 0; k < kRegChunks; ++k)
        mx = __hmax2(__hmax2(mx, __hmax2(AsHalf2(w[k].x), AsHalf2(w[k].y))), __hmax2(AsHalf2(w[k].z), AsHalf2(w[k].w)));
      float m = fmaxf(__low2float(mx), __high2float(mx));
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
      if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
      __syncthreads();
      if (threadIdx.x == 0) {
        float b = warp_max[0];
#pragma unroll
        for (int i = 1; i < kThreads / 32; ++i) b = fmaxf(b, warp_max[i]);
        cta_max = b;
      }
      __syncthreads();
      // The lowest position holding that value (+0 and -0 compare equal, NaN equals nothing): this thread's
      // chunks ascend in k, a chunk's halves in position.
      const float target = cta_max;
      const half2 t2 = __float2half2_rn(target);
      best.v = target;
#pragma unroll
      for (int k = kRegChunks - 1; k >= 0; --k) {
        const int c = begin + threadIdx.x + k * kThreads;
        const uint32_t words[4] = {w[k].x, w[k].y, w[k].z, w[k].w};
        if (c < end && (__heq2_mask(AsHalf2(words[0]), t2) | __heq2_mask(AsHalf2(words[1]), t2) |
                        __heq2_mask(AsHalf2(words[2]), t2) | __heq2_mask(AsHalf2(words[3]), t2))) {
#pragma unroll
          for (int j = 3; j >= 0; --j) {
            const uint32_t hit = __heq2_mask(AsHalf2(words[j]), t2);
            if (hit & 0xFFFF0000u) best.i = c * 8 + 2 * j + 1;
            if (hit & 0x0000FFFFu) best.i = c * 8 + 2 * j;
          }
        }
      }
      if (best.i >= vocab) best.v = -INFINITY;   // this thread does not hold the CTA's maximum
    } else {
      // rows too long for the register file: the streaming form
      for (int c0 = begin + threadIdx.x; c0 < end; c0 += 4 * kThreads) {
        uint4 w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = c0 + k * kThreads;
          if (c < end) w[k] = LdgStream16(x + c * 8);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = c0 + k * kThreads;
          if (c < end) {
            const uint32_t words[4] = {w[k].x, w[k].y, w[k].z, w[k].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __half22float2(AsHalf2(words[j]));
              Offer(best, f.x, c * 8 + 2 * j);
              Offer(best, f.y, c * 8 + 2 * j + 1);
            }
          }
        }
      }
    }
  } else {
    const int per = (vocab + kClusterCtas - 1) / kClusterCtas;
    const int end = min(vocab, (rank + 1) * per);
    for (int i = rank * per + threadIdx.x; i < end; i += kThreads) Offer(best, __half2float(x[i]), i);
  }
  best = WarpChampion(best);
  if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    Champion b = warp_best[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) Offer(b, warp_best[w].v, warp_best[w].i);
    Champion* leader = cluster.map_shared_rank(cta_best, 0);
    leader[rank] = b;
  }
  cluster.sync();  // every CTA's champion is in the leader's shared memory
  if (rank == 0 && threadIdx.x == 0) {
    Champion b = cta_best[0];
#pragma unroll
    for (int r = 1; r < kClusterCtas; ++r) Offer(b, cta_best[r].v, cta_best[r].i);
    out_tokens[row] = b.i >= vocab ? 0 : b.i;  // nothing adopted (all NaN): token 0
  }
}

}  // namespace
}  // namespace rl

extern "C" int rl_launch_greedy_argmax(int32_t* out_tokens, const void* logits, int32_t num_seqs,
                                       int32_t vocab_size, void* stream) {
  using namespace rl;
  if (num_seqs <= 0 || vocab_size <= 0) return RL_OK;
  if (!out_tokens || !logits) return Fail(RL_E_NULL_POINTER, "greedy_argmax: null device pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const half* x = static_cast<const half*>(logits);
  const dim3 grid(static_cast<unsigned>(num_seqs) * kClusterCtas);
  if (vocab_size % 8 == 0 && Aligned16(logits)) {
    ArgmaxClusterKernel<true><<<grid, kThreads, 0, s>>>(out_tokens, x, vocab_size);
  } else {
    ArgmaxClusterKernel<false><<<grid, kThreads, 0, s>>>(out_tokens, x, vocab_size);
  }
  return LaunchStatus("greedy_argmax");
}
