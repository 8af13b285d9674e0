// The two prefill-side launchers of the kernel contract, sm_100a. They are not on the decode hot
// path (never inside the captured decode graph, src/kernels/kv_gather.cu:43-44); they are provided
// so the drop-in header covers every launcher of src/kernels/kernels.cuh.
//
// LaunchKvGather (src/kernels/kernels.cuh:101-123, src/kernels/kv_gather.cu:136-168): the inverse
// bit move of the scatter for ONE sequence - position t comes from block_table_row[t >> 4], slot
// t & 15 - into dense [kv_heads, ctx_len, head_dim] staging views. One warp per position.
//
// LaunchPrefillSoftmax (src/kernels/kernels.cuh:160-187, src/kernels/prefill_attention.cu:103-162):
// causal row softmax FP32 -> FP16 over [heads, chunk_len, kv_len]; query row i sits at position
// chunk_start + i and sees keys j <= it; FP32 max and sum, one FP16 rounding of exp(s - max) / sum
// (the read-once kernel forms the same quotient from per-thread partial maxima and sums, see there);
// masked entries are written as exact +0 and their scores never reach a result. One CTA per (row, head);
// rows of up to 32768 keys are read once and kept in registers, longer or unaligned ones take three
// passes over the row (it stays in L2); fixed reduction trees either way (run-to-run identical bits).
#include "common.cuh"

#if defined(__USE_FAST_MATH__)
#error "the prefill softmax needs the precise expf"
#endif

namespace rl {
namespace {

// One warp per kTokens consecutive positions. A lane's words sit at the same place inside every page slot
// and every staging row, so those offsets are computed once; per position only the page and the slot
// remain, and the reads of all the warp's positions are requested before any of them is stored.
template <typename Word, int kTokens>
__global__ void __launch_bounds__(128)
KvGatherKernel(half* __restrict__ khat, half* __restrict__ vhat, int64_t khat_head_stride,
               int64_t khat_row_stride, int64_t vhat_head_stride, int64_t vhat_row_stride,
               const half* __restrict__ pool, const int32_t* __restrict__ table_row, int ctx_len,
               int num_kv_heads, int head_dim) {
  constexpr int kPer = sizeof(Word) / sizeof(half);
  constexpr int kAhead = 2;  // words per lane held in registers: all of them for 2 heads x 128 in 16-byte words
  const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kTokens;
  if (t0 >= ctx_len) return;
  const int tokens = static_cast<int>(min(static_cast<int64_t>(kTokens), ctx_len - t0));
  const int lane = threadIdx.x & 31;
  const int words_per_head = head_dim / kPer;
  const int words_per_side = num_kv_heads * words_per_head;
  const int words = 2 * words_per_side;
  const int64_t slot_elems = head_dim;
  const int64_t page_elems = 2 * num_kv_heads * kKvBlock * slot_elems;  // [2][heads][16][head_dim]
  auto src_of = [&](int w) {  // inside (page, slot 0)
    const int side_head = w / words_per_head;  // kv * heads + h
    return side_head * kKvBlock * slot_elems + (w - side_head * words_per_head) * kPer;
  };
  auto dst_of = [&](int w, int64_t t) {
    const int kv = w >= words_per_side;
    const int r = w - kv * words_per_side;
    const int h = r / words_per_head;
    half* row = kv ? vhat + h * vhat_head_stride + t * vhat_row_stride
                   : khat + h * khat_head_stride + t * khat_row_stride;
    return reinterpret_cast<Word*>(row) + (r - h * words_per_head);
  };
  const half* cell[kTokens];
#pragma unroll
  for (int i = 0; i < kTokens; ++i) {
    const int64_t t = t0 + (i < tokens ? i : 0);
    cell[i] = pool + table_row[t >> kKvBlockShift] * page_elems + (t & (kKvBlock - 1)) * slot_elems;
  }
  Word held[kTokens][kAhead];
#pragma unroll
  for (int j = 0; j < kAhead; ++j) {
    const int w = lane + 32 * j;
    if (w < words) {
      const int64_t off = src_of(w);
#pragma unroll
      for (int i = 0; i < kTokens; ++i) {
        if (i < tokens) held[i][j] = *reinterpret_cast<const Word*>(cell[i] + off);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kTokens; ++i) {
    if (i >= tokens) break;
#pragma unroll
    for (int j = 0; j < kAhead; ++j) {
      if (lane + 32 * j < words) *dst_of(lane + 32 * j, t0 + i) = held[i][j];
    }
    for (int w = lane + 32 * kAhead; w < words; w += 32) {
      *dst_of(w, t0 + i) = *reinterpret_cast<const Word*>(cell[i] + src_of(w));
    }
  }
}

constexpr int kSoftmaxThreads = 256;

// Max or sum over the block, the same value in every thread: lane trees inside the warps, then the same
// tree over the warps' results (a fixed order: run-to-run identical bits).
template <int kThreads>
__device__ __forceinline__ float BlockReduce(float v, bool is_max, float* scratch) {
  static_assert(kThreads % 32 == 0 && kThreads <= 1024, "one scratch word per warp, at most 32 warps");
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, v, off);
    v = is_max ? fmaxf(v, o) : v + o;
  }
  const int lane = threadIdx.x & 31;
  if (lane == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = lane < kThreads / 32 ? scratch[lane] : (is_max ? -INFINITY : 0.0f);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, r, off);
    r = is_max ? fmaxf(r, o) : r + o;
  }
  __syncthreads();  // scratch is reused by the next reduction
  return r;
}

// A (max, sum of exp(x - max)) pair over part of a row.
struct MaxSum {
  float m, s;
};

// Rows of up to kThreads * kChunks * 8 scores with kv_len a multiple of 8 and 16-byte aligned bases: the
// live part of the row is read once, 8 consecutive scores per thread and step, and stays in registers.
// Each thread takes the max of its own scores and their exponentials against that max at once, with no
// block-wide step in between; fixed trees then merge the threads' (max, sum) pairs, and a thread's
// results are its exponentials times exp(own max - row max) / row sum: one exponential and one multiply
// per element, FP32 throughout, one rounding to FP16. Elements of a 32-byte group that lie beyond the
// causal limit are loaded with the group but replaced by -inf before any use, so their exponential is
// exactly 0 and so is their probability.
template <int kThreads, int kChunks>
__global__ void __launch_bounds__(kThreads)
PrefillSoftmaxRowKernel(half* __restrict__ probs, const float* __restrict__ scores, int chunk_len, int kv_len,
                        int chunk_start) {
  static_assert(kThreads % 32 == 0 && kThreads <= 1024, "one scratch pair per warp, at most 32 warps");
  __shared__ MaxSum scratch[kThreads / 32];
  const int row = blockIdx.x, head = blockIdx.y;
  const size_t base = (static_cast<size_t>(head) * chunk_len + row) * static_cast<size_t>(kv_len);
  const float* s = scores + base;
  half* p = probs + base;
  const int live = min(chunk_start + row + 1, kv_len);
  float x[kChunks][8];
  MaxSum mine = {-INFINITY, 0.0f};
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int j0 = (c * kThreads + threadIdx.x) << 3;
    if (j0 < live) {
      const uint4 a = LdgStream16(s + j0), b = LdgStream16(s + j0 + 4);
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      if (j0 + 8 <= live) {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[c][e] = __uint_as_float(w[e]);
      } else {  // the one group of the row that straddles the causal limit
#pragma unroll
        for (int e = 0; e < 8; ++e) x[c][e] = j0 + e < live ? __uint_as_float(w[e]) : -INFINITY;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) mine.m = fmaxf(mine.m, x[c][e]);
    }
  }
  // scores of -inf (a caller's own masking) must give 0, not exp(-inf + inf), when they are all a thread has
  const float local_max = mine.m == -INFINITY ? 0.0f : mine.m;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int j0 = (c * kThreads + threadIdx.x) << 3;
    if (j0 < live) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        x[c][e] = expf(x[c][e] - local_max);
        mine.s += x[c][e];
      }
    }
  }
  // (max, sum) over the row: the max by a lane tree, each lane's sum rescaled to it once, the sums by the same
  // tree; then the same again over the warps' pairs (every warp redundantly). Fixed order: same bits every run.
  float warp_max = mine.m;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) warp_max = fmaxf(warp_max, __shfl_xor_sync(0xffffffffu, warp_max, off));
  float warp_sum = mine.m == -INFINITY ? 0.0f : mine.s * expf(mine.m - warp_max);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) warp_sum += __shfl_xor_sync(0xffffffffu, warp_sum, off);
  const int lane = threadIdx.x & 31;
  if (lane == 0) scratch[threadIdx.x >> 5] = MaxSum{warp_max, warp_sum};
  __syncthreads();
  const MaxSum theirs = lane < kThreads / 32 ? scratch[lane] : MaxSum{-INFINITY, 0.0f};
  float row_max = theirs.m;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, off));
  float row_sum = theirs.m == -INFINITY ? 0.0f : theirs.s * expf(theirs.m - row_max);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) row_sum += __shfl_xor_sync(0xffffffffu, row_sum, off);
  // exp(own max - row max) / row sum; a thread without live scores stores only zeros
  const float factor = mine.m == -INFINITY ? 0.0f : expf(mine.m - row_max) / row_sum;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int j0 = (c * kThreads + threadIdx.x) << 3;
    if (j0 >= kv_len) continue;
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (j0 < live) {
      uint32_t* o = &out.x;
#pragma unroll
      for (int e = 0; e < 4; ++e) {  // replaced elements hold 0 and give exact +0
        o[e] = AsU32(__floats2half2_rn(x[c][2 * e] * factor, x[c][2 * e + 1] * factor));
      }
    }
    Stg16(p + j0, out);
  }
}

__global__ void __launch_bounds__(kSoftmaxThreads)
PrefillSoftmaxKernel(half* __restrict__ probs, const float* __restrict__ scores, int chunk_len, int kv_len,
                     int chunk_start) {
  __shared__ float scratch[kSoftmaxThreads / 32];
  const int row = blockIdx.x, head = blockIdx.y;
  const size_t base = (static_cast<size_t>(head) * chunk_len + row) * static_cast<size_t>(kv_len);
  const float* s = scores + base;
  half* p = probs + base;
  const int live = min(chunk_start + row + 1, kv_len);
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < live; j += kSoftmaxThreads) mx = fmaxf(mx, s[j]);
  mx = BlockReduce<kSoftmaxThreads>(mx, true, scratch);
  float sum = 0.0f;
  for (int j = threadIdx.x; j < live; j += kSoftmaxThreads) sum += expf(s[j] - mx);
  sum = BlockReduce<kSoftmaxThreads>(sum, false, scratch);
  for (int j = threadIdx.x; j < kv_len; j += kSoftmaxThreads)
    p[j] = j < live ? __float2half_rn(expf(s[j] - mx) / sum) : __ushort_as_half(0);
}

}  // namespace
}  // namespace rl

extern "C" int rl_launch_kv_gather(void* khat, void* vhat, int64_t khat_head_stride, int64_t khat_row_stride,
                                   int64_t vhat_head_stride, int64_t vhat_row_stride, const void* kv_pool_layer,
                                   const int32_t* block_table_row, int32_t ctx_len, int32_t num_kv_heads,
                                   int32_t head_dim, void* stream) {
  using namespace rl;
  if (ctx_len <= 0 || num_kv_heads <= 0 || head_dim <= 0) return RL_OK;
  if (!khat || !vhat || !kv_pool_layer || !block_table_row)
    return Fail(RL_E_NULL_POINTER, "kv_gather: null device pointer");
  half* k = static_cast<half*>(khat);
  half* v = static_cast<half*>(vhat);
  const half* pool = static_cast<const half*>(kv_pool_layer);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool vec = head_dim % 8 == 0 && khat_head_stride % 8 == 0 && khat_row_stride % 8 == 0 &&
                   vhat_head_stride % 8 == 0 && vhat_row_stride % 8 == 0 && Aligned16(khat) && Aligned16(vhat) &&
                   Aligned16(kv_pool_layer);
  // two positions per warp once that still fills the device several times over
  const int tpw = ctx_len >= 64 * CurrentDeviceFacts().sm_count ? 2 : 1;
  const dim3 grid((ctx_len + 4 * tpw - 1) / (4 * tpw)), block(128);
  auto launch = [&](auto kernel) {
    kernel<<<grid, block, 0, s>>>(k, v, khat_head_stride, khat_row_stride, vhat_head_stride, vhat_row_stride, pool,
                                  block_table_row, ctx_len, num_kv_heads, head_dim);
  };
  if (vec && tpw == 2) launch(KvGatherKernel<uint4, 2>);
  else if (vec) launch(KvGatherKernel<uint4, 1>);
  else if (tpw == 2) launch(KvGatherKernel<half, 2>);
  else launch(KvGatherKernel<half, 1>);
  return LaunchStatus("kv_gather");
}

extern "C" int rl_launch_prefill_softmax(void* probs, const float* scores, int32_t num_q_heads, int32_t chunk_len,
                                         int32_t kv_len, int32_t chunk_start, void* stream) {
  using namespace rl;
  if (num_q_heads <= 0 || chunk_len <= 0 || kv_len <= 0) return RL_OK;
  if (!probs || !scores) return Fail(RL_E_NULL_POINTER, "prefill_softmax: null device pointer");
  if (chunk_start < 0) return Fail(RL_E_BAD_SHAPE, "prefill_softmax: negative chunk_start");
  if (num_q_heads > 65535) return Fail(RL_E_TOO_LARGE, "prefill_softmax: more than 65535 heads");
  const dim3 grid(chunk_len, num_q_heads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  half* out = static_cast<half*>(probs);
  const bool vec = kv_len % 8 == 0 && Aligned16(probs) && Aligned16(scores);
  if (vec && kv_len <= 256 * 1 * 8) {
    PrefillSoftmaxRowKernel<256, 1><<<grid, 256, 0, s>>>(out, scores, chunk_len, kv_len, chunk_start);
  } else if (vec && kv_len <= 512 * 1 * 8) {
    PrefillSoftmaxRowKernel<512, 1><<<grid, 512, 0, s>>>(out, scores, chunk_len, kv_len, chunk_start);
  } else if (vec && kv_len <= 512 * 2 * 8) {  // 61.0 us at 12 x 512 x 8192 against 67.5 (256 x 4) and 82.2 (128 x 8)
    PrefillSoftmaxRowKernel<512, 2><<<grid, 512, 0, s>>>(out, scores, chunk_len, kv_len, chunk_start);
  } else if (vec && kv_len <= 1024 * 2 * 8) {
    PrefillSoftmaxRowKernel<1024, 2><<<grid, 1024, 0, s>>>(out, scores, chunk_len, kv_len, chunk_start);
  } else if (vec && kv_len <= 1024 * 4 * 8) {
    PrefillSoftmaxRowKernel<1024, 4><<<grid, 1024, 0, s>>>(out, scores, chunk_len, kv_len, chunk_start);
  } else {  // odd lengths, unaligned bases, rows beyond 32768 keys: three passes over the row
    PrefillSoftmaxKernel<<<grid, kSoftmaxThreads, 0, s>>>(out, scores, chunk_len, kv_len, chunk_start);
  }
  return LaunchStatus("prefill_softmax");
}
