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
// Mapping: one block per token row (two per block for prompt-sized batches), a
// thread row per head. Each thread requests one 8-element chunk of the low half
// of its head and the matching chunk of the high half with 16-byte loads;
// meanwhile the block evaluates sincosf once per (row, pair) into shared
// memory; then the chunks are rotated with half2 arithmetic (fp16 x fp16 and
// fp16 +- fp16 are each one correctly rounded half operation, equal to the
// FP32-then-round form; the _rn intrinsics forbid fusing them into an fma).
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

// Rotates eight pairs held as two 16-byte words against their eight cos and eight sin values, each a
// 16-byte aligned run of FP16 in shared memory.
__device__ __forceinline__ void RotateChunk(uint4& lo, uint4& hi, const half* cosv, const half* sinv) {
  const uint4 c = *reinterpret_cast<const uint4*>(cosv);
  const uint4 s = *reinterpret_cast<const uint4*>(sinv);
  RotateWord(lo.x, hi.x, AsHalf2(c.x), AsHalf2(s.x));
  RotateWord(lo.y, hi.y, AsHalf2(c.y), AsHalf2(s.y));
  RotateWord(lo.z, hi.z, AsHalf2(c.z), AsHalf2(s.z));
  RotateWord(lo.w, hi.w, AsHalf2(c.w), AsHalf2(s.w));
}

constexpr int kRopeThreads = 128;  // upper bound: blocks are (head_dim/16) x (128 / (head_dim/16)) threads

// The cos and sin of `rows` token rows into shared memory, FP16, one sincosf per (row, pair).
template <int kRows>
__device__ __forceinline__ void FillCosSin(half (&cosv)[kRows][kMaxPairs], half (&sinv)[kRows][kMaxPairs],
                                           const int32_t* __restrict__ positions, int row0, int rows,
                                           int half_dim, int tid, int nthreads, const InvFreq& inv_freq) {
  for (int i = tid; i < rows * half_dim; i += nthreads) {
    const int r = i / half_dim;
    const int d = i - r * half_dim;
    const half2 cs = RopeCosSin(static_cast<float>(positions[row0 + r]), inv_freq.f[d]);
    cosv[r][d] = __low2half(cs);
    sinv[r][d] = __high2half(cs);
  }
}

// head_dim/2 a multiple of 8 and every head row 16-byte aligned. Thread (x, y) of a block works on the
// x-th 8-element chunk of the low half of head y (heads y, y + blockDim.y, ...) and on its partner chunk
// in the high half, for each of the block's kRows consecutive token rows: no index arithmetic beyond adds.
// Each thread first requests the data of its first head in every row, which does not depend on the
// positions, and only then takes part in evaluating the rows' cos/sin tables, so the two latencies overlap.
template <int kRows>
__global__ void __launch_bounds__(kRopeThreads)
RopeVecKernel(half* q, half* k, int64_t q_row_stride, int64_t k_row_stride,
              const int32_t* __restrict__ positions, int num_tokens, int num_q_heads, int total_heads,
              int head_dim, const __grid_constant__ InvFreq inv_freq) {
  __shared__ __align__(16) half cosv[kRows][kMaxPairs];
  __shared__ __align__(16) half sinv[kRows][kMaxPairs];
  const int ty = threadIdx.y, ny = blockDim.y;
  const int d0 = threadIdx.x << 3;
  const int row0 = blockIdx.x * kRows;
  const int rows = min(kRows, num_tokens - row0);
  const int half_dim = head_dim >> 1;
  uint4 lo[kRows], hi[kRows];
#pragma unroll
  for (int j = 0; j < kRows; ++j) {
    if (j < rows && ty < total_heads) {
      const half* base = HeadPtr(q, k, q_row_stride, k_row_stride, row0 + j, ty, num_q_heads, head_dim);
      lo[j] = Ldg16(base + d0);
      hi[j] = Ldg16(base + d0 + half_dim);
    }
  }
  FillCosSin<kRows>(cosv, sinv, positions, row0, rows, half_dim, ty * blockDim.x + threadIdx.x, ny * blockDim.x,
                    inv_freq);
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kRows; ++j) {
    if (j < rows && ty < total_heads) {
      half* base = HeadPtr(q, k, q_row_stride, k_row_stride, row0 + j, ty, num_q_heads, head_dim);
      RotateChunk(lo[j], hi[j], cosv[j] + d0, sinv[j] + d0);
      Stg16(base + d0, lo[j]);
      Stg16(base + d0 + half_dim, hi[j]);
    }
  }
  for (int j = 0; j < rows; ++j) {  // more heads than the block has thread rows
    for (int head = ty + ny; head < total_heads; head += ny) {
      half* base = HeadPtr(q, k, q_row_stride, k_row_stride, row0 + j, head, num_q_heads, head_dim);
      uint4 a = Ldg16(base + d0);
      uint4 b = Ldg16(base + d0 + half_dim);
      RotateChunk(a, b, cosv[j] + d0, sinv[j] + d0);
      Stg16(base + d0, a);
      Stg16(base + d0 + half_dim, b);
    }
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

// RoPE and KV scatter in one pass (head_dim a multiple of 16, 16-byte aligned views). A block covers kRows
// consecutive token rows with RopeVecKernel's thread mapping: it rotates Q and K in place exactly as that
// kernel does, and while a rotated K chunk is in registers also stores it to its page slot. V is copied
// to its slot by the same threads read as rows of 2 * blockDim.x 16-byte words: thread row y takes half
// (y & 1) of V head (y >> 1). The qkv buffer ends up bit-identical to the two-launch sequence, and so
// does the pool. The data requests of a thread's first head and first V word in every row go out before
// the positions, table entries and cos/sin values they do not depend on.
template <int kRows>
__global__ void __launch_bounds__(kRopeThreads)
RopeScatterKernel(half* q, half* k, const half* __restrict__ v, int64_t q_row_stride, int64_t k_row_stride,
                  int64_t v_row_stride, half* __restrict__ pool, const int32_t* __restrict__ tables,
                  int64_t table_row_stride, const int32_t* __restrict__ positions, int num_tokens,
                  int num_q_heads, int num_kv_heads, int head_dim, const __grid_constant__ InvFreq inv_freq) {
  __shared__ __align__(16) half cosv[kRows][kMaxPairs];
  __shared__ __align__(16) half sinv[kRows][kMaxPairs];
  __shared__ int64_t cell_of[kRows];  // element offset of (page, K side, head 0, this token's slot)
  // the attention launch that follows may begin its table walk now (it waits for this grid to
  // complete before it reads the pool or Q); this grid itself waits for the QKV GEMM before it
  DependentLaunchGate();
  const int ty = threadIdx.y, ny = blockDim.y;
  const int tid = ty * blockDim.x + threadIdx.x;
  const int d0 = threadIdx.x << 3;
  const int row0 = blockIdx.x * kRows;
  const int rows = min(kRows, num_tokens - row0);
  const int half_dim = head_dim >> 1;
  const int total_heads = num_q_heads + num_kv_heads;
  const int v_rows = 2 * num_kv_heads;               // V of one token as rows of half_dim elements
  const int64_t head_step = static_cast<int64_t>(kKvBlock) * head_dim;  // pool elements from head h to h + 1
  const int64_t side_step = num_kv_heads * head_step;                   // ... from the K side to the V side

  uint4 lo[kRows], hi[kRows], vv[kRows];
#pragma unroll
  for (int j = 0; j < kRows; ++j) {
    if (j < rows && ty < total_heads) {
      const half* base = HeadPtr(q, k, q_row_stride, k_row_stride, row0 + j, ty, num_q_heads, head_dim);
      lo[j] = Ldg16(base + d0);
      hi[j] = Ldg16(base + d0 + half_dim);
    }
    if (j < rows && ty < v_rows) vv[j] = Ldg16(v + (row0 + j) * v_row_stride + ty * half_dim + d0);
  }
  if (tid < rows) {
    const int64_t row = row0 + tid;
    const int p = positions[row];
    const int64_t page = tables[row * table_row_stride + (p >> kKvBlockShift)];
    cell_of[tid] = page * 2 * side_step + static_cast<int64_t>(p & (kKvBlock - 1)) * head_dim;
  }
  FillCosSin<kRows>(cosv, sinv, positions, row0, rows, half_dim, tid, ny * blockDim.x, inv_freq);
  __syncthreads();

  auto finish_head = [&](int j, int head, uint4& a, uint4& b) {
    half* base = HeadPtr(q, k, q_row_stride, k_row_stride, row0 + j, head, num_q_heads, head_dim);
    RotateChunk(a, b, cosv[j] + d0, sinv[j] + d0);
    Stg16(base + d0, a);
    Stg16(base + d0 + half_dim, b);
    if (head >= num_q_heads) {
      half* dst = pool + cell_of[j] + (head - num_q_heads) * head_step;
      Stg16(dst + d0, a);
      Stg16(dst + d0 + half_dim, b);
    }
  };
  auto finish_v = [&](int j, int vy, const uint4& w) {
    half* dst = pool + cell_of[j] + side_step + (vy >> 1) * head_step;
    Stg16(dst + (vy & 1) * half_dim + d0, w);
  };
#pragma unroll
  for (int j = 0; j < kRows; ++j) {
    if (j < rows && ty < total_heads) finish_head(j, ty, lo[j], hi[j]);
    if (j < rows && ty < v_rows) finish_v(j, ty, vv[j]);
  }
  for (int j = 0; j < rows; ++j) {  // more heads / V rows than the block has thread rows
    for (int head = ty + ny; head < total_heads; head += ny) {
      const half* base = HeadPtr(q, k, q_row_stride, k_row_stride, row0 + j, head, num_q_heads, head_dim);
      uint4 a = Ldg16(base + d0);
      uint4 b = Ldg16(base + d0 + half_dim);
      finish_head(j, head, a, b);
    }
    for (int vy = ty + ny; vy < v_rows; vy += ny) {
      finish_v(j, vy, Ldg16(v + (row0 + j) * v_row_stride + vy * half_dim + d0));
    }
  }
}

// Rows per CTA once there are enough token rows to fill the device several times over (prompt chunks);
// decode batches keep one row per CTA for the shortest critical path.
#ifndef RL_ROPE_ROWS_BIG
#define RL_ROPE_ROWS_BIG 2
#endif
constexpr int kRowsBig = RL_ROPE_ROWS_BIG;

// (chunks of 8 pairs per head) x (as many head rows as fit in 128 threads)
inline dim3 RopeBlock(int head_dim) {
  const int chunks = head_dim >> 4;
  return dim3(chunks, kRopeThreads / chunks);
}

inline bool ManyRows(int num_tokens) { return num_tokens >= 16 * CurrentDeviceFacts().sm_count; }

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
  if (vec && ManyRows(num_tokens)) {
    RopeVecKernel<kRowsBig><<<(num_tokens + kRowsBig - 1) / kRowsBig, RopeBlock(head_dim), 0, s>>>(
        qq, kk, q_row_stride, k_row_stride, positions, num_tokens, num_q_heads, total_heads, head_dim, table);
  } else if (vec) {
    RopeVecKernel<1><<<num_tokens, RopeBlock(head_dim), 0, s>>>(qq, kk, q_row_stride, k_row_stride, positions,
                                                                num_tokens, num_q_heads, total_heads, head_dim, table);
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
  const bool many = ManyRows(num_tokens);
  const int per_cta = many ? kRowsBig : 1;
  LaunchOverlapped(many ? RopeScatterKernel<kRowsBig> : RopeScatterKernel<1>,
                   dim3((num_tokens + per_cta - 1) / per_cta), RopeBlock(head_dim), 0,
                   static_cast<cudaStream_t>(stream), static_cast<half*>(q), static_cast<half*>(k),
                   static_cast<const half*>(v), q_row_stride, k_row_stride, v_row_stride,
                   static_cast<half*>(kv_pool_layer), block_tables, block_table_row_stride, positions, num_tokens,
                   num_q_heads, num_kv_heads, head_dim, table);
  return LaunchStatus("rope_kv_scatter");
}
