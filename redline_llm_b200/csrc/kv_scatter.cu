// KV scatter into the 16-token paged pool through block-table indirection,
// for sm_100a. A pure bit move (NaN payloads survive): for token t,
//   p = positions[t]; block = block_tables[t*row_stride + (p >> 4)]; slot = p & 15
//   pool[block][0][h][slot][:] = k[t][h][:],  pool[block][1][h][slot][:] = v[t][h][:]
// (src/kernels/kv_scatter.cu:98-137; pool index formula src/kernels/kv_scatter.cu:82-88).
// row_stride == 0 shares one table row among all tokens (prefill).
//
// Mapping: one warp per token; a token's K and V rows are 2*H*D/8 16-byte
// words (64 for 2 heads x 128), dealt lane-contiguously so both the read and
// the 256-byte pool rows are fully coalesced. A 2-byte-word variant of the
// same body covers odd strides and unaligned bases.
#include "common.cuh"

namespace rl {
namespace {

template <typename Word, int kTokens>
__global__ void __launch_bounds__(128)
KvScatterKernel(half* __restrict__ pool, const half* __restrict__ k, const half* __restrict__ v,
                int64_t k_row_stride, int64_t v_row_stride, const int32_t* __restrict__ tables,
                int64_t table_row_stride, const int32_t* __restrict__ positions, int num_tokens,
                int num_kv_heads, int head_dim) {
  constexpr int kPer = sizeof(Word) / sizeof(half);
  // the attention launch that follows may begin its table walk now (it waits for this grid to
  // complete before it reads the pool)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int64_t t0 = (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kTokens;
  if (t0 >= num_tokens) return;
  const int tokens = static_cast<int>(min(static_cast<int64_t>(kTokens), num_tokens - t0));
  const int lane = threadIdx.x & 31;
  const int words_per_head = head_dim / kPer;
  const int words_per_side = num_kv_heads * words_per_head;
  const int words = 2 * words_per_side;
  const int64_t slot_elems = head_dim;                                  // one token of one head
  const int64_t page_elems = 2 * num_kv_heads * kKvBlock * slot_elems;  // [2][heads][16][head_dim]
  // word w of a token: where it is read (K row or V row) and where it lands inside (page, slot 0)
  auto src_of = [&](int w, int64_t t) {
    return w >= words_per_side ? reinterpret_cast<const Word*>(v + t * v_row_stride) + (w - words_per_side)
                               : reinterpret_cast<const Word*>(k + t * k_row_stride) + w;
  };
  auto dst_of = [&](int w) {
    const int side_head = w / words_per_head;  // kv * heads + h
    return side_head * kKvBlock * slot_elems + (w - side_head * words_per_head) * kPer;
  };
  // a token's first kAhead words per lane (all of them for 2 heads x 128 in 16-byte words) are requested,
  // for every token of the warp, before the positions and table entries that only the destinations need
  constexpr int kAhead = 2;
  Word held[kTokens][kAhead];
  int64_t dst[kAhead];
#pragma unroll
  for (int j = 0; j < kAhead; ++j) {
    const int w = lane + 32 * j;
    if (w < words) {
#pragma unroll
      for (int i = 0; i < kTokens; ++i) {
        if (i < tokens) held[i][j] = *src_of(w, t0 + i);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kAhead; ++j) {
    if (lane + 32 * j < words) dst[j] = dst_of(lane + 32 * j);
  }
#pragma unroll
  for (int i = 0; i < kTokens; ++i) {
    if (i >= tokens) break;
    const int64_t t = t0 + i;
    const int p = positions[t];
    const int64_t block = tables[t * table_row_stride + (p >> kKvBlockShift)];
    half* cell = pool + block * page_elems + (p & (kKvBlock - 1)) * slot_elems;
#pragma unroll
    for (int j = 0; j < kAhead; ++j) {
      if (lane + 32 * j < words) *reinterpret_cast<Word*>(cell + dst[j]) = held[i][j];
    }
    for (int w = lane + 32 * kAhead; w < words; w += 32) {
      *reinterpret_cast<Word*>(cell + dst_of(w)) = *src_of(w, t);
    }
  }
}

}  // namespace
}  // namespace rl

extern "C" int rl_launch_kv_scatter(void* kv_pool_layer, const void* k, const void* v,
                                    int64_t k_row_stride, int64_t v_row_stride,
                                    const int32_t* block_tables, int64_t block_table_row_stride,
                                    const int32_t* positions, int32_t num_tokens,
                                    int32_t num_kv_heads, int32_t head_dim, void* stream) {
  using namespace rl;
  if (num_tokens <= 0 || num_kv_heads <= 0 || head_dim <= 0) return RL_OK;
  if (!kv_pool_layer || !k || !v || !block_tables || !positions)
    return Fail(RL_E_NULL_POINTER, "kv_scatter: null device pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  half* pool = static_cast<half*>(kv_pool_layer);
  const half* kk = static_cast<const half*>(k);
  const half* vv = static_cast<const half*>(v);
  const bool vec = head_dim % 8 == 0 && k_row_stride % 8 == 0 && v_row_stride % 8 == 0 &&
                   Aligned16(pool) && Aligned16(k) && Aligned16(v);
  // decode batches: a warp per token, a block per token; prompt chunks: four warps per block, and once
  // that still fills the device several times over, two tokens per warp
  const int sms = CurrentDeviceFacts().sm_count;
  const int wpb = num_tokens >= 4 * sms ? 4 : 1;
  const int tpw = num_tokens >= 64 * sms ? 2 : 1;
  const dim3 grid((num_tokens + wpb * tpw - 1) / (wpb * tpw)), block(32 * wpb);
  auto launch = [&](auto kernel) {
    kernel<<<grid, block, 0, s>>>(pool, kk, vv, k_row_stride, v_row_stride, block_tables, block_table_row_stride,
                                  positions, num_tokens, num_kv_heads, head_dim);
  };
  if (vec && tpw == 2) launch(KvScatterKernel<uint4, 2>);
  else if (vec) launch(KvScatterKernel<uint4, 1>);
  else if (tpw == 2) launch(KvScatterKernel<half, 2>);
  else launch(KvScatterKernel<half, 1>);
  return LaunchStatus("kv_scatter");
}
