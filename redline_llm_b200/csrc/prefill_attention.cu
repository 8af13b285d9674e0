// Fused paged prefill attention for sm_100a (B200): one prompt chunk of one sequence attends causally
// to everything cached for that sequence - earlier chunks and itself - straight out of the paged pool.
//
// The reference ingests a chunk through a composite (src/core/model_executor.cpp:1219-1290): LaunchKvGather
// copies the sequence's pages into dense K / V staging, cuBLASLt writes FP32 scores [heads, chunk, ctx] to
// global memory, LaunchPrefillSoftmax rewrites them as FP16 probabilities, cuBLASLt multiplies by V; its
// design notes name a fused kernel as the follow-up (docs/DESIGN.md:872-876). This is that kernel: the
// same function - scores q.k * scale in FP32 from FP16 operands, causal SELECT masking (key position <=
// query position; slots past the context never reach a result), softmax with FP32 statistics,
// probabilities rounded to FP16 for the P.V product, FP32 accumulation, one FP16 rounding of acc / l -
// with nothing but Q, the pages and the output ever touching global memory.
//
// Mapping. One CTA per (128-row query tile, query head); 128 threads, thread t owns query row t.
//  * Q tile and K/V blocks of 128 keys (8 pages) arrive by TMA with the 128-byte swizzle. A page tile
//    of the pool is [16 tokens][128 dims]; each 64-dim half of it is one 2 KiB tensor copy landing at row
//    16 * page of a [128 rows][128 B] region, so eight pages form exactly the K-major operand tile
//    tcgen05 expects - block-table indirection costs nothing but the copy's coordinate. K/V blocks are
//    double-buffered; the six query heads of a KV group and all query tiles re-read the same pages from L2.
//  * S = Q.K^T: tcgen05.mma, M = 128 query rows, N = 128 keys, K = 16 dims x 8, both operands K-major
//    in shared memory, FP32 accumulator in tensor memory (columns 0-127).
//  * Softmax: each thread reads its row of S from tensor memory (tcgen05.ld 32x32b) twice - once for the
//    row maximum, once to exponentiate - in the exp2 domain with the running maximum of an online
//    softmax, and writes P as FP16 into shared memory in the swizzled K-major layout by hand.
//  * O_blk = P.V: tcgen05.mma with A = P (K-major) and B = V as it lies in the pool - [key][dim], i.e.
//    MN-major: atoms of 8 keys x 64 dims, 1024 B between key groups, one region per 64-dim half -
//    into tensor-memory columns 128-255; the thread then folds it into its row's running output held in
//    registers, scaled by exp2(m_old - m_new).
//  * The next block's S is issued right behind P.V, so the tensor pipe works on it while the threads fold.
// Every mbarrier wait is bounded and reports through the attention health flag.
#include <cuda.h>

#include <mutex>

#include "tc_ptx.cuh"

namespace rl {
namespace pfa {

using namespace rl::tc;

constexpr int kHeadDim = 128;
constexpr int kBM = 128;                 // query rows per CTA
constexpr int kBN = 128;                 // keys per block (8 pages)
constexpr int kThreads = 128;
constexpr int kPagesPerBlock = kBN / kKvBlock;
constexpr int kRegionBytes = 128 * 128;  // [128 rows][64 halves], 128-byte swizzle
constexpr int kTileBytes = 2 * kRegionBytes;   // two 64-wide halves
constexpr int kQOff = 0;
constexpr int kKOff = kQOff + kTileBytes;          // 2 buffers
constexpr int kVOff = kKOff + 2 * kTileBytes;      // 2 buffers
constexpr int kPOff = kVOff + 2 * kTileBytes;
constexpr int kBarOff = kPOff + kTileBytes;        // mbarriers + tmem slot
constexpr int kSmemBytes = kBarOff + 128 + 1024;   // + slack to align the base to 1024
static_assert(kSmemBytes <= 227 * 1024, "prefill attention shared memory exceeds the per-CTA limit");
constexpr int kTmemCols = 256;           // S: columns 0-127, P.V: 128-255

struct Params {
  half* out;
  int64_t out_stride;
  const int32_t* table_row;
  int chunk_start;
  int chunk_len;
  int max_blocks;
  int q_heads;
  int kv_heads;
  float scale_log2e;
  int* error_flag;
};

// K/V block operand as a B matrix stored [key][dim] (MN-major, 128-byte swizzle): atoms of 8 key rows x 128 B;
// `lbo` bytes between the two 64-dim halves (leading dimension = N), 1024 B between 8-key groups (stride dimension = K).
__device__ __forceinline__ uint64_t TileDescMn(uint32_t smem_addr, uint32_t lbo_bytes) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
         (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint32_t InstrDescBMn(int n) { return InstrDesc(n) | (1u << 16); }

// One 64-dim half of one (block, kv, head) page tile: [16 tokens][64 halves] = 2 KiB.
__device__ __forceinline__ void TmaLoadHalfTile(uint32_t dst, const CUtensorMap* map, int half_idx, int tile,
                                                uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %2, %3, %4}], [%5], %6;" ::"r"(dst),
      "l"(map), "r"(0), "r"(half_idx), "r"(tile), "r"(bar), "l"(policy)
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
PagedPrefillAttentionKernel(const Params p, const __grid_constant__ CUtensorMap q_map,
                            const __grid_constant__ CUtensorMap tile_map) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t s_q = SmemAddr(smem + kQOff), s_k = SmemAddr(smem + kKOff), s_v = SmemAddr(smem + kVOff);
  const uint32_t s_p = SmemAddr(smem + kPOff);
  const uint32_t bars = SmemAddr(smem + kBarOff);
  const uint32_t bar_q = bars, bar_k0 = bars + 8, bar_v0 = bars + 24, bar_s = bars + 40, bar_o = bars + 48;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kBarOff + 64);

  const int tid = threadIdx.x, warp = tid >> 5;
  // long tiles first: the last query tile of the chunk attends to the most keys
  const int tile_q = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int row0 = tile_q * kBM;
  const int kv_len = p.chunk_start + p.chunk_len;
  const int last_pos = min(p.chunk_start + row0 + kBM, kv_len) - 1;   // newest key any row of this tile sees
  const int nblk = last_pos / kBN + 1;
  const int my_pos = min(p.chunk_start + row0 + tid, kv_len - 1);      // rows past the chunk are computed, never stored

  if (tid == 0) {
    MbarInit(bar_q, 1);
    for (int i = 0; i < 2; ++i) {
      MbarInit(bar_k0 + 8 * i, 1);
      MbarInit(bar_v0 + 8 * i, 1);
    }
    MbarInit(bar_s, 1);
    MbarInit(bar_o, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&q_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tile_map) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     SmemAddr(const_cast<uint32_t*>(tmem_slot))),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + kBN;

  const uint64_t keep = L2PolicyEvictLast(), normal = L2PolicyEvictNormal();
  // Block j of K (kv = 0) or V (kv = 1) into buffer j & 1: 8 pages x 2 halves, each 2 KiB at row 16 * page.
  auto load_block = [&](int j, int kv) {
    const int buf = j & 1;
    const uint32_t base = (kv ? s_v : s_k) + buf * kTileBytes;
    const uint32_t bar = (kv ? bar_v0 : bar_k0) + 8 * buf;
    MbarExpectTx(bar, kTileBytes);
#pragma unroll 1
    for (int pg = 0; pg < kPagesPerBlock; ++pg) {
      const int page = j * kPagesPerBlock + pg;
      const int block = page < p.max_blocks ? __ldg(p.table_row + page) : 0;   // past the table: the dummy block
      const int tile = (block * 2 + kv) * p.kv_heads + kv_head;
      TmaLoadHalfTile(base + pg * (kKvBlock * 128), &tile_map, 0, tile, bar, keep);
      TmaLoadHalfTile(base + kRegionBytes + pg * (kKvBlock * 128), &tile_map, 1, tile, bar, keep);
    }
  };
  const uint32_t idesc_kk = InstrDesc(kBN), idesc_mn = InstrDescBMn(kHeadDim);
  // S = Q.K_j^T into tensor-memory columns 0-127 (thread 0 only).
  auto issue_qk = [&](int j) {
    const uint32_t kb = s_k + (j & 1) * kTileBytes;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint64_t a = TileDesc(s_q + h * kRegionBytes), b = TileDesc(kb + h * kRegionBytes);
#pragma unroll
      for (int k = 0; k < 4; ++k) Umma(tmem_s, a + 2 * k, b + 2 * k, idesc_kk, (h | k) ? 1u : 0u);
    }
    UmmaCommit(bar_s);
  };
  // O_blk = P.V_j into columns 128-255: K = 16 keys per instruction, V read MN-major where it landed.
  auto issue_pv = [&](int j) {
    const uint32_t vb = s_v + (j & 1) * kTileBytes;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint64_t a = TileDesc(s_p + h * kRegionBytes);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint64_t b = TileDescMn(vb + (h * 4 + k) * (16 * 128), kRegionBytes);
        Umma(tmem_o, a + 2 * k, b, idesc_mn, (h | k) ? 1u : 0u);
      }
    }
    UmmaCommit(bar_o);
  };

  bool ok = true;
  auto wait = [&](uint32_t bar, int parity) {
    if (ok && !MbarWait(bar, parity)) {
      ok = false;
      atomicExch(p.error_flag, 2);
    }
  };

  if (tid == 0) {
    MbarExpectTx(bar_q, kTileBytes);
    TmaLoad2D(s_q, &q_map, head * kHeadDim, row0, bar_q, normal);
    TmaLoad2D(s_q + kRegionBytes, &q_map, head * kHeadDim + 64, row0, bar_q, normal);
    load_block(0, 0);
    load_block(0, 1);
    if (nblk > 1) {
      load_block(1, 0);
      load_block(1, 1);
    }
    wait(bar_q, 0);
    wait(bar_k0, 0);
    TcFenceAfter();
    if (ok) issue_qk(0);
  }

  float o[kHeadDim];
#pragma unroll
  for (int i = 0; i < kHeadDim; ++i) o[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;
  const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;   // this warp's quarter of the tensor-memory lanes
  uint8_t* p_row = smem + kPOff + tid * 128;

#pragma unroll 1
  for (int j = 0; j < nblk; ++j) {
    const int buf = j & 1;
    wait(bar_s, j & 1);
    TcFenceAfter();
    // K buffer `buf` is free again: fetch block j + 2 into it
    if (tid == 0 && j + 2 < nblk) load_block(j + 2, 0);
    const int key0 = j * kBN;
    const bool diagonal = key0 + kBN - 1 > p.chunk_start + row0;   // some row of the tile is masked inside this block
    // pass 1: the row maximum
    float mx = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < kBN / 16; ++c) {
      uint32_t raw[16];
      TmemLoad16(tmem_s + lane_addr + c * 16, raw);
      TmemWaitLoads(raw);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float s = __uint_as_float(raw[i]) * p.scale_log2e;
        mx = fmaxf(mx, (!diagonal || key0 + c * 16 + i <= my_pos) ? s : -INFINITY);
      }
    }
    const float m_new = fmaxf(m, mx);            // finite: key 0 is visible to every row
    const float alpha = exp2f(m - m_new);        // 0 on the first block
    // pass 2: probabilities, FP16, into the swizzled K-major P tile; their FP32 sum
    float sum = 0.0f;
#pragma unroll 1
    for (int c = 0; c < kBN / 16; ++c) {
      uint32_t raw[16];
      TmemLoad16(tmem_s + lane_addr + c * 16, raw);
      TmemWaitLoads(raw);
      uint32_t packed[8];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        const float s0 = __uint_as_float(raw[i]) * p.scale_log2e, s1 = __uint_as_float(raw[i + 1]) * p.scale_log2e;
        const float p0 = (!diagonal || key0 + c * 16 + i <= my_pos) ? exp2f(s0 - m_new) : 0.0f;
        const float p1 = (!diagonal || key0 + c * 16 + i + 1 <= my_pos) ? exp2f(s1 - m_new) : 0.0f;
        const half2 h2 = __floats2half2_rn(p0, p1);
        sum += __low2float(h2) + __high2float(h2);   // the sum of what the P.V product will actually use
        packed[i >> 1] = AsU32(h2);
      }
      // keys c*16 .. c*16+15 = 16-byte chunks 2c and 2c+1 of this row; region = keys / 64
      uint8_t* region = p_row + (c >> 2) * kRegionBytes;
      const int ch = (2 * c) & 7;
      *reinterpret_cast<uint4*>(region + (((ch) ^ (tid & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      *reinterpret_cast<uint4*>(region + (((ch + 1) ^ (tid & 7)) << 4)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    }
    l = l * alpha + sum;
    m = m_new;
    // V rows at or past the context end (the last block only) may hold anything, NaN included, and 0 * NaN
    // would poison the row: clear them once the block has landed.
    const int rows_valid = kv_len - key0;
    if (rows_valid < kBN) {
      wait(bar_v0 + 8 * buf, (j >> 1) & 1);
      if (tid >= rows_valid) {
        uint4* r0 = reinterpret_cast<uint4*>(smem + kVOff + buf * kTileBytes + tid * 128);
        uint4* r1 = reinterpret_cast<uint4*>(smem + kVOff + buf * kTileBytes + kRegionBytes + tid * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) r0[i] = r1[i] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P (and cleared V rows) visible to the tensor pipe
    TcFenceBefore();
    __syncthreads();
    if (tid == 0) {
      wait(bar_v0 + 8 * buf, (j >> 1) & 1);
      TcFenceAfter();
      if (ok) issue_pv(j);
      if (j + 1 < nblk) {
        wait(bar_k0 + 8 * (buf ^ 1), ((j + 1) >> 1) & 1);
        if (ok) issue_qk(j + 1);
      }
    }
    wait(bar_o, j & 1);
    TcFenceAfter();
    if (tid == 0 && j + 2 < nblk) load_block(j + 2, 1);   // V buffer `buf` is free again
#pragma unroll
    for (int c = 0; c < kHeadDim / 16; ++c) {
      uint32_t raw[16];
      TmemLoad16(tmem_o + lane_addr + c * 16, raw);
      TmemWaitLoads(raw);
#pragma unroll
      for (int i = 0; i < 16; ++i) o[c * 16 + i] = fmaf(o[c * 16 + i], alpha, __uint_as_float(raw[i]));
    }
    TcFenceBefore();
    if (!__syncthreads_and(ok)) break;   // some wait gave up: every thread leaves together
  }

  const int row = row0 + tid;
  if (ok && row < p.chunk_len) {
    const float inv = 1.0f / l;
    half* dst = p.out + static_cast<int64_t>(row) * p.out_stride + head * kHeadDim;
#pragma unroll
    for (int c = 0; c < kHeadDim / 8; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = AsU32(__floats2half2_rn(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv));
      *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  // Copies still in flight target this CTA's shared memory: let them land before it is released.
  if (!ok && tid == 0) {
    for (int i = 0; i < 2; ++i) {
      MbarWait(bar_k0 + 8 * i, 0);
      MbarWait(bar_v0 + 8 * i, 0);
    }
  }
  TcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
constexpr int kMaxDevices = 64;
struct DeviceState {
  bool ready = false;
  int* error_flag = nullptr;
};
DeviceState g_state[kMaxDevices];
EncodeTiledFn g_encode = nullptr;
std::mutex g_mutex;

int EnsureReady(DeviceState** out_state) {
  const int dev = CurrentDeviceIndex();
  DeviceState& st = g_state[dev];
  *out_state = &st;
  if (st.ready) return RL_OK;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (st.ready) return RL_OK;
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
      return Fail(e != cudaSuccess ? static_cast<int>(e) : RL_E_WORKSPACE,
                  "paged_prefill_attention: cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  if (CurrentDeviceFacts().max_smem_optin < kSmemBytes)
    return Fail(RL_E_WORKSPACE, "paged_prefill_attention: device offers %d B of shared memory per block, %d needed",
                CurrentDeviceFacts().max_smem_optin, kSmemBytes);
  cudaError_t e = cudaFuncSetAttribute(PagedPrefillAttentionKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kSmemBytes);
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "paged_prefill_attention: shared-memory opt-in: %s", cudaGetErrorString(e));
  e = cudaMalloc(reinterpret_cast<void**>(&st.error_flag), 256);
  if (e == cudaSuccess) e = cudaMemset(st.error_flag, 0, 256);
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "paged_prefill_attention: flag: %s", cudaGetErrorString(e));
  st.ready = true;
  return RL_OK;
}

}  // namespace pfa
}  // namespace rl

extern "C" int rl_launch_paged_prefill_attention(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride,
                                                 const void* kv_pool_layer, const int32_t* block_table_row,
                                                 int32_t max_blocks_per_seq, int32_t chunk_start, int32_t chunk_len,
                                                 int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                                 float scale, void* stream) {
  using namespace rl;
  using namespace rl::pfa;
  if (chunk_len <= 0) return RL_OK;
  if (!out || !q || !kv_pool_layer || !block_table_row)
    return Fail(RL_E_NULL_POINTER, "paged_prefill_attention: null device pointer");
  if (head_dim != kHeadDim) return Fail(RL_E_BAD_SHAPE, "paged_prefill_attention: head_dim must be 128");
  if (num_kv_heads < 1 || num_kv_heads > 8 || num_q_heads < num_kv_heads || num_q_heads % num_kv_heads != 0)
    return Fail(RL_E_BAD_SHAPE, "paged_prefill_attention: num_q_heads must be a positive multiple of num_kv_heads (<= 8 KV heads)");
  if (chunk_start < 0 || max_blocks_per_seq < 1 ||
      static_cast<int64_t>(chunk_start) + chunk_len > static_cast<int64_t>(max_blocks_per_seq) * kKvBlock)
    return Fail(RL_E_BAD_SHAPE, "paged_prefill_attention: the chunk runs past the block table row");
  const int64_t width = static_cast<int64_t>(num_q_heads) * head_dim;
  if (q_row_stride < width || out_row_stride < width)
    return Fail(RL_E_BAD_SHAPE, "paged_prefill_attention: row stride smaller than the row");
  if ((q_row_stride & 7) || (out_row_stride & 7) || !Aligned16(q) || !Aligned16(out) || !Aligned16(kv_pool_layer))
    return Fail(RL_E_BAD_SHAPE, "paged_prefill_attention: q, out and the pool slice must be 16-byte aligned with row strides in multiples of 8");
  DeviceState* st;
  int rc = EnsureReady(&st);
  if (rc != RL_OK) return rc;
  CUtensorMap q_map, tile_map;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(chunk_len)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(q_row_stride) * 2};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(kBM)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(q), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return Fail(RL_E_BAD_SHAPE, "paged_prefill_attention: q tensor map (CUresult %d)", static_cast<int>(r));
  }
  {
    // the pool slice as [tile][dim-half][token][64 halves]; one box = one 64-dim half of one page tile
    const cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(kKvBlock), 2, 1ull << 26};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(kHeadDim) * 2, 128, static_cast<cuuint64_t>(kKvBlock) * kHeadDim * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(kKvBlock), 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = g_encode(&tile_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(kv_pool_layer), dims, strides,
                                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return Fail(RL_E_BAD_SHAPE, "paged_prefill_attention: pool tensor map (CUresult %d)", static_cast<int>(r));
  }
  Params p;
  p.out = static_cast<half*>(out);
  p.out_stride = out_row_stride;
  p.table_row = block_table_row;
  p.chunk_start = chunk_start;
  p.chunk_len = chunk_len;
  p.max_blocks = max_blocks_per_seq;
  p.q_heads = num_q_heads;
  p.kv_heads = num_kv_heads;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.error_flag = st->error_flag;
  const dim3 grid((chunk_len + kBM - 1) / kBM, num_q_heads);
  PagedPrefillAttentionKernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(p, q_map, tile_map);
  return LaunchStatus("paged_prefill_attention");
}

extern "C" int rl_prefill_attention_health(int* flag_out) {
  using namespace rl;
  using namespace rl::pfa;
  if (!flag_out) return Fail(RL_E_NULL_POINTER, "rl_prefill_attention_health: null pointer");
  *flag_out = 0;
  DeviceState& st = g_state[CurrentDeviceIndex()];
  if (!st.ready) return RL_OK;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(flag_out, st.error_flag, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && *flag_out != 0) e = cudaMemset(st.error_flag, 0, sizeof(int));
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "rl_prefill_attention_health: %s", cudaGetErrorString(e));
  return RL_OK;
}
