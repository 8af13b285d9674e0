// Decode-sized linear layer for sm_100a (B200): out[T, N] = x[T, K] . W[N, K]^T (+ bias), T <= 64.
//
// In the reference every linear layer of the decode step is a cuBLASLt call whose algorithm is the
// first heuristic result (src/gemm/cublaslt_gemm.cpp:569-598, called from
// src/core/model_executor.cpp:916-951). With at most 64 token rows these products are weight
// streams: every weight is read once and used 64 times, so the bound is HBM, and the library
// kernels reach 15-70 % of it at the reference model's shapes. This kernel is built for exactly that case.
//
//  * The weight matrix is the M operand. A CTA owns 128 weight rows and a contiguous range of
//    64-wide k-blocks; tcgen05.mma (M=128, N=tokens padded to 16, K=16, FP16 in, FP32 accumulate)
//    reads both operands from shared memory and keeps the 128 x T accumulator in tensor memory.
//    One thread issues the MMAs; one thread issues the TMA loads; a ring of (128 x 64 weights,
//    T x 64 activations) tiles, 128-byte swizzled, keeps 16 KB of weights per stage in flight.
//    Every CTA loads its own tiles; no peer GPU memory is ever touched.
//  * Weights do not depend on the previous kernel of the stream: under programmatic dependent
//    launch the first stages of weights are requested BEFORE griddepcontrol.wait, the activations
//    after it, so the stream of weights starts while the previous kernel drains.
//  * Shapes with few row tiles are split along K so that tiles x splits fills the GPU. The S splits
//    of a tile (2, 4 or 8) form one thread-block cluster. Token t of the tile is finished by CTA
//    t mod S: every CTA sends the FP32 partial sums of that token into the owner's shared memory
//    with asynchronous distributed-shared-memory stores (st.async) that count bytes on the owner's
//    mbarrier; the owner waits (bounded) until everything it expects has landed and adds the S
//    slices in split order 0..S-1 from its own shared memory. No global workspace, no atomics;
//    results do not depend on arrival order.
//  * Epilogue 0 adds the bias in FP32 and rounds once to FP16. Epilogue 1 is the gated MLP input:
//    W holds `gate` rows then `up` rows; a CTA takes 64 of each, rounds both accumulators to FP16
//    (what a separate GEMM would have stored) and writes fp16(silu(gate) * up) - bit-identical to
//    running the SiLU kernel on the GEMM's output (src/kernels/silu_mul.cu:67-83), without the
//    [T, 2I] round trip. Epilogue 2 is the fused QKV projection: a 128-row tile is exactly one head, so
//    the CTA that finishes a token of a tile holds the whole head of that token; it adds the bias,
//    rounds to FP16 (the GEMM output), rotates Q and K heads with the RoPE kernel's own arithmetic
//    (rope_math.cuh), writes the row of the qkv buffer, and stores K and V heads to their slot of the
//    paged pool - bit-identical to GEMM + RoPE + KV scatter (src/core/model_executor.cpp:916-930), two
//    launches fewer.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "rope_math.cuh"
#include "tc_ptx.cuh"
#include "silu_math.cuh"

namespace rl {
namespace lin {

constexpr int kTileRows = 128;   // weight rows per CTA = MMA M
constexpr int kHalfRows = 64;    // rows per weight TMA box (two boxes per stage)
constexpr int kBlockK = 64;      // halves per k-block: one 128-byte swizzle row
constexpr int kMaxTokens = 64;   // MMA N
constexpr int kThreads = 256;    // two warps per tensor-memory lane quadrant in the epilogue
constexpr int kMaxStages = 8;
constexpr int kMaxSplits = 8;    // portable cluster size
constexpr int kWTileBytes = kTileRows * 128;    // 16384
constexpr int kXTileBytes = kMaxTokens * 128;   // 8192 (T x 128 B used)
constexpr int kStageBytes = kWTileBytes + kXTileBytes;
// Shared memory, from a 1024-byte aligned base: barriers and small slots, the receive area of a
// split launch, then the ring. Without splits the idle ring stages the FP16 tile for the output pass.
constexpr int kBarOff = 0;     // full[kMaxStages], empty[kMaxStages], accum, receive, tmem slot
constexpr int kRecvOff = 1024;                      // split K only: partial sums received from the cluster
constexpr int kRecvBytes = kMaxTokens * kTileRows * 4;   // S slices x (64 / S) tokens x 128 rows, FP32
// Epilogue 2 only: {cos, sin} of this CTA's tokens (FP16 pairs) and each token's position and page block,
// prepared by the idle epilogue warps while the weights stream.
constexpr int kRopeSlots = 16;                              // tokens per owner covered by the table (T / S <= 16 for S >= 4)
constexpr int kRopeOff = kRecvOff + kRecvBytes;
constexpr int kRopeBytes = kRopeSlots * (kMaxPairs * 4 + 8) + 512;   // 4 KB of pairs + (pos, block) per token, rounded to 5 KB
static_assert((kRopeOff + 5120) % 1024 == 0 && kRopeBytes <= 5120, "rope table carve");
__host__ __device__ constexpr int RingOff(int splits) { return splits > 1 ? kRopeOff + 5120 : 1024; }
__host__ __device__ constexpr int SmemBytes(int stages, int splits) { return RingOff(splits) + stages * kStageBytes + 1024; }  // + slack to align the base
static_assert(SmemBytes(kMaxStages, 1) <= 227 * 1024, "decode linear shared memory exceeds the 227 KB per-CTA limit");
static_assert(SmemBytes(kMaxStages - 1, 8) <= 227 * 1024, "decode linear shared memory exceeds the 227 KB per-CTA limit");
static_assert(2 * kStageBytes >= kMaxTokens * kTileRows * 4, "the tile (FP16, or FP32 before a split's exchange) is staged in two idle stages");

enum Epilogue { kEpilogueBias = 0, kEpilogueSiluMul = 1, kEpilogueQkvRope = 2 };
enum ErrorCode { kErrProducerWait = 1, kErrMmaWait = 2, kErrAccumWait = 3, kErrSplitWait = 4 };

struct Params {
  half* out;
  int64_t out_stride;
  const half* bias;      // may be null
  int tokens;            // T
  int tokens_padded;     // MMA N: T rounded up to 16
  int out_cols;          // columns of `out`
  int up_row_offset;     // epilogue 1: first `up` row of W; unused otherwise
  int k_blocks;          // ceil(K / 64)
  int splits;            // CTAs per row tile along K = cluster size: 1, 2, 4 or 8
  int split_shift;       // log2(splits)
  int stages;            // ring depth
  int weights_sweep_l2;  // weight tiles at normal L2 priority instead of evict-first
  int epilogue;
  int tmem_cols;         // 32 or 64
  int out_vec;           // out rows are 16-byte aligned: vector stores allowed
  int* error_flag;
  unsigned long long* timeline;  // diagnostics build only
};

// Epilogue 2 only: where the rotated K and the V of each token go, and the RoPE table.
struct RopeArgs {
  const int32_t* positions;
  const int32_t* tables;
  int64_t table_row_stride;
  half* pool;          // one layer: [blocks][2][kv_heads][16][128]
  int q_heads;
  int kv_heads;
  InvFreq inv_freq;
};

using namespace tc;

#ifdef RL_LIN_TIMELINE
__device__ __forceinline__ unsigned long long GlobalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define RL_LSTAMP(slot) \
  if (p.timeline) p.timeline[blockIdx.x * 16 + (slot)] = GlobalTimerNs()
#else
#define RL_LSTAMP(slot)
#endif

// ------------------------------------------------------------------ kernel

__global__ void __launch_bounds__(kThreads)
DecodeLinearKernel(const Params p, const __grid_constant__ CUtensorMap w_map,
                   const __grid_constant__ CUtensorMap x_map, const __grid_constant__ RopeArgs rope) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int ring_off = RingOff(p.splits);
  const uint32_t ring = SmemAddr(smem + ring_off);
  const uint32_t bars = SmemAddr(smem + kBarOff);
  const uint32_t full0 = bars, empty0 = bars + kMaxStages * 8, accum_bar = bars + 2 * kMaxStages * 8;
  const uint32_t recv_bar = bars + (2 * kMaxStages + 1) * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kBarOff + (2 * kMaxStages + 2) * 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x / p.splits, split = blockIdx.x - tile * p.splits;  // split = rank in the cluster
  const int kb0 = static_cast<int>(static_cast<long long>(split) * p.k_blocks / p.splits);
  const int kb1 = static_cast<int>(static_cast<long long>(split + 1) * p.k_blocks / p.splits);
  const int nkb = kb1 - kb0;
  const int T = p.tokens, TP = p.tokens_padded, stages = p.stages;
  const int first_row0 = (p.epilogue == kEpilogueSiluMul) ? tile * kHalfRows : tile * kTileRows;
  const int second_row0 = (p.epilogue == kEpilogueSiluMul) ? p.up_row_offset + tile * kHalfRows
                                                            : tile * kTileRows + kHalfRows;
  const int stage_tx = kWTileBytes + TP * 128;
  const int pre = nkb < stages ? nkb : stages;

  if (tid == 0) {
    RL_LSTAMP(0);
    for (int s = 0; s < stages; ++s) {
      MbarInit(full0 + s * 8, 1);
      MbarInit(empty0 + s * 8, 1);
    }
    MbarInit(accum_bar, 1);
    MbarInit(recv_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // The first ring of weight tiles is requested at once: weights never depend on the previous
    // kernel of the stream, so this runs ahead of the dependency gate and of the TMEM set-up.
    const uint64_t stream_policy = p.weights_sweep_l2 ? L2PolicyEvictNormal() : L2PolicyEvictFirst();
    for (int i = 0; i < pre; ++i) {
      const uint32_t dst = ring + i * kStageBytes, bar = full0 + i * 8;
      MbarExpectTx(bar, stage_tx);
      TmaLoad2D(dst, &w_map, (kb0 + i) * kBlockK, first_row0, bar, stream_policy);
      TmaLoad2D(dst + kHalfRows * 128, &w_map, (kb0 + i) * kBlockK, second_row0, bar, stream_policy);
    }
    RL_LSTAMP(2);
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     SmemAddr(const_cast<uint32_t*>(tmem_slot))),
                 "r"(p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem_base = *tmem_slot;
  // Split launches: tell the cluster this CTA is running with its barriers initialised (thread 0
  // fenced the initialisation at cluster scope above, so a relaxed arrival is enough - a releasing one
  // would wait here for the weight loads already in flight); the matching wait comes just before the
  // first remote store.
  if (p.splits > 1) ClusterArriveRelaxed();
  if (tid == 0) { RL_LSTAMP(1); }

  // Epilogue 2: positions and block tables were uploaded at the start of the step, so warps 2-7 - idle until the
  // accumulator is ready - prepare what the RoPE + scatter epilogue needs for the tokens this CTA will finish
  // (t = split, split + S, ...): position, page block, and the FP16 {cos, sin} of all 64 rotation pairs.
  half2* rope_cs = reinterpret_cast<half2*>(smem + kRopeOff);
  int* rope_pos = reinterpret_cast<int*>(smem + kRopeOff + kRopeSlots * kMaxPairs * 4);
  int* rope_block = rope_pos + kRopeSlots;
  const bool rope_table = p.epilogue == kEpilogueQkvRope && p.splits > 1 &&
                          ((T + p.splits - 1) >> p.split_shift) <= kRopeSlots;
  if (rope_table && warp >= 2) {
    const int mine = T > split ? (T - split + p.splits - 1) >> p.split_shift : 0;
    const bool rotate = tile < rope.q_heads + rope.kv_heads;
    for (int u = tid - 64; u < mine * kMaxPairs; u += kThreads - 64) {
      const int k = u >> 6, d = u & (kMaxPairs - 1);
      const int t = (k << p.split_shift) + split;
      const int pos = rope.positions[t];
      if (d == 0) {
        rope_pos[k] = pos;
        rope_block[k] = tile >= rope.q_heads ? rope.tables[t * rope.table_row_stride + (pos >> kKvBlockShift)] : 0;
      }
      if (rotate) rope_cs[k * kMaxPairs + d] = RopeCosSin(static_cast<float>(pos), rope.inv_freq.f[d]);
    }
  }

  // The bias of the columns this thread will finish in a split epilogue-2 launch (column group fixed per thread),
  // fetched now rather than after the exchange.
  float bias_lo[4] = {0.0f, 0.0f, 0.0f, 0.0f}, bias_hi[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (p.epilogue == kEpilogueQkvRope && p.bias) {
    const half* bl = p.bias + tile * kTileRows + (tid & 15) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      bias_lo[e] = __half2float(bl[e]);
      bias_hi[e] = __half2float(bl[64 + e]);
    }
  }

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: activations once the previous kernel has completed, then the steady state
      const uint64_t stream_policy = p.weights_sweep_l2 ? L2PolicyEvictNormal() : L2PolicyEvictFirst();
      const uint64_t keep_policy = L2PolicyEvictLast();
      asm volatile("griddepcontrol.wait;" ::: "memory");
      RL_LSTAMP(9);
      for (int i = 0; i < pre; ++i)
        TmaLoad2D(ring + i * kStageBytes + kWTileBytes, &x_map, (kb0 + i) * kBlockK, 0, full0 + i * 8, keep_policy);
      int s = 0, parity = 0;  // stage and the phase of empty[s] that frees it
      for (int i = pre; i < nkb; ++i) {
        if (!MbarWait(empty0 + s * 8, parity)) {
          atomicExch(p.error_flag, kErrProducerWait);
          break;
        }
        const uint32_t dst = ring + s * kStageBytes, bar = full0 + s * 8;
        MbarExpectTx(bar, stage_tx);
        TmaLoad2D(dst, &w_map, (kb0 + i) * kBlockK, first_row0, bar, stream_policy);
        TmaLoad2D(dst + kHalfRows * 128, &w_map, (kb0 + i) * kBlockK, second_row0, bar, stream_policy);
        TmaLoad2D(dst + kWTileBytes, &x_map, (kb0 + i) * kBlockK, 0, bar, keep_policy);
        if (++s == stages) {
          s = 0;
          parity ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issue: four K=16 slices per k-block, accumulator stays in tensor memory
      const uint32_t idesc = InstrDesc(TP);
      bool ok = true;
      int s = 0, parity = 0;
      for (int i = 0; i < nkb; ++i) {
        if (!MbarWait(full0 + s * 8, parity)) {
          atomicExch(p.error_flag, kErrMmaWait);
          ok = false;
          break;
        }
        TcFenceAfter();
        if (i == 0) { RL_LSTAMP(3); }
        const uint64_t a_desc = TileDesc(ring + s * kStageBytes);
        const uint64_t b_desc = TileDesc(ring + s * kStageBytes + kWTileBytes);
#pragma unroll
        for (int k = 0; k < kBlockK / 16; ++k)
          Umma(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        UmmaCommit(empty0 + s * 8);
        if (++s == stages) {
          s = 0;
          parity ^= 1;
        }
      }
      RL_LSTAMP(4);
      if (ok) UmmaCommit(accum_bar);
    }
    __syncwarp();
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- accumulator to registers. Warp w reads tensor-memory lanes 32*(w%4)..+31 (accumulator rows);
  // warps 0-3 take the even 16-token column chunks, warps 4-7 the odd ones.
  const int row = (warp & 3) * 32 + lane;
  const int chunk0 = warp >> 2;
  bool good = MbarWait(accum_bar, 0);
  good = __all_sync(0xffffffffu, good);
  if (tid == 0) { RL_LSTAMP(5); }
  if (!good && lane == 0) atomicExch(p.error_flag, kErrAccumWait);
  TcFenceAfter();
  uint32_t raw[2][16];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int i = 0; i < 16; ++i) raw[j][i] = 0u;
  if (good) {
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
#pragma unroll
    for (int j = 0; j < 2; ++j)
      if ((chunk0 + 2 * j) * 16 < TP) TmemLoad16(taddr + (chunk0 + 2 * j) * 16, raw[j]);
    TmemWaitLoads(raw[0]);
    TmemWaitLoads(raw[1]);
  }
  float v[2][16];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int i = 0; i < 16; ++i) v[j][i] = __uint_as_float(raw[j][i]);
  TcFenceBefore();
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols)
                 : "memory");
  }
  if (tid == 0) { RL_LSTAMP(6); }
  // From here on every thread of every CTA runs the same barriers whatever `good` says: a CTA whose
  // wait gave up has raised the error flag and contributes zeros.
  // Every MMA has completed, so the ring is idle: it stages the tile, token-major, for the
  // cooperative output pass of an unsplit launch ([token][128 rows], FP16).

  if (p.splits == 1) {
    half* stage = reinterpret_cast<half*>(smem + ring_off);
    const bool silu = p.epilogue == kEpilogueSiluMul;
    const int col = tile * kTileRows + row;
    const float b = (!silu && p.bias && col < p.out_cols) ? __half2float(p.bias[col]) : 0.0f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int t = (chunk0 + 2 * j) * 16 + i;
        if (t < T) stage[t * kTileRows + row] = __float2half_rn(v[j][i] + b);
      }
    }
    __syncthreads();
    if (!silu) {
      // 16 chunks of 8 columns per token
      const int col_base = tile * kTileRows;
      for (int u = tid; u < T * 16; u += kThreads) {
        const int t = u >> 4, c0 = (u & 15) * 8;
        const half* src = stage + t * kTileRows + c0;
        half* dst = p.out + t * p.out_stride + col_base + c0;
        if (p.out_vec && col_base + c0 + 8 <= p.out_cols) {
          Stg16(dst, *reinterpret_cast<const uint4*>(src));
        } else {
          for (int e = 0; e < 8; ++e)
            if (col_base + c0 + e < p.out_cols) dst[e] = src[e];
        }
      }
    } else {
      // rows 0-63 hold `gate`, rows 64-127 `up`, both already rounded to FP16: 8 chunks of 8 columns per token
      const int col_base = tile * kHalfRows;
      for (int u = tid; u < T * 8; u += kThreads) {
        const int t = u >> 3, c0 = (u & 7) * 8;
        const uint4 g = *reinterpret_cast<const uint4*>(stage + t * kTileRows + c0);
        const uint4 up = *reinterpret_cast<const uint4*>(stage + t * kTileRows + kHalfRows + c0);
        const uint4 r = SiluMulChunk(g, up);
        half* dst = p.out + t * p.out_stride + col_base + c0;
        if (p.out_vec && col_base + c0 + 8 <= p.out_cols) {
          Stg16(dst, r);
        } else {
          const half* rh = reinterpret_cast<const half*>(&r);
          for (int e = 0; e < 8; ++e)
            if (col_base + c0 + e < p.out_cols) dst[e] = rh[e];
        }
      }
    }
    if (tid == 0) { RL_LSTAMP(8); }
    return;
  }

  // ---- split K: token t belongs to CTA t mod S of the cluster. Every CTA sends its partial sums of
  // token t into slice [its split][t / S] of the owner's receive area with asynchronous stores that
  // count bytes on the owner's mbarrier; the owner waits for all it expects (nobody waits for anything
  // else), adds the S slices of each of its tokens in split order and writes the row.
  const int S = p.splits, shift = p.split_shift;
  const int slots = (T + S - 1) >> shift;   // tokens per owner, at most
  const int my_tokens = T > split ? (T - split + S - 1) >> shift : 0;
  float* recv = reinterpret_cast<float*>(smem + kRecvOff);
  // The owner expects 512 bytes per token from each of the S CTAs (its own included).
  if (tid == 0) MbarExpectTx(recv_bar, my_tokens * S * kTileRows * 4);
  // Transpose through the idle ring: [token][row] so that four rows of one token leave as one 16-byte store.
  float* stage = reinterpret_cast<float*>(smem + ring_off);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int t = (chunk0 + 2 * j) * 16 + i;
      if (t < T) stage[t * kTileRows + row] = v[j][i];
    }
  }
  __syncthreads();
  ClusterWait();  // every CTA of the cluster has started and armed its barrier
  {
    const uint32_t recv_slice = SmemAddr(recv) + static_cast<uint32_t>(split * slots * kTileRows) * 4;
    for (int u = tid; u < T * 32; u += kThreads) {
      const int t = u >> 5, c0 = (u & 31) * 4;
      const int d = t & (S - 1), k = t >> shift;
      const float4 val = *reinterpret_cast<const float4*>(stage + t * kTileRows + c0);
      StAsyncPeerF32x4(PeerSmemAddr(recv_slice + static_cast<uint32_t>(k * kTileRows + c0) * 4, d),
                       PeerSmemAddr(recv_bar, d), val);
    }
  }
  if (!MbarWait(recv_bar, 0)) {
    if (tid == 0) atomicExch(p.error_flag, kErrSplitWait);
    // Peers' slices may still be on their way into this CTA's receive area: give them one more bounded chance
    // to land before the area is read (the launch is reported as failed either way) and, later, released. A
    // barrier over the cluster would make this airtight but would have to run in every launch, failed or not.
    MbarWait(recv_bar, 0);
  }
  if (tid == 0) { RL_LSTAMP(7); }
  if (p.epilogue == kEpilogueQkvRope) {
    // The tile is head `tile` of the fused QKV row (Q heads, then K heads, then V heads). A unit is four
    // columns d..d+3 of the low half of the head together with their rotation partners d+64..d+67.
    const int head = tile;
    const bool rotate = head < rope.q_heads + rope.kv_heads;
    for (int u = tid; u < my_tokens * 16; u += kThreads) {
      const int k = u >> 4, c0 = (u & 15) * 4;
      const int t = (k << shift) + split;
      const float* src = recv + k * kTileRows + c0;
      float4 lo4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi4 = lo4;
#pragma unroll
      for (int s2 = 0; s2 < kMaxSplits; ++s2) {
        if (s2 < S) {
          const float4 a = *reinterpret_cast<const float4*>(src + s2 * slots * kTileRows);
          const float4 b4 = *reinterpret_cast<const float4*>(src + s2 * slots * kTileRows + 64);
          lo4.x += a.x; lo4.y += a.y; lo4.z += a.z; lo4.w += a.w;
          hi4.x += b4.x; hi4.y += b4.y; hi4.z += b4.z; hi4.w += b4.w;
        }
      }
      const int col = head * kTileRows + c0;
      lo4.x += bias_lo[0]; lo4.y += bias_lo[1]; lo4.z += bias_lo[2]; lo4.w += bias_lo[3];   // zeros without a bias
      hi4.x += bias_hi[0]; hi4.y += bias_hi[1]; hi4.z += bias_hi[2]; hi4.w += bias_hi[3];
      // the projection's FP16 output ...
      uint32_t lo[2] = {AsU32(__floats2half2_rn(lo4.x, lo4.y)), AsU32(__floats2half2_rn(lo4.z, lo4.w))};
      uint32_t hi[2] = {AsU32(__floats2half2_rn(hi4.x, hi4.y)), AsU32(__floats2half2_rn(hi4.z, hi4.w))};
      const int pos = rope_table ? rope_pos[k] : rope.positions[t];
      if (rotate) {  // ... rotated in place for Q and K heads
        const float fpos = static_cast<float>(pos);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const half2 a = rope_table ? rope_cs[k * kMaxPairs + c0 + 2 * j] : RopeCosSin(fpos, rope.inv_freq.f[c0 + 2 * j]);
          const half2 b2 = rope_table ? rope_cs[k * kMaxPairs + c0 + 2 * j + 1]
                                      : RopeCosSin(fpos, rope.inv_freq.f[c0 + 2 * j + 1]);
          RotateWord(lo[j], hi[j], __lows2half2(a, b2), __highs2half2(a, b2));
        }
      }
      half* dst = p.out + t * p.out_stride + col;
      *reinterpret_cast<uint2*>(dst) = make_uint2(lo[0], lo[1]);
      *reinterpret_cast<uint2*>(dst + 64) = make_uint2(hi[0], hi[1]);
      if (head >= rope.q_heads) {  // K (rotated) and V heads also go to this token's slot of the paged pool
        const int kv = head >= rope.q_heads + rope.kv_heads ? 1 : 0;
        const int kv_head = head - rope.q_heads - kv * rope.kv_heads;
        const int64_t block = rope_table ? rope_block[k] : rope.tables[t * rope.table_row_stride + (pos >> kKvBlockShift)];
        const int slot = pos & (kKvBlock - 1);
        half* cell = rope.pool + (((block * 2 + kv) * rope.kv_heads + kv_head) * kKvBlock + slot) *
                                     static_cast<int64_t>(kTileRows) + c0;
        *reinterpret_cast<uint2*>(cell) = make_uint2(lo[0], lo[1]);
        *reinterpret_cast<uint2*>(cell + 64) = make_uint2(hi[0], hi[1]);
      }
    }
  } else {
    const int col_base = tile * kTileRows;
    for (int u = tid; u < my_tokens * 32; u += kThreads) {
      const int k = u >> 5, c0 = (u & 31) * 4;
      const int t = (k << shift) + split;
      const float* src = recv + k * kTileRows + c0;
      float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int s2 = 0; s2 < kMaxSplits; ++s2) {
        if (s2 < S) {
          const float4 part = *reinterpret_cast<const float4*>(src + s2 * slots * kTileRows);
          sum.x += part.x;
          sum.y += part.y;
          sum.z += part.z;
          sum.w += part.w;
        }
      }
      const int col = col_base + c0;
      float bias4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      if (p.bias) {
        for (int e = 0; e < 4; ++e)
          if (col + e < p.out_cols) bias4[e] = __half2float(p.bias[col + e]);
      }
      const half2 lo = __floats2half2_rn(sum.x + bias4[0], sum.y + bias4[1]);
      const half2 hi = __floats2half2_rn(sum.z + bias4[2], sum.w + bias4[3]);
      half* dst = p.out + t * p.out_stride + col;
      if (p.out_vec && col + 4 <= p.out_cols) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(AsU32(lo), AsU32(hi));
      } else {
        const half r[4] = {__low2half(lo), __high2half(lo), __low2half(hi), __high2half(hi)};
        for (int e = 0; e < 4; ++e)
          if (col + e < p.out_cols) dst[e] = r[e];
      }
    }
  }
  if (tid == 0) { RL_LSTAMP(8); }
}

// ------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceState {
  bool ready = false;
  void* workspace = nullptr;  // error flag
  int sm_count = 0;
};
constexpr int kMaxDevices = 64;
DeviceState g_state[kMaxDevices];
EncodeTiledFn g_encode = nullptr;
std::mutex g_mutex;
void* g_timeline = nullptr;  // diagnostics build only
int g_max_splits = kMaxSplits;
constexpr int kManyTileStages = 3;
int g_stages = 6;  // measured best inside the decode step (4: 20.2k, 6: 20.4k, 8: 20.35k tok/s)

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
                  "decode_linear: cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const DeviceFacts& facts = CurrentDeviceFacts();
  constexpr int kMostSmem = SmemBytes(kMaxStages, 1) > SmemBytes(kMaxStages - 1, 8) ? SmemBytes(kMaxStages, 1)
                                                                                    : SmemBytes(kMaxStages - 1, 8);
  if (facts.max_smem_optin < kMostSmem)
    return Fail(RL_E_WORKSPACE, "decode_linear: device offers %d B of shared memory per block, %d needed",
                facts.max_smem_optin, kMostSmem);
  cudaError_t e = cudaFuncSetAttribute(DecodeLinearKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMostSmem);
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "decode_linear: shared-memory opt-in: %s", cudaGetErrorString(e));
  e = cudaMalloc(&st.workspace, 256);
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "decode_linear: workspace: %s", cudaGetErrorString(e));
  e = cudaMemset(st.workspace, 0, 256);
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "decode_linear: workspace clear: %s", cudaGetErrorString(e));
  st.sm_count = facts.sm_count;
  st.ready = true;
  return RL_OK;
}

// A row-major [rows, cols] FP16 matrix with `row_stride` elements between rows, boxes of 64 columns
// (128 bytes, the swizzle span) by `box_rows` rows. Rows and columns past the extents read as zero.
int EncodeMatrixMap(const void* base, int64_t rows, int64_t cols, int64_t row_stride, int box_rows,
                    CUtensorMap* map) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Fail(RL_E_BAD_SHAPE, "decode_linear: tensor map encode failed (CUresult %d)", static_cast<int>(r));
  return RL_OK;
}

// CTAs per row tile along K (= cluster size: 1, 2, 4 or 8): the largest that keeps tiles x splits
// within the SM count, unless a smaller one already gives every split a single k-block.
int ChooseSplits(int tiles, int k_blocks, int sm_count) {
  int best = 1;
  for (int s = 2; s <= g_max_splits; s *= 2) {
    if (tiles * s > sm_count || s > k_blocks) break;
    best = s;
  }
  return best;
}

}  // namespace lin

int DecodeLinearInit() {
  lin::DeviceState* st;
  return lin::EnsureReady(&st);
}
}  // namespace rl

extern "C" int rl_decode_linear_health(int* flag_out) {
  using namespace rl;
  using namespace rl::lin;
  if (!flag_out) return Fail(RL_E_NULL_POINTER, "rl_decode_linear_health: null pointer");
  *flag_out = 0;
  DeviceState& st = g_state[CurrentDeviceIndex()];
  if (!st.ready) return RL_OK;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(flag_out, st.workspace, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && *flag_out != 0) e = cudaMemset(st.workspace, 0, sizeof(int));
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "rl_decode_linear_health: %s", cudaGetErrorString(e));
  return RL_OK;
}

#ifdef RL_LIN_TIMELINE
// Diagnostics build (-DRL_LIN_TIMELINE): per-CTA %globaltimer stamps of the last launch, 16 slots per CTA.
extern "C" int rl_debug_linear_timeline(unsigned long long* host_out, int max_entries) {
  cudaDeviceSynchronize();
  const int n = 128 * 2048 * 16;
  return cudaMemcpy(host_out, rl::lin::g_timeline, sizeof(unsigned long long) * (n < max_entries ? n : max_entries),
                    cudaMemcpyDeviceToHost);
}
extern "C" int rl_debug_linear_timeline_init(void) {
  const size_t bytes = sizeof(unsigned long long) * 128 * 2048 * 16;
  if (!rl::lin::g_timeline) cudaMalloc(&rl::lin::g_timeline, bytes);
  return cudaMemset(rl::lin::g_timeline, 0, bytes);
}
#endif

extern "C" int rl_decode_linear_set_stages(int stages) {
  using namespace rl;
  if (stages < 2 || stages > lin::kMaxStages)
    return Fail(RL_E_BAD_SHAPE, "rl_decode_linear_set_stages: 2..%d stages, got %d", lin::kMaxStages, stages);
  lin::g_stages = stages;
  return RL_OK;
}

extern "C" int rl_decode_linear_set_max_splits(int max_splits) {
  using namespace rl;
  if (max_splits != 1 && max_splits != 2 && max_splits != 4 && max_splits != 8)
    return Fail(RL_E_BAD_SHAPE, "rl_decode_linear_set_max_splits: 1, 2, 4 or 8, got %d", max_splits);
  lin::g_max_splits = max_splits;
  return RL_OK;
}

namespace rl {
namespace lin {

// Shared by the two entry points. `rope` is read by epilogue 2 only.
int Launch(void* out, int64_t out_row_stride, const void* x, int64_t x_row_stride, const void* weight,
           int64_t weight_row_stride, const void* bias, int num_tokens, int out_features, int in_features,
           int epilogue, const RopeArgs& rope, void* stream, int* splits_out) {
  if (!out || !x || !weight) return Fail(RL_E_NULL_POINTER, "decode_linear: null device pointer");
  if (num_tokens > kMaxTokens)
    return Fail(RL_E_TOO_LARGE, "decode_linear: at most %d token rows per call, got %d", kMaxTokens, num_tokens);
  if (in_features < 8 || (in_features & 7) || (x_row_stride & 7) || (weight_row_stride & 7) || !Aligned16(x) ||
      !Aligned16(weight))
    return Fail(RL_E_BAD_SHAPE, "decode_linear: x and weight rows must be 16-byte aligned, in_features a multiple of 8");
  if (x_row_stride < in_features || weight_row_stride < in_features || out_row_stride < out_features)
    return Fail(RL_E_BAD_SHAPE, "decode_linear: row stride smaller than the row");
  DeviceState* st;
  int rc;
  if ((rc = EnsureReady(&st)) != RL_OK) return rc;

  const int weight_rows = epilogue == kEpilogueSiluMul ? 2 * out_features : out_features;
  const int rows_per_tile = epilogue == kEpilogueSiluMul ? kHalfRows : kTileRows;
  const int tiles = (out_features + rows_per_tile - 1) / rows_per_tile;
  Params p;
  p.out = static_cast<half*>(out);
  p.out_stride = out_row_stride;
  p.bias = static_cast<const half*>(bias);
  p.tokens = num_tokens;
  p.tokens_padded = (num_tokens + 15) & ~15;
  p.out_cols = out_features;
  p.up_row_offset = out_features;
  p.k_blocks = (in_features + kBlockK - 1) / kBlockK;
  p.splits = epilogue == kEpilogueSiluMul ? 1 : ChooseSplits(tiles, p.k_blocks, st->sm_count);
  if (splits_out) *splits_out = p.splits;
  if (epilogue == kEpilogueQkvRope && p.splits == 1) return RL_OK;  // the caller takes the unfused route
  const int longest_split = (p.k_blocks + p.splits - 1) / p.splits;
  p.stages = longest_split < g_stages ? (longest_split < 2 ? 2 : longest_split) : g_stages;
  if (p.splits > 1 && p.stages > kMaxStages - 1) p.stages = kMaxStages - 1;  // room for the receive area
  // Many more row tiles than SMs (the vocabulary projection: 1187 tiles): a short ring lets three CTAs share
  // an SM, so one CTA's prologue and epilogue hide behind the others' streams (64 x 151936 x 1536: 100.9 us
  // with 6 stages, 84.4 with 4, 79.0 with 3, all with evict-first weight tiles; the library GEMM takes 82.1).
  // Such a launch also takes its weights at normal L2 priority (82.3 us alone): the sweep of some hundred MB
  // through L2 retires the dead lines of the step (logits, activations, freshly written K/V) once per step,
  // which inside the decode step measured 24 us per step better than leaving them for the following launches
  // to push out.
  const bool many_tiles = p.splits == 1 && tiles >= 3 * st->sm_count;
  if (many_tiles && p.stages > kManyTileStages) p.stages = kManyTileStages;
  p.weights_sweep_l2 = many_tiles ? 1 : 0;
  p.split_shift = p.splits == 8 ? 3 : p.splits == 4 ? 2 : p.splits == 2 ? 1 : 0;
  p.epilogue = epilogue;
  p.tmem_cols = p.tokens_padded <= 32 ? 32 : 64;
  p.out_vec = (Aligned16(out) && (out_row_stride & 7) == 0) ? 1 : 0;
  p.error_flag = static_cast<int*>(st->workspace);
  p.timeline = nullptr;
#ifdef RL_LIN_TIMELINE
  {  // one 2048 x 16 region per launch, 128 regions in rotation
    static int launch_seq = 0;
    p.timeline = g_timeline ? static_cast<unsigned long long*>(g_timeline) + static_cast<size_t>(launch_seq++ % 128) * 2048 * 16
                            : nullptr;
  }
#endif
  CUtensorMap w_map, x_map;
  if ((rc = EncodeMatrixMap(weight, weight_rows, in_features, weight_row_stride, kHalfRows, &w_map)) != RL_OK) return rc;
  if ((rc = EncodeMatrixMap(x, num_tokens, in_features, x_row_stride, p.tokens_padded, &x_map)) != RL_OK) return rc;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.splits);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = SmemBytes(p.stages, p.splits);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_launch_overlap ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = p.splits;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, DecodeLinearKernel, p, w_map, x_map, rope);
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "decode_linear: %s", cudaGetErrorString(e));
  return LaunchStatus("decode_linear");
}

}  // namespace lin
}  // namespace rl

extern "C" int rl_launch_decode_linear(void* out, int64_t out_row_stride, const void* x, int64_t x_row_stride,
                                       const void* weight, int64_t weight_row_stride, const void* bias,
                                       int32_t num_tokens, int32_t out_features, int32_t in_features,
                                       int32_t epilogue, void* stream) {
  using namespace rl;
  using namespace rl::lin;
  if (num_tokens <= 0 || out_features <= 0) return RL_OK;
  if (epilogue != kEpilogueBias && epilogue != kEpilogueSiluMul)
    return Fail(RL_E_BAD_SHAPE, "decode_linear: epilogue must be 0 (bias) or 1 (silu-mul)");
  if (epilogue == kEpilogueSiluMul && bias)
    return Fail(RL_E_BAD_SHAPE, "decode_linear: the silu-mul epilogue takes no bias");
  static const RopeArgs no_rope = {};
  return Launch(out, out_row_stride, x, x_row_stride, weight, weight_row_stride, bias, num_tokens, out_features,
                in_features, epilogue, no_rope, stream, nullptr);
}

extern "C" int rl_launch_qkv_rope_kv_scatter(void* qkv, int64_t qkv_row_stride, const void* x, int64_t x_row_stride,
                                             const void* weight, int64_t weight_row_stride, const void* bias,
                                             int32_t num_tokens, int32_t in_features, void* kv_pool_layer,
                                             const int32_t* block_tables, int64_t block_table_row_stride,
                                             const int32_t* positions, int32_t num_q_heads, int32_t num_kv_heads,
                                             int32_t head_dim, float rope_theta, void* stream) {
  using namespace rl;
  using namespace rl::lin;
  if (num_tokens <= 0) return RL_OK;
  if (!kv_pool_layer || !block_tables || !positions)
    return Fail(RL_E_NULL_POINTER, "qkv_rope_kv_scatter: null device pointer");
  if (head_dim != kTileRows || num_q_heads < 1 || num_kv_heads < 1 || !(rope_theta > 0.0f))
    return Fail(RL_E_BAD_SHAPE, "qkv_rope_kv_scatter: head_dim must be 128, heads >= 1, theta > 0");
  if (!Aligned16(qkv) || (qkv_row_stride & 7) || !Aligned16(kv_pool_layer))
    return Fail(RL_E_BAD_SHAPE, "qkv_rope_kv_scatter: qkv rows and the pool slice must be 16-byte aligned");
  const int out_features = (num_q_heads + 2 * num_kv_heads) * head_dim;
  RopeArgs rope;
  rope.positions = positions;
  rope.tables = block_tables;
  rope.table_row_stride = block_table_row_stride;
  rope.pool = static_cast<half*>(kv_pool_layer);
  rope.q_heads = num_q_heads;
  rope.kv_heads = num_kv_heads;
  rope.inv_freq = RopeTableFor(rope_theta, head_dim);
  int splits = 0;
  int rc = Launch(qkv, qkv_row_stride, x, x_row_stride, weight, weight_row_stride, bias, num_tokens, out_features,
                  in_features, kEpilogueQkvRope, rope, stream, &splits);
  if (rc != RL_OK || splits > 1) return rc;
  // A shape this kernel does not split along K (few k-blocks, or splitting capped at 1): the same
  // result in two launches.
  static const RopeArgs no_rope = {};
  rc = Launch(qkv, qkv_row_stride, x, x_row_stride, weight, weight_row_stride, bias, num_tokens, out_features,
              in_features, kEpilogueBias, no_rope, stream, nullptr);
  if (rc != RL_OK) return rc;
  half* q = static_cast<half*>(qkv);
  return rl_launch_rope_kv_scatter(q, q + num_q_heads * head_dim, q + (num_q_heads + num_kv_heads) * head_dim,
                                   qkv_row_stride, qkv_row_stride, qkv_row_stride, kv_pool_layer, block_tables,
                                   block_table_row_stride, positions, num_tokens, num_q_heads, num_kv_heads,
                                   head_dim, rope_theta, stream);
}
