// Fused paged prefill attention for sm_100a (B200): one prompt chunk of one sequence attends causally
// to everything cached for that sequence - earlier chunks and itself - straight out of the paged pool.
//
// The reference ingests a chunk through a composite (src/core/model_executor.cpp:1219-1290): LaunchKvGather
// copies the sequence's pages into dense K / V staging, cuBLASLt writes FP32 scores [heads, chunk, ctx] to
// global memory, LaunchPrefillSoftmax rewrites them as FP16 probabilities, cuBLASLt multiplies by V; its
// design notes name a fused kernel as the follow-up (docs/DESIGN.md:872-876 in its tree). This is that kernel: the
// same function - scores q.k * scale in FP32 from FP16 operands, causal SELECT masking (key position <=
// query position; slots past the context never reach a result), softmax with FP32 statistics,
// probabilities rounded to FP16 for the P.V product, FP32 accumulation, one FP16 rounding of acc / l -
// with nothing but Q, the pages and the output ever touching global memory.
//
// Mapping. One CTA per (128-row query tile, query head) - or per run of key blocks of such a pair when the launch
// would otherwise leave SMs idle (the run length is chosen per launch): the runs' unnormalised outputs meet in a
// scratch area and a small second kernel, launched behind this one, combines them in run
// order, so long contexts fill the machine and the result does not depend on timing. Ten warps.
//  * Warp 9 requests every tile by TMA (copies spread over its lanes), warp 8 issues every tcgen05.mma: table
//    reads and copy requests never sit between two products. Q tile and K/V
//    blocks of 128 keys (8 pages) arrive with the 128-byte swizzle. A page tile of the pool is
//    [16 tokens][128 dims] = 4 KiB and arrives - K and V alike - as ONE copy through a 5-D view of the pool
//    that lands it as [token group of 8][dim half][8 tokens][128 B] at 4 KiB * page: swizzle atoms of 8 rows x 128 B,
//    the two dim halves 1 KiB apart, the 8-token groups 2 KiB apart. Eight pages are then the K-major operand
//    tile of an N = 128 product for Q.K^T (per dim half: sixteen 8-key groups at a stride of 2 KiB), and each page
//    is one K = 16 slice of the MN-major operand of P.V. (The TMA unit is paid per copy - 16 per block this way,
//    24 or 32 with K in halves - and the tensor pipe per instruction.)
//    Block-table indirection costs nothing but the copy's coordinate. K and V blocks are double-buffered;
//    the six query heads of a KV group and all query tiles re-read the same pages from L2.
//  * S = Q.K^T: M = 128 query rows, N = 128 keys, K = 16 dims x 8, both operands K-major in shared memory,
//    FP32 accumulator in tensor memory. Two S buffers (columns 0-127, 128-255): the product of
//    block j+2 is issued as soon as the softmax of block j has released its buffer - ahead of P_j.V_j, because
//    the softmax warps wait for scores and never for the output - so the tensor pipe runs under the softmax of
//    block j+1.
//  * Softmax: warps 0-7, two threads per query row (keys 0-63 and 64-127 of the block; a warp may only touch
//    its own quarter of the tensor-memory lanes). Each thread reads its half row of S from tensor memory once
//    (tcgen05.ld 32x32b) and writes P = exp2(s * scale - reference) as FP16 pairs into tensor memory
//    (tcgen05.st, two P buffers of 64 columns), from where the P.V product takes its A operand: P never
//    touches shared memory. The sweep is bound by instruction issue, so two scores are scaled per
//    fma.rn.f32x2 and two probabilities summed per add.rn.f32x2. The reference is the row's maximum of the
//    FIRST block; later blocks are written against it without looking at their maximum, and only a half row
//    whose probabilities sum to 2^15 or more (a score more than 2^9 above the reference) sends its two warps
//    to the full treatment: exact maximum exchanged through shared memory, reference moved, row sum and running
//    output (a read-modify-write of the row in tensor memory) rescaled, block written again. Numerator and
//    denominator always share one reference, so the result does not depend on when it moves.
//  * O += P.V: A = P (in tensor memory) and B = V as it lies in the pool - [key][dim], i.e. MN-major: atoms of
//    8 keys x 64 dims, 2 KiB between key groups, 1 KiB between the dim halves, one page per K = 16 slice -
//    accumulated over all blocks in tensor-memory columns 256-383; read once at the end, divided by the row
//    sum, rounded once.
// Every mbarrier wait is bounded and reports through rl_prefill_attention_health.
#include <cuda.h>

#include <algorithm>
#include <functional>
#include <mutex>
#include <vector>

#include "tc_ptx.cuh"

namespace rl {
namespace pfa {

using namespace rl::tc;

constexpr int kHeadDim = 128;
constexpr int kBM = 128;                 // query rows per CTA
constexpr int kBN = 128;                 // keys per block (8 pages)
constexpr int kRowSplit = 2;             // softmax threads per query row (4 - sixteen softmax warps, 96 registers - measured 6 % slower)
constexpr int kSoftmaxThreads = kBM * kRowSplit;   // warps 0-7: two threads per query row
constexpr int kMmaWarp = kSoftmaxThreads / 32, kLoadWarp = kMmaWarp + 1;
constexpr int kThreads = kSoftmaxThreads + 64;   // + the MMA-issue warp and the loader warp
constexpr int kKeysPerThread = kBN / kRowSplit;        // scores of a block one softmax thread owns
constexpr int kScoreChunks = kKeysPerThread / 16;      // in tensor-memory loads of 16 columns
constexpr int kDimsPerThread = kHeadDim / kRowSplit;   // output dims one softmax thread owns at the end
constexpr int kDimChunks = kDimsPerThread / 16;
static_assert(kDimChunks == kScoreChunks, "the registers that held a block's scores take the output row at the end");
constexpr int kPagesPerBlock = kBN / kKvBlock;
constexpr int kRegionBytes = 128 * 128;  // [128 rows][64 halves], 128-byte swizzle
constexpr int kTileBytes = 2 * kRegionBytes;   // two 64-wide halves
constexpr int kQOff = 0;
constexpr int kKOff = kQOff + kTileBytes;          // 2 buffers
constexpr int kVOff = kKOff + 2 * kTileBytes;      // 2 buffers
constexpr int kBarOff = kVOff + 2 * kTileBytes;    // mbarriers, tmem slot
constexpr int kXOff = kBarOff + 128;               // row maxima [2 iterations][threads of a row][128] (row sums reuse one half at the end)
constexpr int kXFloats = kRowSplit * kBM;          // one iteration's exchange buffer
constexpr int kSmemNeeded = kXOff + 2 * kXFloats * 4;   // from a 1024-byte aligned base
constexpr int kSmemBytes = kSmemNeeded + 1024;     // + slack for aligning the base
static_assert(kSmemBytes <= 227 * 1024, "prefill attention shared memory exceeds the per-CTA limit");
constexpr int kTmemCols = 512;           // S: columns 0-127 and 128-255, O: 256-383, P (FP16 pairs): 384-447 and 448-511
constexpr int kTmemP = 384;
constexpr float kRescaleThreshold = 8.0f;   // log2: when a block's maximum is looked at, the reference moves if it lies more than this above it
constexpr float kOverflowSum = 32768.0f;    // a half row of P that sums to 2^15 or more may hold a value near FP16's largest: look at the maximum
// A run's record: o unnormalised as [dim / 4][row][4] - the 32 rows of a warp write, and later read, 512 contiguous
// bytes per instruction - then m[128], l[128].
constexpr int kPartialFloats = kBM * kHeadDim + 2 * kBM;

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
  int n_tiles;        // query tiles of the chunk
  int split_blocks;   // longest run of key blocks one CTA takes
  float* partials;    // one record of kPartialFloats per (head, work item) for pairs cut across CTAs
};

// Where a page lands in a K or V block buffer: [token group of 8][dim half][8 tokens][128 B].
constexpr int kHalfStride = 1024;    // between the two 64-dim halves of an 8-token group
constexpr int kGroupStride = 2048;   // between the two 8-token groups of a page
// V page as the B operand of P.V, stored [key][dim] (MN-major, 128-byte swizzle): atoms of 8 key rows x 128 B;
// leading byte offset = between the 64-dim halves (N runs over dims), stride byte offset = between the 8-key
// groups (K runs over keys).
__device__ __forceinline__ uint64_t PageDescMn(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(kHalfStride >> 4) << 16) |
         (static_cast<uint64_t>(kGroupStride >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// K block as the B operand of Q.K^T (K-major, 128-byte swizzle), one dim half: 8-key groups 2 KiB apart.
__device__ __forceinline__ uint64_t KeyBlockDesc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) |
         (static_cast<uint64_t>(kGroupStride >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint32_t InstrDescBMn(int n) { return InstrDesc(n) | (1u << 16); }

// One (block, kv, head) page tile in one copy of 4 KiB: the pool seen as [tile][token group][dim half][8 tokens]
// [64 halves], 128-byte swizzled. Into this CTA's own shared memory; no multicast.
__device__ __forceinline__ void TmaLoadPage(uint32_t dst, const CUtensorMap* map, int tile, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %2, %2, %2, %3}], [%4], %5;" ::"r"(dst),
      "l"(map), "r"(0), "r"(tile), "r"(bar), "l"(policy)
      : "memory");
}
constexpr int kPageTileBytes = kKvBlock * kHeadDim * 2;   // 4096
__device__ __forceinline__ void MbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ float Ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two FP32 lanes in one 64-bit register for the packed FP32 pipe (sm_100): one issue slot scales two scores,
// another adds two probabilities to the two running sums. Each lane is the ordinary IEEE operation.
__device__ __forceinline__ uint64_t Pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float2 Unpack2(uint64_t v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}
__device__ __forceinline__ uint64_t Fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t Add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// max(a, b, c) in one instruction (sm_100): halves the comparisons of the maximum pass.
__device__ __forceinline__ float Max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 16 accumulator columns of this thread's lane back into tensor memory.
__device__ __forceinline__ void TmemStore16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void TmemStore8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
// D (+)= A.B with A in tensor memory (row i in lane i, two FP16 per 32-bit column along K) and B in shared memory.
// Called by all 32 lanes of a converged warp with identical arguments; one elected lane issues (see UmmaElected).
__device__ __forceinline__ void UmmaTsElected(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void TmemWaitStores() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void SoftmaxBarrier() { asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory"); }
// The two warps that share 32 query rows (keys 0-63 and 64-127 of a block) meet on a barrier of their own:
// a plain rendezvous, and one that also tells both whether any of their 64 threads raised `pred`.
__device__ __forceinline__ void PairBarrier(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(32 * kRowSplit) : "memory"); }
__device__ __forceinline__ bool PairAny(int id, bool pred) {
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %2, 0;\n\t"
      "bar.red.or.pred p, %1, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(any)
      : "r"(id), "r"(static_cast<uint32_t>(pred)), "n"(32 * kRowSplit)
      : "memory");
  return any != 0;
}

__global__ void __launch_bounds__(kThreads, 1)
PagedPrefillAttentionKernel(const Params p, const __grid_constant__ CUtensorMap q_map,
                            const __grid_constant__ CUtensorMap page_map) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  // The tiles fill all but a few hundred bytes of what a CTA may have: should the base ever need more
  // alignment padding than that, report it instead of running past the end.
  if (static_cast<int>(smem - smem_raw) + kSmemNeeded > kSmemBytes) {
    if (threadIdx.x == 0) atomicExch(p.error_flag, 3);
    return;
  }
  const uint32_t s_q = SmemAddr(smem + kQOff), s_k = SmemAddr(smem + kKOff), s_v = SmemAddr(smem + kVOff);
  const uint32_t bars = SmemAddr(smem + kBarOff);
  // Every barrier that more than one phase passes through belongs to ONE buffer (index = block & 1): a waiter
  // names a phase by its parity alone, which is only safe while the barrier cannot run two phases ahead of
  // it - and the next phase of a buffer's barrier always needs something this waiter itself provides.
  const uint32_t bar_q = bars, bar_k0 = bars + 8, bar_v0 = bars + 24, bar_s0 = bars + 40, bar_p0 = bars + 56,
                 bar_o0 = bars + 72, bar_done = bars + 88;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kBarOff + 96);
  float* xmax = reinterpret_cast<float*>(smem + kXOff);          // [2][kRowSplit][128]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Work items of a head, long tiles first (the last query tile of the chunk attends to the most keys): a tile
  // whose keys fill more than `split_blocks` blocks is cut into equal runs of blocks, one CTA each; this CTA is
  // item blockIdx.y = run `split` of `nsplit` of tile `tile_q`, blocks jb0 .. jb0 + nblk - 1 of that tile. The head
  // is the fast grid index: CTAs start in the order item 0 of every head, item 1 of every head, ... - longest
  // items first over the WHOLE launch, which is what lets the short ones level the SMs at the end - and the heads
  // of a KV group read the same pages at the same time.
  const int head = blockIdx.x;
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int kv_len = p.chunk_start + p.chunk_len;

  // Barriers and tensor memory first: both take a while and need nothing of what follows.
  if (tid == 0) {
    MbarInit(bar_q, 1);
    for (int i = 0; i < 2; ++i) {
      MbarInit(bar_k0 + 8 * i, 1);
      MbarInit(bar_v0 + 8 * i, 1);
      MbarInit(bar_s0 + 8 * i, 1);
      MbarInit(bar_p0 + 8 * i, kSoftmaxThreads);
      MbarInit(bar_o0 + 8 * i, 1);
    }
    MbarInit(bar_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     SmemAddr(const_cast<uint32_t*>(tmem_slot))),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // Which item: every warp works it out for itself, 32 tiles at a time - lane i takes the i-th tile from the end,
  // a shuffle scan sums the runs before it, a ballot finds the tile that holds the item. (One tile after the other,
  // with its integer division, this took a microsecond of every CTA's life at 16 tiles.)
  int tile_q = 0, split = 0, nsplit = 1, tile_blocks = 1;
  {
    const int item = blockIdx.y;
    int before = 0;                       // runs of the tiles already passed
    bool found = false;
    for (int base = 0; base < p.n_tiles && !found; base += 32) {
      const int t = p.n_tiles - 1 - base - lane;
      const int nb = t >= 0 ? (min(p.chunk_start + (t + 1) * kBM, kv_len) - 1) / kBN + 1 : 0;
      const int ns = t >= 0 ? (nb + p.split_blocks - 1) / p.split_blocks : 0;
      int upto = ns;                      // inclusive scan over the lanes
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, upto, d);
        if (lane >= d) upto += v;
      }
      const unsigned holds = __ballot_sync(0xffffffffu, t >= 0 && item < before + upto);
      if (holds) {
        const int src = __ffs(holds) - 1;
        tile_q = __shfl_sync(0xffffffffu, t, src);
        nsplit = __shfl_sync(0xffffffffu, ns, src);
        tile_blocks = __shfl_sync(0xffffffffu, nb, src);
        split = item - (before + __shfl_sync(0xffffffffu, upto - ns, src));
        found = true;
      }
      before += __shfl_sync(0xffffffffu, upto, 31);
    }
    if (!found) {                         // an item past the last one: the launcher never asks for it
      tile_q = 0;
      tile_blocks = (min(p.chunk_start + kBM, kv_len) - 1) / kBN + 1;
      nsplit = 1;
      split = 0;
    }
  }
  const int row0 = tile_q * kBM;
  const int jb0 = split * tile_blocks / nsplit;
  const int nblk = (split + 1) * tile_blocks / nsplit - jb0;          // blocks of THIS item, indexed 0 .. nblk - 1 below

  // The loader's first table reads (lane l < 8 serves page l of a block) are under way before the CTA's barrier.
  auto table_entry = [&](int j) {
    const int page = (jb0 + j) * kPagesPerBlock + lane;
    return (lane < kPagesPerBlock && j < nblk && page < p.max_blocks) ? __ldg(p.table_row + page) : 0;   // past the table: the dummy block
  };
  int blk = 0, blk_next = 0, blk_next2 = 0;
  if (warp == kLoadWarp) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&q_map) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&page_map) : "memory");
    }
    blk = table_entry(0);
    blk_next = table_entry(1);
    blk_next2 = table_entry(2);
  }
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * kBN;

  bool ok = true;
  auto wait = [&](uint32_t bar, int parity) {
    if (ok && !MbarWait(bar, parity)) {
      ok = false;
      atomicExch(p.error_flag, 2);
    }
  };

  if (warp == kLoadWarp) {
    // ------------------------------------------------------------ loader: every TMA request
    // A block is 8 copies of 4 KiB for K and 8 for V, one per page, spread over the lanes. The block id of a page
    // serves K and V alike and is read from the table two blocks ahead of its use.
    const uint64_t keep = L2PolicyEvictLast(), normal = L2PolicyEvictNormal();
    auto load_k = [&](int j, int block) {   // K block j into buffer j & 1, page l at 4 KiB * l
      const uint32_t base = s_k + (j & 1) * kTileBytes, bar = bar_k0 + 8 * (j & 1);
      if (lane == 0) MbarExpectTx(bar, kTileBytes);
      __syncwarp();
      if (lane < kPagesPerBlock)
        TmaLoadPage(base + lane * kPageTileBytes, &page_map, (block * 2 + 0) * p.kv_heads + kv_head, bar, keep);
    };
    auto load_v = [&](int j, int block) {   // V block j likewise
      const uint32_t base = s_v + (j & 1) * kTileBytes, bar = bar_v0 + 8 * (j & 1);
      if (lane == 0) MbarExpectTx(bar, kTileBytes);
      __syncwarp();
      if (lane < kPagesPerBlock)
        TmaLoadPage(base + lane * kPageTileBytes, &page_map, (block * 2 + 1) * p.kv_heads + kv_head, bar, keep);
    };
    if (lane == 0) {
      MbarExpectTx(bar_q, kTileBytes);
      TmaLoad2D(s_q, &q_map, head * kHeadDim, row0, bar_q, normal);
      TmaLoad2D(s_q + kRegionBytes, &q_map, head * kHeadDim + 64, row0, bar_q, normal);
    }
    // K runs one block ahead of V: K_{t+1}'s buffer is free as soon as Q.K_{t-1}^T has completed, long before
    // P_{t-2}.V_{t-2} - which V_t's buffer waits for - so no K request ever queues behind a V wait.
    load_k(0, blk);
    load_v(0, blk);
    if (nblk > 1) load_k(1, blk_next);
#pragma unroll 1
    for (int t = 1; t < nblk; ++t) {
      blk = blk_next;                  // block t
      blk_next = blk_next2;            // block t + 1
      blk_next2 = table_entry(t + 2);
      if (t + 1 < nblk) {
        wait(bar_s0 + 8 * ((t + 1) & 1), ((t - 1) >> 1) & 1);       // K buffer: free once Q.K_{t-1}^T has completed
        load_k(t + 1, blk_next);
      }
      if (t >= 2) wait(bar_o0 + 8 * (t & 1), ((t - 2) >> 1) & 1);   // V buffer: free once P_{t-2}.V_{t-2} has completed
      load_v(t, blk);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issue
    // The whole warp walks the schedule converged and every product is issued by one elected lane: the
    // descriptors depend on the block's buffer, and computed inside a one-lane branch they cost the issue
    // ~20 cycles more per product than the tensor pipe needs to execute it.
    const uint32_t idesc_kk = InstrDesc(kBN), idesc_mn = InstrDescBMn(kHeadDim);
    bool good = true;   // warp-uniform: every lane waits on the same barrier and votes
    auto wait_all = [&](uint32_t bar, int parity) {
      if (good) {
        good = __all_sync(0xffffffffu, MbarWait(bar, parity));
        if (!good && lane == 0) atomicExch(p.error_flag, 2);
      }
    };
    // S[j & 1] = Q.K_j^T
    auto issue_qk = [&](int j) {
      const uint32_t kb = s_k + (j & 1) * kTileBytes;
      const uint32_t d = tmem_base + (j & 1) * kBN;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint64_t a = TileDesc(s_q + h * kRegionBytes), b = KeyBlockDesc(kb + h * kHalfStride);
#pragma unroll
        for (int k = 0; k < 4; ++k) UmmaElected(d, a + 2 * k, b + 2 * k, idesc_kk, (h | k) ? 1u : 0u);
      }
      UmmaCommitElected(bar_s0 + 8 * (j & 1));
    };
    // O += P_j.V_j: K = 16 keys = one page per instruction; V read MN-major where it landed.
    auto issue_pv = [&](int j) {
      const uint32_t vb = s_v + (j & 1) * kTileBytes;
      const uint32_t pt = tmem_base + kTmemP + (j & 1) * (kBN / 2);
#pragma unroll
      for (int k = 0; k < kPagesPerBlock; ++k) {   // 16 keys = 8 columns of P = one page of V per instruction
        UmmaTsElected(tmem_o, pt + 8 * k, PageDescMn(vb + k * kPageTileBytes), idesc_mn, (j | k) ? 1u : 0u);
      }
      UmmaCommitElected(bar_o0 + 8 * (j & 1));
    };
    wait_all(bar_q, 0);
    wait_all(bar_k0, 0);
    TcFenceAfter();
    if (good) issue_qk(0);
    if (nblk > 1) {
      wait_all(bar_k0 + 8, 0);
      if (good) issue_qk(1);
    }
#pragma unroll 1
    for (int j = 0; j < nblk; ++j) {
      const int buf = j & 1, par = (j >> 1) & 1;
      // Q.K_{j+2}^T FIRST: the softmax warps wait for scores, never for the output. (With P_j.V_j first, S_{j+1} became
      // visible ~1700 cycles after P_{j-1} was reported - two groups of eight products and the latencies around
      // them - while the softmax of block j had finished after ~1500 and stood waiting 220-350 cycles every block.)
      wait_all(bar_p0 + 8 * buf, par);                 // P_j written, S[buf] read out
      TcFenceAfter();
      if (j + 2 < nblk) {
        wait_all(bar_k0 + 8 * buf, ((j + 2) >> 1) & 1);
        if (good) issue_qk(j + 2);
      }
      wait_all(bar_v0 + 8 * buf, par);                 // V_j landed
      if (good) issue_pv(j);
    }
    // One-shot barrier for the readers of the finished output.
    if (good) UmmaCommitElected(bar_done);
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax: two threads per query row
    const int row = (warp & 3) * 32 + lane;          // the tensor-memory lane = query row of the tile
    const int hw = warp >> 2;                        // which 64 keys of a block (and which 64 output dims at the end)
    const int my_pos = min(p.chunk_start + row0 + row, kv_len - 1);   // rows past the chunk are computed, never stored
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float m_ref = -INFINITY, l = 0.0f;
    // This thread's 64 scores of a block are fetched from tensor memory once, all four loads in flight together,
    // and kept in registers for both passes. The fetch for block j+1 is made at the END of block j, before this
    // thread reports P_j: when all have reported P_j, both S buffers have been read out, and the MMA warp writes
    // S_{j+2} over S_j (and, one report later, S_{j+3} over S_{j+1}).
    uint32_t raw[kScoreChunks][16];
    auto fetch_scores = [&](int j) {
      wait(bar_s0 + 8 * (j & 1), (j >> 1) & 1);
      TcFenceAfter();
      const uint32_t s_addr = tmem_base + (j & 1) * kBN + hw * kKeysPerThread + lane_addr;
#pragma unroll
      for (int c = 0; c < kScoreChunks; ++c) TmemLoad16(s_addr + c * 16, raw[c]);
#pragma unroll
      for (int c = 0; c < kScoreChunks; ++c) TmemWaitLoads(raw[c]);
    };
    fetch_scores(0);

#pragma unroll 1
    for (int j = 0; j < nblk; ++j) {
      const int buf = j & 1;
      const int key0 = (jb0 + j) * kBN + hw * kKeysPerThread;
      const bool diagonal = (jb0 + j) * kBN + kBN - 1 > p.chunk_start + row0;   // some row of the tile is masked inside this block
      const uint32_t p_addr = tmem_base + kTmemP + buf * (kBN / 2) + lane_addr + (kKeysPerThread / 2) * hw;
      const int pair_bar = 2 + (warp & 3);
      // The raw maximum of this thread's 64 scores (raw: the scale is positive), masked keys left out.
      auto row_max = [&]() {
        float mx = -INFINITY;
        if (diagonal) {
#pragma unroll
          for (int c = 0; c < kScoreChunks; ++c)
#pragma unroll
            for (int i = 0; i < 16; ++i)
              mx = fmaxf(mx, key0 + c * 16 + i <= my_pos ? __uint_as_float(raw[c][i]) : -INFINITY);
        } else {
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, two scores per instruction
#pragma unroll
          for (int c = 0; c < kScoreChunks; ++c)
#pragma unroll
            for (int i = 0; i < 16; i += 2)
              m4[(i >> 1) & 3] = Max3(m4[(i >> 1) & 3], __uint_as_float(raw[c][i]), __uint_as_float(raw[c][i + 1]));
          mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
        return mx;
      };
      // Probabilities against the reference, FP16, into tensor memory in key order (two per column: keys
      // 64 * hw + 16 * c .. + 15 of this row - the A operand of P.V); returns their FP32 sum.
      auto write_probabilities = [&](float ref) {
        const uint64_t scale2 = Pack2(p.scale_log2e, p.scale_log2e), neg_ref2 = Pack2(-ref, -ref);
        uint64_t sums = Pack2(0.0f, 0.0f);   // even keys, odd keys
#pragma unroll
        for (int c = 0; c < kScoreChunks; ++c) {
          uint32_t packed[8];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float2 x = Unpack2(Fma2(Pack2(__uint_as_float(raw[c][i]), __uint_as_float(raw[c][i + 1])), scale2, neg_ref2));
            float p0 = Ex2(x.x);
            float p1 = Ex2(x.y);
            if (diagonal) {
              p0 = key0 + c * 16 + i <= my_pos ? p0 : 0.0f;
              p1 = key0 + c * 16 + i + 1 <= my_pos ? p1 : 0.0f;
            }
            sums = Add2(sums, Pack2(p0, p1));
            packed[i >> 1] = AsU32(__floats2half2_rn(p0, p1));
          }
          TmemStore8(p_addr + 8 * c, packed);
        }
        const float2 sum01 = Unpack2(sums);
        return sum01.x + sum01.y;
      };
      // After the first block the row's maximum is not looked at block by block: the probabilities are written
      // against the running reference right away, and only a half row whose sum reaches 2^15 - some score lies more
      // than 2^9 above the reference, so a value may come near FP16's largest - sends its two warps (one barrier
      // that also carries the vote) to the full treatment: the exact maximum, exchanged with the partner; the
      // reference moved; row sum and running output rescaled; the block written again. Numerator and denominator
      // always share one reference, so the result does not depend on when it moves; P stays below 2^16.
      float sum = 0.0f;
      bool settle = true;
      // P_j goes where P_{j-2} was: that product must have completed. (Scores no longer imply it: Q.K_j^T was issued
      // ahead of P_{j-2}.V_{j-2}.)
      if (j >= 2) wait(bar_o0 + 8 * buf, ((j - 2) >> 1) & 1);
      if (j > 0) {
        sum = write_probabilities(m_ref);
        settle = PairAny(pair_bar, !(sum < kOverflowSum));
      }
      if (settle) {
        float mx = row_max();
        float* xm = xmax + buf * kXFloats;
        xm[hw * kBM + row] = mx;
        PairBarrier(pair_bar);
#pragma unroll
        for (int o = 1; o < kRowSplit; ++o) mx = fmaxf(mx, xm[((hw + o) % kRowSplit) * kBM + row]);
        mx *= p.scale_log2e;
        // Rescale the row sum and, from the second block on, this thread's half of the running output row in
        // tensor memory (the previous block's P.V must have completed). Tensor-memory accesses are warp-wide:
        // rows that keep their reference take part with a factor of one.
        const bool move = mx > m_ref + kRescaleThreshold;
        const float alpha = move ? Ex2(m_ref - mx) : 1.0f;       // 0 on the first block
        l *= alpha;
        if (move) m_ref = mx;
        if (j > 0) {
          TmemWaitStores();                                      // the first sweep's P, about to be overwritten
          if (__any_sync(0xffffffffu, move)) {
            wait(bar_o0 + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1);
            TcFenceAfter();
#pragma unroll
            for (int c = 0; c < kDimChunks; ++c) {
              uint32_t acc[16];
              TmemLoad16(tmem_o + hw * kDimsPerThread + lane_addr + c * 16, acc);
              TmemWaitLoads(acc);
#pragma unroll
              for (int i = 0; i < 16; ++i) acc[i] = __float_as_uint(__uint_as_float(acc[i]) * alpha);
              TmemStore16(tmem_o + hw * kDimsPerThread + lane_addr + c * 16, acc);
            }
            TmemWaitStores();
          }
        }
        sum = write_probabilities(m_ref);
      }
      TmemWaitStores();
      l += sum;
      // V rows at or past the context end (the last block only) may hold anything, NaN included, and 0 * NaN
      // would poison the row: clear them once the block has landed.
      const int rows_valid = kv_len - (jb0 + j) * kBN;
      if (rows_valid < kBN) {
        wait(bar_v0 + 8 * buf, (j >> 1) & 1);
        if (row >= rows_valid) {
          // key `row` of the block: page row / 16, token group (row / 8) % 2, token row % 8; the row's threads
          // clear its 256 bytes between them (the swizzle only permutes 16-byte pieces inside a 128-byte row, and
          // all of them are cleared)
          constexpr int kClearBytes = 2 * kHeadDim / kRowSplit;
          const int byte0 = hw * kClearBytes;
          uint4* r = reinterpret_cast<uint4*>(smem + kVOff + buf * kTileBytes + (row >> 4) * kPageTileBytes +
                                              ((row >> 3) & 1) * kGroupStride + (byte0 >> 7) * kHalfStride +
                                              (row & 7) * 128 + (byte0 & 127));
#pragma unroll
          for (int i = 0; i < kClearBytes / 16; ++i) r[i] = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the cleared rows, visible to the tensor pipe
      }
      if (j + 1 < nblk) fetch_scores(j + 1);
      TcFenceBefore();
      MbarArrive(bar_p0 + 8 * buf);
    }

    // ---- the running output: this thread's 64 dims of its row
    // (the row sums of the two key halves meet through the exchange buffer the last block did not use: every
    // read of it lies before that block's barrier)
    float* xsum = xmax + (nblk & 1) * kXFloats;
    xsum[hw * kBM + row] = l;
    SoftmaxBarrier();
    float l_row = 0.0f;   // the same order in every thread of the row
#pragma unroll
    for (int o = 0; o < kRowSplit; ++o) l_row += xsum[o * kBM + row];
    wait(bar_done, 0);
    TcFenceAfter();
    if (nsplit == 1) {
      // The whole key range was this CTA's: divide by the row's sum, round once - and hand the tile to the warps
      // row by row through shared memory (K buffer 0: every copy has landed, every product has completed), so that
      // a store instruction writes two whole 256-byte rows instead of 16 bytes of each of 32 rows. 16-byte pieces
      // of a row are permuted by the row number, which keeps both sides free of bank conflicts.
      const float inv = 1.0f / l_row;
      uint8_t* stage = smem + kKOff;
#pragma unroll
      for (int c = 0; c < kDimChunks; ++c) TmemLoad16(tmem_o + hw * kDimsPerThread + lane_addr + c * 16, raw[c]);
#pragma unroll
      for (int c = 0; c < kDimChunks; ++c) TmemWaitLoads(raw[c]);
#pragma unroll
      for (int c = 0; c < kDimChunks; ++c) {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          w[i] = AsU32(__floats2half2_rn(__uint_as_float(raw[c][2 * i]) * inv, __uint_as_float(raw[c][2 * i + 1]) * inv));
        const int piece = (hw * kDimsPerThread + c * 16) / 8;
        *reinterpret_cast<uint4*>(stage + row * 256 + (((piece + 0) ^ (row & 15)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(stage + row * 256 + (((piece + 1) ^ (row & 15)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
      }
      SoftmaxBarrier();
      constexpr int kRowsPerPass = kSoftmaxThreads / 32 * 2;
#pragma unroll
      for (int i = 0; i < kBM / kRowsPerPass; ++i) {
        const int r = i * kRowsPerPass + warp * 2 + (lane >> 4), piece = lane & 15;
        const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((piece ^ (r & 15)) << 4));
        if (ok && row0 + r < p.chunk_len)
          *reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(row0 + r) * p.out_stride + head * kHeadDim + piece * 8) = v;
      }
    } else {
      // One run of a tile's key blocks: leave (o unnormalised, reference, row sum) for the kernel that follows this
      // one in the stream and combines a pair's runs in run order.
      float* rec = p.partials + (static_cast<size_t>(head) * gridDim.y + blockIdx.y) * kPartialFloats;
#pragma unroll
      for (int c = 0; c < kDimChunks; ++c) {
        uint32_t raw[16];
        TmemLoad16(tmem_o + hw * kDimsPerThread + lane_addr + c * 16, raw);
        TmemWaitLoads(raw);
        float4* o4 = reinterpret_cast<float4*>(rec) + ((hw * kDimsPerThread + c * 16) / 4) * kBM + row;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          o4[i * kBM] = make_float4(__uint_as_float(raw[4 * i]), __uint_as_float(raw[4 * i + 1]), __uint_as_float(raw[4 * i + 2]),
                                    __uint_as_float(raw[4 * i + 3]));
      }
      if (hw == 0) {
        rec[kBM * kHeadDim + row] = m_ref;
        rec[kBM * kHeadDim + kBM + row] = l_row;
      }
    }
  }
  TcFenceBefore();
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the combining kernel may be set up (it waits for this grid to complete)
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// The pairs that were cut into runs: their records - unnormalised output, reference and row sum against that
// reference - are combined in run order, so the result does not depend on which CTA ran when. One CTA per (head,
// tile, 32 query rows); a warp takes 16 dims of those rows, one row per lane; every row of a cut pair is handled by
// exactly one thread group, and pairs that one CTA held whole were stored by the main kernel and are left alone. Launched
// behind the main kernel in the same stream, over the chunk's last tiles only (the cut ones), as a dependent launch
// that every main CTA releases as its last act: the CTAs of this kernel are then set up while the main grid drains
// and wait (griddepcontrol.wait) until it has completed - 0.4-0.7 us on launches of 15-40 us. (Released when the
// main CTAs START, it measured 4-6 us slower.)
constexpr int kCombineThreads = 256;
constexpr int kCombineRows = 32;
static_assert(kCombineThreads / 32 * 16 == kHeadDim, "one warp per 16 dims");
__global__ void __launch_bounds__(kCombineThreads)
PrefillCombineKernel(const Params p, int items) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int head = blockIdx.x, tile = p.n_tiles - 1 - blockIdx.y;
  const int kv_len = p.chunk_start + p.chunk_len;
  int runs = 1, item0 = 0;   // the pair's runs and its first work item: the items of later tiles come first
  for (int t = p.n_tiles - 1; t >= tile; --t) {
    const int nb = (min(p.chunk_start + (t + 1) * kBM, kv_len) - 1) / kBN + 1;
    runs = (nb + p.split_blocks - 1) / p.split_blocks;
    if (t > tile) item0 += runs;
  }
  if (runs == 1) return;
  const int row = blockIdx.z * kCombineRows + threadIdx.x % 32, d0 = (threadIdx.x / 32) * 16;
  const int out_row = tile * kBM + row;
  if (out_row >= p.chunk_len) return;
  const float* rec0 = p.partials + (static_cast<size_t>(head) * items + item0) * kPartialFloats;
  float mx = -INFINITY;
  for (int r = 0; r < runs; ++r) mx = fmaxf(mx, __ldcg(rec0 + static_cast<size_t>(r) * kPartialFloats + kBM * kHeadDim + row));
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
  float den = 0.0f;
  // (the next run's values are requested before the present run's are used: one L2 latency for all runs, not one each)
  float m_next, l_next;
  float4 v_next[4];
  auto request = [&](int r) {
    const float* rec = rec0 + static_cast<size_t>(r) * kPartialFloats;
    m_next = __ldcg(rec + kBM * kHeadDim + row);
    l_next = __ldcg(rec + kBM * kHeadDim + kBM + row);
    const float4* o4 = reinterpret_cast<const float4*>(rec) + (d0 / 4) * kBM + row;
#pragma unroll
    for (int i = 0; i < 4; ++i) v_next[i] = __ldcg(o4 + i * kBM);
  };
  request(0);
#pragma unroll 1
  for (int r = 0; r < runs; ++r) {
    const float m_run = m_next, l_run = l_next;
    float4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = v_next[i];
    if (r + 1 < runs) request(r + 1);
    const float wgt = Ex2(m_run - mx);      // 0 for a run that saw no key of this row
    den = fmaf(wgt, l_run, den);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[4 * i] = fmaf(wgt, v[i].x, acc[4 * i]);
      acc[4 * i + 1] = fmaf(wgt, v[i].y, acc[4 * i + 1]);
      acc[4 * i + 2] = fmaf(wgt, v[i].z, acc[4 * i + 2]);
      acc[4 * i + 3] = fmaf(wgt, v[i].w, acc[4 * i + 3]);
    }
  }
  const float inv = 1.0f / den;
  half* dst = p.out + static_cast<int64_t>(out_row) * p.out_stride + head * kHeadDim + d0;
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = AsU32(__floats2half2_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv));
  *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
}

// ------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
constexpr int kMaxDevices = 64;
struct DeviceState {
  bool ready = false;
  int* error_flag = nullptr;
  // Scratch of launches that cut (tile, head) pairs across CTAs: grown on demand, never shrunk. (Prompt
  // ingestion is not captured in a graph; a launch that needs more than it has synchronises the device once.)
  float* partials = nullptr;
  size_t partial_floats = 0;
};
DeviceState g_state[kMaxDevices];
EncodeTiledFn g_encode = nullptr;
std::mutex g_mutex;
int g_split_blocks = 0;   // 0: chosen per launch (ChooseSplitBlocks); > 0: forced (rl_prefill_attention_set_split_blocks)

// Longest run of key blocks one CTA should take: a (tile, head) pair with more blocks is cut into equal runs.
// The launch is replayed on the host the way the hardware runs it - CTAs start in grid order, each on the SM that
// frees first - with costs measured on B200 (1.15 us per key block, 8 us of set-up and tear-down per CTA, kPublishUs
// for a run's record, kCombineUs once for the kernel that combines the records), and the candidate with the shortest
// makespan wins; on every chunk shape swept on B200 that choice was the best forced run length or level with it.
// Cutting only the LONGEST tiles often does best (2048 rows at context 8192: runs of at most 60 blocks turn 192
// items in two waves into 240 that level out, 120 -> 104 us); a prompt's last 128 rows against 32768 keys are cut
// into a dozen runs each (263 -> 37 us). The choice depends on the chunk alone, so it is remembered across the
// layers of a model.
double SimulatedMakespan(int chunk_start, int chunk_len, int heads, int split_blocks, int sm_count, std::vector<double>& free_at) {
  constexpr double kBlockUs = 1.15, kSetupUs = 8.0, kPublishUs = 1.5, kCombineUs = 4.0;
  const int64_t kv_len = static_cast<int64_t>(chunk_start) + chunk_len;
  const int n_tiles = (chunk_len + kBM - 1) / kBM;
  free_at.assign(sm_count, 0.0);                       // a min-heap of the times at which the SMs free up
  double end = 0.0;
  bool any_cut = false;
  for (int t = n_tiles - 1; t >= 0; --t) {
    const int64_t last = std::min<int64_t>(static_cast<int64_t>(chunk_start) + static_cast<int64_t>(t + 1) * kBM, kv_len) - 1;
    const int nb = static_cast<int>(last / kBN) + 1;
    const int ns = (nb + split_blocks - 1) / split_blocks;
    for (int run = 0; run < ns; ++run) {
      const int blocks = (run + 1) * nb / ns - run * nb / ns;
      const double cost = kSetupUs + blocks * kBlockUs + (ns > 1 ? kPublishUs : 0.0);
      any_cut |= ns > 1;
      for (int h = 0; h < heads; ++h) {
        std::pop_heap(free_at.begin(), free_at.end(), std::greater<double>());
        const double done = free_at.back() + cost;
        free_at.back() = done;
        std::push_heap(free_at.begin(), free_at.end(), std::greater<double>());
        end = std::max(end, done);
      }
    }
  }
  return end + (any_cut ? kCombineUs : 0.0);
}

int ChooseSplitBlocks(int chunk_start, int chunk_len, int heads, int sm_count) {
  struct Memo { int start, len, heads, sms, choice; };
  static Memo memo = {-1, -1, -1, -1, 0};
  static std::mutex memo_mutex;
  std::lock_guard<std::mutex> lock(memo_mutex);
  if (memo.start == chunk_start && memo.len == chunk_len && memo.heads == heads && memo.sms == sm_count) return memo.choice;
  const int max_blocks = static_cast<int>((static_cast<int64_t>(chunk_start) + chunk_len - 1) / kBN) + 1;
  const int n_tiles = (chunk_len + kBM - 1) / kBM;
  std::vector<double> heap;
  int best = max_blocks;
  double best_us = SimulatedMakespan(chunk_start, chunk_len, heads, max_blocks, sm_count, heap);   // every pair whole
  // A chunk that fills the machine many times over gains nothing from cuts, and replaying it would cost more than it saves.
  if (static_cast<int64_t>(n_tiles) * heads <= 6LL * sm_count) {
    const int64_t pairs = static_cast<int64_t>(n_tiles) * heads;
    auto consider = [&](int run) {
      if (run < 4 || run >= max_blocks) return;
      if (pairs * ((max_blocks + run - 1) / run) > 8LL * sm_count) return;   // bounds the replay at ~1200 items
      const double us = SimulatedMakespan(chunk_start, chunk_len, heads, run, sm_count, heap);
      if (us < best_us) {
        best_us = us;
        best = run;
      }
    };
    for (int r : {2, 3, 4, 5, 6, 8, 10, 12, 16, 20, 24, 32}) consider((max_blocks + r - 1) / r);   // equal cuts of the longest tile
    for (int run = max_blocks - 4; run > max_blocks / 2; run -= 4) consider(run);                   // cuts that only the longer tiles get
  }
  memo = {chunk_start, chunk_len, heads, sm_count, best};
  return best;
}

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
  CUtensorMap q_map, page_map;
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
    // The pool slice as [tile][token group of 8][dim half][token in group][64 halves] (strides 4096, 2048, 128, 256,
    // 2 bytes): a box of one whole tile lands as [token group][dim half][8 tokens][128 B]. The tile count is not
    // part of the launch contract, so the view claims more tiles than a 180 GB device can hold; only tiles of
    // real pages are ever requested.
    const cuuint64_t dims[5] = {64, 8, 2, 2, 1ull << 26};
    const cuuint64_t strides[4] = {static_cast<cuuint64_t>(kHeadDim) * 2, 128, 8ull * kHeadDim * 2,
                                   static_cast<cuuint64_t>(kKvBlock) * kHeadDim * 2};
    const cuuint32_t box[5] = {64, 8, 2, 2, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = g_encode(&page_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(kv_pool_layer), dims, strides,
                                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return Fail(RL_E_BAD_SHAPE, "paged_prefill_attention: pool tensor map (CUresult %d)", static_cast<int>(r));
  }
  // Work items per head: a tile with more than split_blocks key blocks is cut into ceil(blocks / split_blocks) runs.
  const int split_blocks = g_split_blocks > 0 ? g_split_blocks
                                              : ChooseSplitBlocks(chunk_start, chunk_len, num_q_heads, CurrentDeviceFacts().sm_count);
  const int n_tiles = (chunk_len + kBM - 1) / kBM;
  const int64_t kv_len = static_cast<int64_t>(chunk_start) + chunk_len;
  int64_t items = 0;
  bool any_split = false;
  for (int t = 0; t < n_tiles; ++t) {
    const int64_t last = (static_cast<int64_t>(chunk_start) + static_cast<int64_t>(t + 1) * kBM < kv_len
                              ? static_cast<int64_t>(chunk_start) + static_cast<int64_t>(t + 1) * kBM
                              : kv_len) - 1;
    const int nb = static_cast<int>(last / kBN) + 1;
    const int ns = (nb + split_blocks - 1) / split_blocks;
    items += ns;
    any_split |= ns > 1;
  }
  if (items > 65535) return Fail(RL_E_TOO_LARGE, "paged_prefill_attention: chunk too large (%lld work items per head)", static_cast<long long>(items));
  if (any_split) {
    const size_t need = static_cast<size_t>(num_q_heads) * static_cast<size_t>(items) * kPartialFloats;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (st->partial_floats < need) {
      cudaDeviceSynchronize();
      if (st->partials) cudaFree(st->partials);
      st->partials = nullptr;
      st->partial_floats = 0;
      const cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&st->partials), need * sizeof(float));
      if (e != cudaSuccess) return Fail(static_cast<int>(e), "paged_prefill_attention: %zu MB of scratch: %s", need * 4 >> 20, cudaGetErrorString(e));
      st->partial_floats = need;
    }
  }
  Params p;
  p.n_tiles = n_tiles;
  p.split_blocks = split_blocks;
  p.partials = st->partials;
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
  const dim3 grid(num_q_heads, static_cast<unsigned>(items));
  PagedPrefillAttentionKernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(p, q_map, page_map);
  rc = LaunchStatus("paged_prefill_attention");
  if (rc != RL_OK || !any_split) return rc;
  // Only the chunk's last tiles - the ones with more key blocks than the run length - were cut.
  int cut_tiles = 0;
  for (int t = n_tiles - 1; t >= 0; --t) {
    const int64_t last = std::min<int64_t>(static_cast<int64_t>(chunk_start) + static_cast<int64_t>(t + 1) * kBM, kv_len) - 1;
    if (static_cast<int>(last / kBN) + 1 <= split_blocks) break;
    ++cut_tiles;
  }
  // (a dependent launch whatever the process-wide switch says: the kernel begins with the wait for the stream's
  // previous kernel, which is the one above)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_q_heads, cut_tiles, kBM / kCombineRows);
  cfg.blockDim = dim3(kCombineThreads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, PrefillCombineKernel, p, static_cast<int>(items));
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "paged_prefill_attention (combine): %s", cudaGetErrorString(e));
  return LaunchStatus("paged_prefill_attention (combine)");
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

extern "C" int rl_prefill_attention_run_length(int32_t chunk_start, int32_t chunk_len, int32_t num_q_heads,
                                               int32_t sm_count, int32_t* run_blocks_out) {
  using namespace rl;
  if (!run_blocks_out) return Fail(RL_E_NULL_POINTER, "rl_prefill_attention_run_length: null pointer");
  if (chunk_start < 0 || chunk_len < 1 || num_q_heads < 1 || sm_count < 1)
    return Fail(RL_E_BAD_SHAPE, "rl_prefill_attention_run_length: chunk_start >= 0, chunk_len, heads and SMs >= 1");
  *run_blocks_out = rl::pfa::g_split_blocks > 0 ? rl::pfa::g_split_blocks
                                                : rl::pfa::ChooseSplitBlocks(chunk_start, chunk_len, num_q_heads, sm_count);
  return RL_OK;
}

extern "C" int rl_prefill_attention_set_split_blocks(int blocks) {
  if (blocks < 0) return rl::Fail(RL_E_BAD_SHAPE, "rl_prefill_attention_set_split_blocks: 0 (automatic) or a positive block count");
  rl::pfa::g_split_blocks = blocks;
  return RL_OK;
}
