// Paged grouped-query decode attention for sm_100a (B200).
//
// Contract: src/kernels/kernels.cuh:125-146 of the reference; the math is that
// of its decode kernel (src/kernels/paged_attention.cu:122-375): scores
// q.k * scale, SELECT-style masking of slots past seq_len (garbage or NaN in
// unwritten pool slots never reaches a result), online softmax with FP32
// statistics, FP32 accumulation, one FP16 rounding of acc / l. Rows with
// seq_len <= 0 are not written. head_dim 128, 6 query heads per KV head.
//
// What is different, and why (B200: 148 SMs, ~6.5 TB/s measured HBM):
//  * The KV axis is split across the WHOLE grid. All (sequence, kv head) items
//    are laid end to end in 16-token pages and the page range is cut into one
//    equal contiguous share per CTA (one persistent CTA per SM). A batch of 64
//    short sequences and a batch holding a few 32k-token sequences both load
//    every SM equally; the reference walks one (sequence, head) per CTA serially
//    (src/kernels/paged_attention.cu:176,214) and has no split variant. The launch shape
//    depends only on the SM count, never on device-side seq_lens, so it can be
//    frozen in a CUDA graph.
//  * A CTA writes an item it covers completely straight to `out`. An item cut
//    by a CTA boundary is finished by whichever contributor comes LAST, and
//    nobody ever waits: a contributor first looks (load-acquire) whether all
//    the others have already published - usual at the tail of a share, whose
//    neighbour met the same item at the very start of its own share - and then
//    simply reads their (o, m, l) records, under its own fold, and writes the
//    item; otherwise it publishes its record in a small per-device workspace
//    (at most two per CTA) and takes a ticket from an atomic counter, and the
//    holder of the last ticket merges. Either way the records are combined in
//    CTA order with the same arithmetic, so results are bit-reproducible run to
//    run whoever ends up doing it.
//  * K/V pages are fetched by TMA - one cp.async.bulk.tensor per page brings the
//    K tile and the V tile of a head (8 KiB, 128-byte swizzle, so the ldmatrix
//    reads are bank-conflict free) - into a private 3-deep ring per warp, with
//    completion tracked by mbarriers; no warp waits on another except at item
//    boundaries. Loads never use cluster multicast and never touch another
//    GPU's memory.
//  * The 6-query x 16-token dot products and the P.V products run on tensor
//    cores (mma.sync m16n8k16, FP16 in / FP32 accumulate) in the transposed
//    form S^T = K.Q^T, O^T = V^T.P^T so the 6 queries sit in the N=8 dimension
//    and the 16 tokens of a page fill M=16 exactly. CUDA-core FMAs cannot keep
//    up with the HBM stream here: 24.6k FMAs per 8 KiB page is ~48 TFLOP/s of
//    FP32 at 8 TB/s.
//  * The running max is only re-reduced across lanes when some lane sees a
//    score above it (one warp vote per page otherwise); probabilities are
//    rounded to FP16 for the P.V product, their sum is kept in FP32.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace rl {
namespace attn {

constexpr int kHeadDim = 128;
constexpr int kGroup = 6;               // query heads per KV head
#ifndef RL_ATTN_WARPS
#define RL_ATTN_WARPS 8
#endif
#ifndef RL_ATTN_STAGES
#define RL_ATTN_STAGES 3
#endif
constexpr int kWarps = RL_ATTN_WARPS;   // 4, 8 or 12: the merge maps 128 threads to one head's 128 columns
constexpr int kThreads = kWarps * 32;
constexpr int kStages = RL_ATTN_STAGES; // pages in flight per warp
constexpr int kMergeGroups = kThreads / 128;          // heads merged side by side
constexpr int kHeadsPerGroup = 6 / kMergeGroups;      // heads each 128-thread group walks
static_assert(kThreads % 128 == 0 && 6 % kMergeGroups == 0, "warps per CTA must be 4, 8 or 12");
#ifndef RL_ATTN_CTAS_PER_SM
#define RL_ATTN_CTAS_PER_SM 1
#endif
#ifndef RL_ATTN_MAX_SEQS
#define RL_ATTN_MAX_SEQS 1024
#endif
constexpr int kCtasPerSm = RL_ATTN_CTAS_PER_SM;
constexpr int kSeqsPerThread = (RL_ATTN_MAX_SEQS + kThreads - 1) / kThreads;
constexpr int kInlineContributors = 3;  // items over at most this many CTAs are merged from registers
constexpr int kMergeBatch = 8;          // longer items: records fetched this many contributors at a time
constexpr int kPageBytes = kKvBlock * kHeadDim * 2;  // 4096: one (block, kv, head) tile
constexpr int kStageBytes = 2 * kPageBytes;          // K tile + V tile
constexpr int kMaxSeqsPerLaunch = RL_ATTN_MAX_SEQS;
constexpr int kORowPad = 132;           // floats per query row in the merge buffer (bank spread)
constexpr int kPartialFloats = kGroup * kHeadDim + 16;  // o[6][128], m[6], l[6], pad
constexpr int kMaxCtas = 256 * kCtasPerSm;  // workspace is sized for this many CTAs
constexpr int kNewestPageBit = 1 << 30; // tile indices stay below 2^30: a 180 GB device holds < 2^26 tiles

// Shared-memory carve (offsets from a 1024-byte aligned base).
constexpr int kRingOff = 0;
constexpr int kRingBytes = kWarps * kStages * kStageBytes;  // 196608
constexpr int kOBufOff = kRingOff + kRingBytes;
constexpr int kOBufBytes = kWarps * kGroup * kORowPad * 4;  // 25344
constexpr int kMlStride = (kWarps + 3) & ~3;                // m[head][warp], l[head][warp]: a head's values of all
constexpr int kMlOff = kOBufOff + kOBufBytes;               // warps are consecutive (read 16 bytes at a time)
constexpr int kMlBytes = 2 * 8 * kMlStride * 4;
static_assert(kOBufBytes % 16 == 0, "m / l rows must stay 16-byte aligned");
constexpr int kBarOff = kMlOff + kMlBytes;
constexpr int kBarBytes = kWarps * kStages * 8;
constexpr int kPrefixOff = kBarOff + kBarBytes;
constexpr int kPrefixBytes = (kMaxSeqsPerLaunch + 8) * 4;
constexpr int kSmemBytes = kPrefixOff + kPrefixBytes + 1024;  // + slack to align the base
static_assert(kSmemBytes <= 227 * 1024, "attention shared memory exceeds the 227 KB per-CTA limit");
static_assert(kCtasPerSm * (kSmemBytes + 1024) <= 228 * 1024, "that many CTAs do not fit one SM's shared memory");

// Workspace (one per device): meta ints, then kMaxCtas * 2 partial records.
constexpr int kTicketOff = 16;                     // meta[0] = error flag, meta[16 + c] = tickets of
constexpr int kMetaInts = kTicketOff + kMaxCtas;   // the item that starts in CTA c and runs on
constexpr size_t kWorkspaceBytes =
    static_cast<size_t>(kMetaInts) * 4 + static_cast<size_t>(kMaxCtas) * 2 * kPartialFloats * 4;

constexpr long long kWaitCycles = 2000000000LL;  // ~1 s: a load that never lands sets the error flag

struct Params {
  half* out;
  int64_t out_stride;
  const half* q;
  int64_t q_stride;
  const int32_t* tables;
  const int32_t* seq_lens;
  int num_seqs;
  int max_blocks;
  int kv_heads;
  float scale_log2e;
  int* meta;        // workspace meta
  float* partials;  // workspace partial records
  long long wait_cycles;  // limit of every mbarrier wait (kWaitCycles unless a test shortened it)
  int drop_first_copy;    // test hook: warp 0 of CTA 0 never requests its first page, so its wait must run out
  unsigned long long* timeline;  // diagnostics build only
};

// ------------------------------------------------------------------ PTX

__device__ __forceinline__ uint32_t SmemAddr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void MbarInit(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void MbarExpectTx(uint32_t bar, int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint32_t bar, int parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the phase never completed within `limit` cycles.
__device__ __forceinline__ bool MbarWait(uint32_t bar, int parity, long long limit) {
  if (MbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!MbarTryWait(bar, parity)) {
    if (clock64() - t0 > limit) return false;
  }
  return true;
}
// One page of one KV head - its K tile and its V tile, 8 KiB - in a single tensor copy into this CTA's
// shared memory, 128-byte swizzled; completion is counted in bytes on `bar`. No cluster multicast.
// KV pages are read once per launch: they are marked evict-first in L2 so that the stream does not
// push out the small data every launch re-reads (seq_lens, block tables - loaded evict-last below).
__device__ __forceinline__ void TmaLoadPage(uint32_t dst, const CUtensorMap* map, int tile, uint32_t bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %2, %2, %3}], [%4], %5;" ::"r"(dst),
      "l"(map), "r"(0), "r"(tile), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t L2PolicyEvictFirst() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t L2PolicyEvictLast() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ int LdgKeepInL2(const int32_t* ptr, uint64_t policy) {
  int v;
  asm volatile("ld.global.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(ptr), "l"(policy));
  return v;
}
#ifdef RL_ATTN_TIMELINE
__device__ __forceinline__ unsigned long long GlobalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define RL_STAMP(slot) \
  if (p.timeline && lane == 0) p.timeline[(blockIdx.x * kWarps + warp) * 8 + (slot)] = GlobalTimerNs()
#else
#define RL_STAMP(slot)
#endif
__device__ __forceinline__ void Ldsm4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void Ldsm4T(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t MovmT(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void Mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float Exp2(float x) {
  float y;
  asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t PackHalf2(float lo, float hi) {
  return AsU32(__floats2half2_rn(lo, hi));
}

// ------------------------------------------------------- work partition

// First flattened page index of CTA c's share when `total` pages are cut into `ctas` shares.
__host__ __device__ __forceinline__ long long ShareBegin(long long c, long long total, int ctas) {
  return c * total / ctas;
}
// The CTA whose share holds flattened page t.
__host__ __device__ __forceinline__ int ShareOf(long long t, long long total, int ctas) {
  return static_cast<int>(((t + 1) * ctas - 1) / total);
}

// Position in the flattened page order: sequence-major, then KV head, then page.
struct Cursor {
  int seq;
  int head;
  int page;
  int pages;  // pages of `seq`
};

__device__ __forceinline__ Cursor Locate(long long t, const int* prefix, int num_seqs, int heads) {
  int lo = 0, hi = num_seqs - 1;
  while (lo < hi) {  // first seq with heads * prefix[seq+1] > t (empty sequences skipped)
    const int mid = (lo + hi) >> 1;
    if (static_cast<long long>(heads) * prefix[mid + 1] <= t) lo = mid + 1; else hi = mid;
  }
  Cursor c;
  c.seq = lo;
  c.pages = prefix[lo + 1] - prefix[lo];
  const int rem = static_cast<int>(t - static_cast<long long>(heads) * prefix[lo]);
  c.head = rem / c.pages;
  c.page = rem - c.head * c.pages;
  return c;
}

// --------------------------------------------------------------- kernel

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
PagedAttentionSplitKernel(const Params p, const __grid_constant__ CUtensorMap tile_map) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t ring = SmemAddr(smem + kRingOff);
  float* obuf = reinterpret_cast<float*>(smem + kOBufOff);
  float* mbuf = reinterpret_cast<float*>(smem + kMlOff);
  float* lbuf = mbuf + 8 * kMlStride;
  const uint32_t bars = SmemAddr(smem + kBarOff);
  int* prefix = reinterpret_cast<int*>(smem + kPrefixOff);

  __shared__ bool merge_here, others_done;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int heads = p.kv_heads;
  const int num_seqs = p.num_seqs;
  RL_STAMP(0);
  // Let a dependent launch (the next attention call, when prologue overlap is on) start its own
  // prologue as soon as this grid is resident; it still waits for this grid to finish before it
  // touches anything this grid writes.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tile_map) : "memory");
  }

  const uint64_t keep_policy = L2PolicyEvictLast(), stream_policy = L2PolicyEvictFirst();
  // ---- page prefix over sequences (every CTA computes the same table) ----
  {
    __shared__ int warp_tot[kWarps];
    int n[kSeqsPerThread], sum = 0;
#pragma unroll
    for (int i = 0; i < kSeqsPerThread; ++i) {
      const int s = tid * kSeqsPerThread + i;
      int len = s < num_seqs ? LdgKeepInL2(p.seq_lens + s, keep_policy) : 0;
      len = min(len, p.max_blocks * kKvBlock);
      n[i] = len > 0 ? (len + kKvBlock - 1) >> kKvBlockShift : 0;
      sum += n[i];
    }
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += warp_tot[w];
    int run = base + incl - sum;
#pragma unroll
    for (int i = 0; i < kSeqsPerThread; ++i) {
      const int s = tid * kSeqsPerThread + i;
      if (s <= num_seqs) prefix[s] = run;
      run += n[i];
    }
    if (tid == kThreads - 1 && num_seqs >= kThreads * kSeqsPerThread) prefix[num_seqs] = run;
    for (int b = tid; b < kStages * kWarps; b += kThreads) MbarInit(bars + b * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
  }
  const long long total = static_cast<long long>(heads) * prefix[num_seqs];
  if (total == 0) return;
  const long long share_begin = ShareBegin(blockIdx.x, total, gridDim.x);
  const long long share_end = ShareBegin(blockIdx.x + 1, total, gridDim.x);
  if (share_begin >= share_end) return;

  // ---- this warp's pages: share-relative indices warp, warp + kWarps, ... ----
  const int share_len = static_cast<int>(share_end - share_begin);
  const int n_mine = share_len > warp ? (share_len - warp + kWarps - 1) / kWarps : 0;
  const uint32_t my_ring = ring + warp * (kStages * kStageBytes);
  const uint32_t my_bars = bars + warp * (kStages * 8);
  bool failed = false;
  int fail_at = 0;  // index of the page whose wait gave up; copies from there on are drained before exit

  // Page metadata is looked up 32 pages at a time, one page per lane: lane j of batch b holds the
  // index of the K tile of this warp's page 32b + j, counted in 4 KiB (block, kv, head) tiles; the V
  // tile is `heads` tiles further. The block-table read of a batch is issued a whole batch ahead of
  // its first use.
  auto fetch_tiles = [&](int batch) -> int {
    const int k = 32 * batch + lane;
    if (k >= n_mine) return 0;
    const Cursor c = Locate(share_begin + warp + kWarps * k, prefix, num_seqs, heads);
    const int block = LdgKeepInL2(p.tables + static_cast<int64_t>(c.seq) * p.max_blocks + c.page, keep_policy);
    // The last page of a sequence holds the token this step has just written: it is marked, so that it
    // is never requested before the previous kernel of the stream has completed.
    return (block * 2 * heads + c.head) | (c.page == c.pages - 1 ? kNewestPageBit : 0);
  };
  int tiles_cur = fetch_tiles(0);
  int tiles_next = n_mine > 32 ? fetch_tiles(1) : 0;
  // Everything above read only seq_lens and the block tables. When this grid was launched with
  // programmatic stream serialisation it may have started while the previous kernel of the stream
  // (the KV scatter of this layer, or the previous attention call) was still running: wait for it
  // to complete before reading the pool or Q, or writing the output and the workspace. A no-op for
  // an ordinary launch.
  //
  // The first ring of pages is requested BEFORE that wait, except pages that hold a sequence's newest
  // token: every other page was written by an earlier step, so its load can run under the tail of the
  // previous kernel and its DRAM latency is off the critical path. (Contract of the overlap option:
  // kernels still in flight when this one starts may write only each sequence's last page.)
  int n_issue = 0, n_use = 0;
  int deferred = 0;  // bit i: page i of the first ring waits for the dependency gate
  {
    const int first = n_mine < kStages ? n_mine : kStages;
#pragma unroll 1
    for (int i = 0; i < first; ++i) {
      const int tile_k = __shfl_sync(0xffffffffu, tiles_cur, i);
      if (tile_k & kNewestPageBit) {
        deferred |= 1 << i;
      } else if (p.drop_first_copy && blockIdx.x == 0 && warp == 0 && i == 0) {
        // test hook: this copy is never requested, the wait for it below gives up and raises the flag
      } else if (lane == 0) {
        MbarExpectTx(my_bars + i * 8, kStageBytes);
        TmaLoadPage(my_ring + i * kStageBytes, &tile_map, tile_k, my_bars + i * 8, stream_policy);
      }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll 1
    for (int i = 0; i < first; ++i) {
      if ((deferred >> i) & 1) {
        const int tile_k = __shfl_sync(0xffffffffu, tiles_cur, i) & ~kNewestPageBit;
        if (lane == 0) {
          MbarExpectTx(my_bars + i * 8, kStageBytes);
          TmaLoadPage(my_ring + i * kStageBytes, &tile_map, tile_k, my_bars + i * 8, stream_policy);
        }
      }
    }
    n_issue = first;
  }
  auto issue_one = [&]() {
    const int tile_k = __shfl_sync(0xffffffffu, tiles_cur, n_issue & 31) & ~kNewestPageBit;
    if (lane == 0) {
      const int stage = n_issue % kStages;
      const uint32_t dst = my_ring + stage * kStageBytes;
      const uint32_t bar = my_bars + stage * 8;
      MbarExpectTx(bar, kStageBytes);
      TmaLoadPage(dst, &tile_map, tile_k, bar, stream_policy);
    }
    ++n_issue;
    if ((n_issue & 31) == 0) {
      tiles_cur = tiles_next;
      tiles_next = fetch_tiles((n_issue >> 5) + 1);
    }
  };
  // ldmatrix byte offsets inside a stage, fixed per lane. K tile: k-steps j and j+4 are 2048
  // apart (the two 64-dim boxes); V tile likewise for dim tiles j and j+4.
  uint32_t koff[4], voff[4];
  {
    const int k_row = (lane & 7) + ((lane >> 3) & 1) * 8;  // token row, A operand of S^T
    const int k_sel = lane >> 4;                            // which 8-dim chunk of the k-step
    const int v_row = (lane & 7) + (lane >> 4) * 8;         // token row, transposed loads of V
    const int v_sel = (lane >> 3) & 1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      koff[j] = k_row * 128 + (((2 * j + k_sel) ^ (k_row & 7)) << 4);
      voff[j] = 4096 + v_row * 128 + (((2 * j + v_sel) ^ (v_row & 7)) << 4);
    }
  }
  constexpr uint32_t hi_delta = 2048;  // dims 64..127 of a tile sit one 2 KiB box further
  RL_STAMP(1);

  // ---- walk the share one (sequence, head) segment at a time ----
  long long seg_begin = share_begin;
#pragma unroll 1
  while (seg_begin < share_end) {
    const Cursor sc = Locate(seg_begin, prefix, num_seqs, heads);
    const long long item_begin = static_cast<long long>(heads) * prefix[sc.seq] +
                                 static_cast<long long>(sc.head) * sc.pages;
    const long long item_end = item_begin + sc.pages;
    const long long seg_end = item_end < share_end ? item_end : share_end;
    const int seq_len = min(p.seq_lens[sc.seq], p.max_blocks * kKvBlock);
    const int seg_end_rel = static_cast<int>(seg_end - share_begin);
    const int item_begin_rel = static_cast<int>(item_begin - share_begin);  // may be negative
    // Q fragments of this item: B operand of S^T = K.Q^T, query g (< 6) in column g.
    uint32_t qb[8][2];
    {
      const half* qrow = p.q + static_cast<int64_t>(sc.seq) * p.q_stride +
                         (static_cast<int64_t>(sc.head) * kGroup + g) * kHeadDim + 2 * tig;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        qb[kk][0] = g < kGroup ? __ldg(reinterpret_cast<const uint32_t*>(qrow + 16 * kk)) : 0u;
        qb[kk][1] = g < kGroup ? __ldg(reinterpret_cast<const uint32_t*>(qrow + 16 * kk + 8)) : 0u;
      }
    }
    // Who else works on this item (uniform over the CTA; worked out here, under the loads of Q, not after the
    // last page, where nothing would hide the two 64-bit divisions).
    const bool whole = seg_begin == item_begin && seg_end == item_end;
    const int ctas = gridDim.x;
    int c_first = blockIdx.x, c_last = blockIdx.x, contributors = 1;
    bool sparse = false;
    if (!whole) {
      c_first = item_begin < share_begin ? ShareOf(item_begin, total, ctas) : blockIdx.x;
      c_last = item_end > share_end ? ShareOf(item_end - 1, total, ctas) : blockIdx.x;
      sparse = total < ctas;  // then every non-empty share is exactly one page
      contributors = sparse ? sc.pages : c_last - c_first + 1;
    }
    // Have all the other contributors of this item published already? (Usual for the tail of a share: the next
    // CTA met the same item at the very start of its own share.) Then this CTA is the last one, reads their
    // records - under the fold below - and neither publishes its own nor takes a ticket. Thread 0 looks while
    // its warp still has two pages of the segment to go, so the answer is there when the last page is done; a
    // contributor that publishes after the look is simply met through the tickets.
    const bool may_read_inline = !whole && !sparse && contributors <= kInlineContributors;
    int seen = -1;

    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

#pragma unroll 1
    for (int rel = warp + kWarps * n_use; rel < seg_end_rel; rel += kWarps) {
      const int stage = n_use % kStages;
      const uint32_t st = my_ring + stage * kStageBytes;
      if (!failed && !MbarWait(my_bars + stage * 8, (n_use / kStages) & 1, p.wait_cycles)) {
        failed = true;
        fail_at = n_use;
        if (lane == 0) atomicExch(p.meta, 1);
      }
      if (n_use == 0) { RL_STAMP(2); }
      if (may_read_inline && tid == 0 && seen < 0 && rel + 2 * kWarps >= seg_end_rel)
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.meta + kTicketOff + c_first) : "memory");
      if (!failed) {
        const int valid = seq_len - (rel - item_begin_rel) * kKvBlock;  // >= 1; >= 16 for a full page

        // S^T[token][query] = sum_d K[token][d] * Q[query][d]; two chains for latency
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t a[4], a2[4];
          Ldsm4(st + koff[j], a);
          Ldsm4(st + koff[j] + hi_delta, a2);
          Mma16816(s, a, qb[j][0], qb[j][1]);
          Mma16816(s2, a2, qb[j + 4][0], qb[j + 4][1]);
        }
        // scale into the log2 domain; SELECT masking of slots past seq_len
        s[0] = g < valid ? (s[0] + s2[0]) * p.scale_log2e : -INFINITY;
        s[1] = g < valid ? (s[1] + s2[1]) * p.scale_log2e : -INFINITY;
        s[2] = g + 8 < valid ? (s[2] + s2[2]) * p.scale_log2e : -INFINITY;
        s[3] = g + 8 < valid ? (s[3] + s2[3]) * p.scale_log2e : -INFINITY;
        float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
        if (__any_sync(0xffffffffu, mx0 > m0 || mx1 > m1)) {
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
          }
          const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
          const float a0 = Exp2(m0 - n0), a1 = Exp2(m1 - n1);  // exp2(-inf) = 0 on the first page
          m0 = n0;
          m1 = n1;
          l0 *= a0;
          l1 *= a1;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            o[i][0] *= a0;
            o[i][1] *= a1;
            o[i][2] *= a0;
            o[i][3] *= a1;
          }
        }
        const float p0 = Exp2(s[0] - m0), p1 = Exp2(s[1] - m1);
        const float p2 = Exp2(s[2] - m0), p3 = Exp2(s[3] - m1);
        l0 += p0 + p2;
        l1 += p1 + p3;
        // P^T as the B operand of O^T = V^T.P^T: transpose the two 8x8 [token][query] blocks.
        const uint32_t b0 = MovmT(PackHalf2(p0, p1));
        const uint32_t b1 = MovmT(PackHalf2(p2, p3));
        if (valid >= kKvBlock) {
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) {
            uint32_t a[4];
            Ldsm4T(st + voff[mt & 3] + (mt >> 2) * hi_delta, a);
            Mma16816(o[mt], a, b0, b1);
          }
        } else {
          // Last, partial page: V rows past seq_len may hold NaN and 0 * NaN would poison the
          // accumulator, so those token columns of V^T are cleared in registers.
          const uint32_t k01 = (2 * tig < valid ? 0x0000FFFFu : 0u) | (2 * tig + 1 < valid ? 0xFFFF0000u : 0u);
          const uint32_t k23 = (2 * tig + 8 < valid ? 0x0000FFFFu : 0u) | (2 * tig + 9 < valid ? 0xFFFF0000u : 0u);
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) {
            uint32_t a[4];
            Ldsm4T(st + voff[mt & 3] + (mt >> 2) * hi_delta, a);
            a[0] &= k01;
            a[1] &= k01;
            a[2] &= k23;
            a[3] &= k23;
            Mma16816(o[mt], a, b0, b1);
          }
        }
      }
      ++n_use;
      __syncwarp();  // every lane is done reading this stage before it is refilled
      if (!failed && n_issue < n_mine) issue_one();
    }

    RL_STAMP(3);
    // ---- the segment is done: fold the warps' (o, m, l); then write the item, or hand it on ----
    if (tid == 0) {
      if (may_read_inline && seen < 0)   // warp 0 had fewer than two pages in this segment
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.meta + kTicketOff + c_first) : "memory");
      others_done = may_read_inline && seen == contributors - 1;
    }
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, off);
      l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    if (tig < 3) {
      float* ob = obuf + warp * (kGroup * kORowPad);
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) {
        ob[(2 * tig) * kORowPad + 16 * mt + g] = o[mt][0];
        ob[(2 * tig + 1) * kORowPad + 16 * mt + g] = o[mt][1];
        ob[(2 * tig) * kORowPad + 16 * mt + g + 8] = o[mt][2];
        ob[(2 * tig + 1) * kORowPad + 16 * mt + g + 8] = o[mt][3];
      }
      if (g == 0) {
        mbuf[(2 * tig) * kMlStride + warp] = m0;
        mbuf[(2 * tig + 1) * kMlStride + warp] = m1;
        lbuf[(2 * tig) * kMlStride + warp] = l0;
        lbuf[(2 * tig + 1) * kMlStride + warp] = l1;
      }
    }
    __syncthreads();
    RL_STAMP(5);
    {
      const int d = tid & 127;
      const int q0 = tid >> 7;  // this thread's heads: q0, q0 + kMergeGroups, ...
      // Records of the OTHER contributors (at most two when read inline), in CTA order.
      float om[kInlineContributors - 1][kHeadsPerGroup], ol[kInlineContributors - 1][kHeadsPerGroup],
          oo[kInlineContributors - 1][kHeadsPerGroup];
      // (An item over exactly two CTAs - the usual case - takes straight-line code: at the end of a share the
      // fetch of every instruction is on the critical path. Never reached by `sparse` launches.)
      auto load_others = [&]() {
        if (contributors == 2) {
          const int c = c_first == static_cast<int>(blockIdx.x) ? c_last : c_first;
          const float* r = p.partials + (static_cast<size_t>(c) * 2 + (c == c_first ? 1 : 0)) * kPartialFloats;
#pragma unroll
          for (int qi = 0; qi < kHeadsPerGroup; ++qi) {
            const int qh = q0 + kMergeGroups * qi;
            om[0][qi] = __ldcg(r + kGroup * kHeadDim + qh);
            ol[0][qi] = __ldcg(r + kGroup * kHeadDim + 8 + qh);
            oo[0][qi] = __ldcg(r + qh * kHeadDim + d);
          }
          return;
        }
        int k = 0;
        for (int c = c_first; c <= c_last; ++c) {
          if (c == static_cast<int>(blockIdx.x)) continue;
          const float* r = p.partials + (static_cast<size_t>(c) * 2 + (c == c_first ? 1 : 0)) * kPartialFloats;
#pragma unroll
          for (int j = 0; j < kInlineContributors - 1; ++j) {
            if (j == k) {
#pragma unroll
              for (int qi = 0; qi < kHeadsPerGroup; ++qi) {
                const int qh = q0 + kMergeGroups * qi;
                om[j][qi] = __ldcg(r + kGroup * kHeadDim + qh);
                ol[j][qi] = __ldcg(r + kGroup * kHeadDim + 8 + qh);
                oo[j][qi] = __ldcg(r + qh * kHeadDim + d);
              }
            }
          }
          ++k;
        }
      };
      const bool fast = !whole && others_done;
      if (fast) load_others();

      // The warps' (o, m, l) folded in warp order, every thread for its own heads and column: the eight maxima
      // and sums of a head are broadcast reads, the eight scale factors exp2(m_w - max) are recomputed by each
      // thread. (Six threads computing them once for all, behind a CTA barrier of its own, was measured at
      // ~1000 cycles at the end of every share - after the last page nothing hides latency.)
      float acc[kHeadsPerGroup], mxo[kHeadsPerGroup], deno[kHeadsPerGroup];
#pragma unroll
      for (int qi = 0; qi < kHeadsPerGroup; ++qi) {
        const int qh = q0 + kMergeGroups * qi;
        float mw[kMlStride], lw[kMlStride];
#pragma unroll
        for (int i = 0; i < kMlStride / 4; ++i) {
          const float4 m4 = reinterpret_cast<const float4*>(mbuf + qh * kMlStride)[i];
          const float4 l4 = reinterpret_cast<const float4*>(lbuf + qh * kMlStride)[i];
          mw[4 * i] = m4.x, mw[4 * i + 1] = m4.y, mw[4 * i + 2] = m4.z, mw[4 * i + 3] = m4.w;
          lw[4 * i] = l4.x, lw[4 * i + 1] = l4.y, lw[4 * i + 2] = l4.z, lw[4 * i + 3] = l4.w;
        }
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, mw[w]);
        float a = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const float f = Exp2(mw[w] - mx);  // 0 for a warp that saw no page
          a = fmaf(f, obuf[(w * kGroup + qh) * kORowPad + d], a);
          den = fmaf(f, lw[w], den);
        }
        acc[qi] = a;
        mxo[qi] = mx;
        deno[qi] = den;
      }
      half* out_row = p.out + static_cast<int64_t>(sc.seq) * p.out_stride +
                      static_cast<int64_t>(sc.head) * kGroup * kHeadDim + d;
      // The item from this CTA's fold and the other contributors' records, always combined in CTA
      // order with the same arithmetic, whichever CTA happens to do it.
      auto combine_inline = [&]() {
        if (contributors == 2) {  // the same arithmetic in the same (CTA) order, without the loops
          const bool me_first = c_first == static_cast<int>(blockIdx.x);
#pragma unroll
          for (int qi = 0; qi < kHeadsPerGroup; ++qi) {
            const float mx = fmaxf(mxo[qi], om[0][qi]);
            const float f_me = Exp2(mxo[qi] - mx), f_other = Exp2(om[0][qi] - mx);
            const float f1 = me_first ? f_me : f_other, f2 = me_first ? f_other : f_me;
            const float x1 = me_first ? acc[qi] : oo[0][qi], x2 = me_first ? oo[0][qi] : acc[qi];
            const float l1 = me_first ? deno[qi] : ol[0][qi], l2 = me_first ? ol[0][qi] : deno[qi];
            const float a = fmaf(f2, x2, fmaf(f1, x1, 0.0f));
            const float dn = fmaf(f2, l2, fmaf(f1, l1, 0.0f));
            out_row[(q0 + kMergeGroups * qi) * kHeadDim] = __float2half_rn(a / dn);
          }
          return;
        }
#pragma unroll
        for (int qi = 0; qi < kHeadsPerGroup; ++qi) {
          float mx = mxo[qi];
#pragma unroll
          for (int j = 0; j < kInlineContributors - 1; ++j)
            if (j < contributors - 1) mx = fmaxf(mx, om[j][qi]);
          float a = 0.0f, dn = 0.0f;
          int k = 0;
          for (int c = c_first; c <= c_last; ++c) {
            if (c == static_cast<int>(blockIdx.x)) {
              const float f = Exp2(mxo[qi] - mx);
              a = fmaf(f, acc[qi], a);
              dn = fmaf(f, deno[qi], dn);
            } else {
#pragma unroll
              for (int j = 0; j < kInlineContributors - 1; ++j) {
                if (j == k) {
                  const float f = Exp2(om[j][qi] - mx);
                  a = fmaf(f, oo[j][qi], a);
                  dn = fmaf(f, ol[j][qi], dn);
                }
              }
              ++k;
            }
          }
          out_row[(q0 + kMergeGroups * qi) * kHeadDim] = __float2half_rn(a / dn);
        }
      };
      if (whole) {
#pragma unroll
        for (int qi = 0; qi < kHeadsPerGroup; ++qi)
          out_row[(q0 + kMergeGroups * qi) * kHeadDim] = __float2half_rn(acc[qi] / deno[qi]);
      } else if (fast) {
        combine_inline();
        if (tid == 0) p.meta[kTicketOff + c_first] = 0;  // everyone had arrived: re-arm for the next launch
      } else {
        // Publish this CTA's record, take a ticket; the last contributor of the item merges.
        // slot 0: the item started in an earlier CTA; slot 1: it starts here and runs on
        float* rec = p.partials +
                     (static_cast<size_t>(blockIdx.x) * 2 + (item_begin < share_begin ? 0 : 1)) * kPartialFloats;
#pragma unroll
        for (int qi = 0; qi < kHeadsPerGroup; ++qi) {
          const int qh = q0 + kMergeGroups * qi;
          rec[qh * kHeadDim + d] = acc[qi];
          if (d == 0) {
            rec[kGroup * kHeadDim + qh] = mxo[qi];
            rec[kGroup * kHeadDim + 8 + qh] = deno[qi];
          }
        }
        RL_STAMP(6);
        __syncthreads();  // the whole record is written (CTA scope) ...
        if (tid == 0) {
          __threadfence();  // ... and ordered before the ticket at device scope (fences are cumulative)
          const int ticket = atomicAdd(p.meta + kTicketOff + c_first, 1);
          merge_here = ticket == contributors - 1;
          if (merge_here) p.meta[kTicketOff + c_first] = 0;  // everyone has arrived: re-arm
        }
        __syncthreads();
        RL_STAMP(7);
        if (merge_here) {
          __threadfence();
          if (!sparse && contributors <= kInlineContributors) {
            load_others();
            combine_inline();
          } else {
            // Many contributors (a long sequence over many CTAs). This CTA is the last to arrive, so the whole
            // grid waits for it: the records are fetched kMergeBatch contributors at a time, every load of a
            // batch in flight before the first use (one L2 round trip per batch instead of one per
            // contributor), and folded in CTA order with a running maximum, as an online softmax does.
            float mx[kHeadsPerGroup], a[kHeadsPerGroup], dn[kHeadsPerGroup];
#pragma unroll
            for (int qi = 0; qi < kHeadsPerGroup; ++qi) {
              mx[qi] = -INFINITY;
              a[qi] = dn[qi] = 0.0f;
            }
#pragma unroll 1
            for (int c0 = c_first; c0 <= c_last; c0 += kMergeBatch) {
              float mv[kMergeBatch][kHeadsPerGroup], ov[kMergeBatch][kHeadsPerGroup], lv[kMergeBatch][kHeadsPerGroup];
              bool live[kMergeBatch];
#pragma unroll
              for (int j = 0; j < kMergeBatch; ++j) {
                const int c = c0 + j;
                live[j] = c <= c_last && !(sparse && ShareBegin(c, total, ctas) == ShareBegin(c + 1, total, ctas));
                if (live[j]) {
                  const float* r = p.partials + (static_cast<size_t>(c) * 2 + (c == c_first ? 1 : 0)) * kPartialFloats;
#pragma unroll
                  for (int qi = 0; qi < kHeadsPerGroup; ++qi) {
                    const int qh = q0 + kMergeGroups * qi;
                    mv[j][qi] = __ldcg(r + kGroup * kHeadDim + qh);
                    ov[j][qi] = __ldcg(r + qh * kHeadDim + d);
                    lv[j][qi] = __ldcg(r + kGroup * kHeadDim + 8 + qh);
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < kMergeBatch; ++j) {
                if (live[j]) {
#pragma unroll
                  for (int qi = 0; qi < kHeadsPerGroup; ++qi) {
                    const float m_new = fmaxf(mx[qi], mv[j][qi]);
                    const float keep = Exp2(mx[qi] - m_new), add = Exp2(mv[j][qi] - m_new);
                    a[qi] = fmaf(add, ov[j][qi], a[qi] * keep);
                    dn[qi] = fmaf(add, lv[j][qi], dn[qi] * keep);
                    mx[qi] = m_new;
                  }
                }
              }
            }
#pragma unroll
            for (int qi = 0; qi < kHeadsPerGroup; ++qi)
              out_row[(q0 + kMergeGroups * qi) * kHeadDim] = __float2half_rn(a[qi] / dn[qi]);
          }
        }
      }
    }
    __syncthreads();
    seg_begin = seg_end;
    RL_STAMP(4);
  }
  // A warp that gave up on a load still owns copies in flight: give them one more bounded
  // chance to land before the CTA's shared memory is released.
  if (failed) {
    for (int k = fail_at; k < n_issue; ++k) MbarWait(my_bars + (k % kStages) * 8, (k / kStages) & 1, p.wait_cycles);
  }
}

// Cross-check kernel for tests: one warp per (sequence, query head), textbook
// two-pass softmax on CUDA cores straight from global memory.
__global__ void __launch_bounds__(32)
PagedAttentionCheckKernel(half* out, int64_t out_stride, const half* q, int64_t q_stride,
                          const half* pool, const int32_t* tables, const int32_t* seq_lens,
                          int max_blocks, int kv_heads, int group, float scale) {
  const int seq = blockIdx.x, qh = blockIdx.y, lane = threadIdx.x;
  const int len = min(seq_lens[seq], max_blocks * kKvBlock);
  if (len <= 0) return;
  const int kvh = qh / group;
  const int32_t* row = tables + static_cast<int64_t>(seq) * max_blocks;
  float qv[4];
  for (int i = 0; i < 4; ++i) qv[i] = __half2float(q[seq * q_stride + qh * kHeadDim + lane * 4 + i]);
  auto tile = [&](int t, int kv) {
    const int64_t b = row[t >> kKvBlockShift];
    return pool + ((((b * 2 + kv) * kv_heads + kvh) * kKvBlock) + (t & (kKvBlock - 1))) * kHeadDim;
  };
  auto score = [&](int t) {
    const half* kr = tile(t, 0);
    float dot = 0.0f;
    for (int i = 0; i < 4; ++i) dot = fmaf(qv[i], __half2float(kr[lane * 4 + i]), dot);
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    return dot * scale;
  };
  float mx = -INFINITY;
  for (int t = 0; t < len; ++t) mx = fmaxf(mx, score(t));
  float den = 0.0f, acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int t = 0; t < len; ++t) {
    const float w = expf(score(t) - mx);
    den += w;
    const half* vr = tile(t, 1);
    for (int i = 0; i < 4; ++i) acc[i] = fmaf(w, __half2float(vr[lane * 4 + i]), acc[i]);
  }
  for (int i = 0; i < 4; ++i)
    out[seq * out_stride + qh * kHeadDim + lane * 4 + i] = __float2half_rn(acc[i] / den);
}

// ----------------------------------------------------------- host side

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceState {
  bool ready = false;
  void* workspace = nullptr;
  int ctas = 0;
};
constexpr int kMaxDevices = 64;
DeviceState g_state[kMaxDevices];
EncodeTiledFn g_encode = nullptr;
void* g_timeline = nullptr;  // diagnostics build only
std::mutex g_mutex;
long long g_wait_cycles = kWaitCycles;   // rl_attention_test_wait_expiry
int g_drop_first_copy = 0;

// First call per device: driver entry point, shared-memory opt-in, workspace.
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
                  "paged_attention: cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const DeviceFacts& facts = CurrentDeviceFacts();
  if (facts.max_smem_optin < kSmemBytes)
    return Fail(RL_E_WORKSPACE, "paged_attention: device offers %d B of shared memory per block, %d needed",
                facts.max_smem_optin, kSmemBytes);
  cudaError_t e = cudaFuncSetAttribute(PagedAttentionSplitKernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "paged_attention: shared-memory opt-in: %s", cudaGetErrorString(e));
  e = cudaMalloc(&st.workspace, kWorkspaceBytes);
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "paged_attention: workspace: %s", cudaGetErrorString(e));
  e = cudaMemset(st.workspace, 0, kWorkspaceBytes);
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "paged_attention: workspace clear: %s", cudaGetErrorString(e));
  st.ctas = facts.sm_count * kCtasPerSm < kMaxCtas ? facts.sm_count * kCtasPerSm : kMaxCtas;
  st.ready = true;
  return RL_OK;
}

// The pool slice as the 4-D tensor [tile][dim-half][token][64 halves] (strides 4096, 128, 256, 2
// bytes): a box {64, 16, 2, 1} is one whole (block, kv, head) tile laid out as two 128-byte-swizzled
// 16 x 128 B boxes. The box spans heads+1 tiles walked at element stride `heads`, so one copy brings
// the K tile and the V tile of one head (tiles t and t + heads). The tile count is not part of the
// launch contract, so the map claims more tiles than a 180 GB device can hold; only tiles of real
// pages are ever requested.
int EncodeTileMap(const void* pool, int tile_stride, CUtensorMap* map) {
  const cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(kKvBlock), 2, 1ull << 26};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(kHeadDim) * 2, 128, static_cast<cuuint64_t>(kPageBytes)};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(kKvBlock), 2, static_cast<cuuint32_t>(tile_stride + 1)};
  const cuuint32_t estr[4] = {1, 1, 1, static_cast<cuuint32_t>(tile_stride)};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(pool), dims,
                              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Fail(RL_E_BAD_SHAPE, "paged_attention: tile map encode failed (CUresult %d)", static_cast<int>(r));
  return RL_OK;
}

int CheckContract(const char* fn, const void* out, int64_t out_stride, const void* q,
                  int64_t q_stride, const void* pool, const void* tables, const void* lens,
                  int max_blocks, int q_heads, int kv_heads, int head_dim) {
  if (!out || !q || !pool || !tables || !lens) return Fail(RL_E_NULL_POINTER, "%s: null device pointer", fn);
  if (head_dim != kHeadDim) return Fail(RL_E_BAD_SHAPE, "%s: head_dim must be 128", fn);
  if (kv_heads < 1 || q_heads < kv_heads || q_heads % kv_heads != 0)
    return Fail(RL_E_BAD_SHAPE, "%s: num_q_heads must be a positive multiple of num_kv_heads", fn);
  if (max_blocks < 1) return Fail(RL_E_BAD_SHAPE, "%s: max_blocks_per_seq must be >= 1", fn);
  const int64_t width = static_cast<int64_t>(q_heads) * head_dim;
  if (q_stride < width || out_stride < width) return Fail(RL_E_BAD_SHAPE, "%s: row stride smaller than the row", fn);
  return RL_OK;
}

}  // namespace attn
}  // namespace rl

namespace rl {
namespace attn {
void* StaticScratchIfReady(int dev);  // device address of the built-in scratch array once the static launcher ran
}
}  // namespace rl

extern "C" int rl_kernels_init(int device) {
  if (device >= 0) {
    const cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return rl::Fail(static_cast<int>(e), "rl_kernels_init: %s", cudaGetErrorString(e));
  }
  rl::CurrentDeviceFacts();
  rl::attn::DeviceState* st;
  const int rc = rl::attn::EnsureReady(&st);
  return rc != RL_OK ? rc : rl::DecodeLinearInit();
}

#ifdef RL_ATTN_TIMELINE
// Diagnostics build (-DRL_ATTN_TIMELINE): per-warp %globaltimer stamps of the last launch.
extern "C" int rl_debug_attention_timeline(unsigned long long* host_out, int max_entries) {
  cudaDeviceSynchronize();
  const int n = 32 * rl::attn::kMaxCtas * rl::attn::kWarps * 8;
  return cudaMemcpy(host_out, rl::attn::g_timeline, sizeof(unsigned long long) * (n < max_entries ? n : max_entries),
                    cudaMemcpyDeviceToHost);
}
extern "C" int rl_debug_attention_timeline_init(void) {
  const size_t bytes = sizeof(unsigned long long) * 32 * rl::attn::kMaxCtas * rl::attn::kWarps * 8;
  if (!rl::attn::g_timeline) cudaMalloc(&rl::attn::g_timeline, bytes);
  return cudaMemset(rl::attn::g_timeline, 0, bytes);
}
#endif

extern "C" int rl_attention_health(int* flag_out) {
  using namespace rl;
  using namespace rl::attn;
  if (!flag_out) return Fail(RL_E_NULL_POINTER, "rl_attention_health: null pointer");
  *flag_out = 0;
  const int dev = CurrentDeviceIndex();
  // Both scratch areas carry a flag: the allocated workspace of rl_launch_paged_attention_decode and the
  // array built into the library that rl_launch_paged_attention_decode_static uses. Either is read (and
  // cleared) only if its launcher has run on this device; the result is the OR of the two.
  void* areas[2] = {g_state[dev].ready ? g_state[dev].workspace : nullptr, StaticScratchIfReady(dev)};
  if (!areas[0] && !areas[1]) return RL_OK;
  cudaError_t e = cudaDeviceSynchronize();
  for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
    if (!areas[i]) continue;
    int flag = 0;
    e = cudaMemcpy(&flag, areas[i], sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && flag != 0) e = cudaMemset(areas[i], 0, sizeof(int));
    *flag_out |= flag;
  }
  if (e != cudaSuccess) return Fail(static_cast<int>(e), "rl_attention_health: %s", cudaGetErrorString(e));
  return RL_OK;
}

extern "C" int rl_attention_test_wait_expiry(int drop_first_copy, int64_t wait_cycles) {
  rl::attn::g_drop_first_copy = drop_first_copy != 0;
  rl::attn::g_wait_cycles = wait_cycles > 0 ? wait_cycles : rl::attn::kWaitCycles;
  return RL_OK;
}

extern "C" int rl_attention_set_prologue_overlap(int enable) {
  rl::g_launch_overlap = enable != 0;
  return RL_OK;
}

extern "C" int rl_launch_paged_attention_decode(void* out, int64_t out_row_stride, const void* q,
                                                int64_t q_row_stride, const void* kv_pool_layer,
                                                const int32_t* block_tables, const int32_t* seq_lens,
                                                int32_t num_seqs, int32_t max_blocks_per_seq,
                                                int32_t num_q_heads, int32_t num_kv_heads,
                                                int32_t head_dim, float scale, void* stream) {
  using namespace rl;
  using namespace rl::attn;
  if (num_seqs <= 0) return RL_OK;
  int rc = CheckContract("paged_attention_decode", out, out_row_stride, q, q_row_stride, kv_pool_layer,
                         block_tables, seq_lens, max_blocks_per_seq, num_q_heads, num_kv_heads, head_dim);
  if (rc != RL_OK) return rc;
  if (num_q_heads != num_kv_heads * kGroup)
    return Fail(RL_E_BAD_SHAPE, "paged_attention_decode: needs 6 query heads per KV head");
  if ((q_row_stride & 1) || (reinterpret_cast<uintptr_t>(q) & 3))
    return Fail(RL_E_BAD_SHAPE, "paged_attention_decode: q rows must be 4-byte aligned");
  if (!Aligned16(kv_pool_layer))
    return Fail(RL_E_BAD_SHAPE, "paged_attention_decode: the pool slice must be 16-byte aligned");
  DeviceState* st;
  if ((rc = EnsureReady(&st)) != RL_OK) return rc;
  if (num_kv_heads > 8)
    return Fail(RL_E_BAD_SHAPE, "paged_attention_decode: at most 8 KV heads (tensor-copy element stride)");
  CUtensorMap tile_map;
  if ((rc = EncodeTileMap(kv_pool_layer, num_kv_heads, &tile_map)) != RL_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int first = 0; first < num_seqs; first += kMaxSeqsPerLaunch) {
    const int n = num_seqs - first < kMaxSeqsPerLaunch ? num_seqs - first : kMaxSeqsPerLaunch;
    Params p;
    p.out = static_cast<half*>(out) + static_cast<int64_t>(first) * out_row_stride;
    p.out_stride = out_row_stride;
    p.q = static_cast<const half*>(q) + static_cast<int64_t>(first) * q_row_stride;
    p.q_stride = q_row_stride;
    p.tables = block_tables + static_cast<int64_t>(first) * max_blocks_per_seq;
    p.seq_lens = seq_lens + first;
    p.num_seqs = n;
    p.max_blocks = max_blocks_per_seq;
    p.kv_heads = num_kv_heads;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.meta = static_cast<int*>(st->workspace);
    p.partials = reinterpret_cast<float*>(static_cast<int*>(st->workspace) + kMetaInts);
    p.wait_cycles = g_wait_cycles;
    p.drop_first_copy = g_drop_first_copy;
    p.timeline = nullptr;
#ifdef RL_ATTN_TIMELINE
    {  // one region per launch, 32 regions in rotation
      static int launch_seq = 0;
      p.timeline = g_timeline ? static_cast<unsigned long long*>(g_timeline) +
                                    static_cast<size_t>(launch_seq++ % 32) * kMaxCtas * kWarps * 8
                              : nullptr;
    }
#endif
    const cudaError_t e = LaunchOverlapped(PagedAttentionSplitKernel, dim3(st->ctas), dim3(kThreads), kSmemBytes, s,
                                           p, tile_map);
    if (e != cudaSuccess) return Fail(static_cast<int>(e), "paged_attention_decode: %s", cudaGetErrorString(e));
  }
  return LaunchStatus("paged_attention_decode");
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the attention launcher.
//
// Some hosts may not allocate device memory at all: a process that was handed a
// fixed memory budget and a sealed allocator, or a plugin running inside somebody
// else's CUDA context under a "no cudaMalloc after start-up" rule. For them the
// split/merge scratch lives in the library image itself: a file-scope device
// array of kStaticScratchBytes, resident on every GPU that loads the library
// until the process exits. Inputs and outputs are still the caller's.
//
// The first call on a device resolves the array's device address, opts the kernel
// in to its shared memory and looks up one driver entry point; make that call
// outside stream capture. Later calls issue a memset node and the launch only.
// ---------------------------------------------------------------------------
namespace rl {
namespace attn {

constexpr size_t kStaticScratchBytes = kWorkspaceBytes;  // ~1.6 MB: flag, tickets, 2 records x 256 CTAs
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticState {
  bool ready = false;
  void* scratch = nullptr;  // DEVICE address of g_static_scratch on this device
  int ctas = 0;
};
StaticState g_static_state[kMaxDevices];

// Once per device, with that device current. In host code the name g_static_scratch is only a
// handle for the runtime, not a device address - handing it to a kernel would fault or, where the
// GPU can reach host memory, quietly use the wrong bytes - so the real address is asked for here.
int EnsureStaticReady(StaticState** out_state) {
  const int dev = CurrentDeviceIndex();
  StaticState& st = g_static_state[dev];
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
                  "paged_attention (static): cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const DeviceFacts& facts = CurrentDeviceFacts();
  if (facts.max_smem_optin < kSmemBytes)
    return Fail(RL_E_WORKSPACE, "paged_attention (static): %d B of shared memory per block, %d needed",
                facts.max_smem_optin, kSmemBytes);
  if (facts.sm_count * kCtasPerSm > kMaxCtas)
    return Fail(RL_E_TOO_LARGE, "paged_attention (static): %d SMs, the built-in scratch covers %d CTAs",
                facts.sm_count, kMaxCtas);
  cudaError_t e = cudaFuncSetAttribute(PagedAttentionSplitKernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess)
    return Fail(static_cast<int>(e), "paged_attention (static): shared-memory opt-in: %s", cudaGetErrorString(e));
  void* ptr = nullptr;
  e = cudaGetSymbolAddress(&ptr, g_static_scratch);
  if (e != cudaSuccess || !ptr)
    return Fail(e != cudaSuccess ? static_cast<int>(e) : RL_E_WORKSPACE,
                "paged_attention (static): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
  st.scratch = ptr;
  // the same grid as the allocating launcher, so that both cut the page range alike and merge in the same order
  st.ctas = facts.sm_count * kCtasPerSm < kMaxCtas ? facts.sm_count * kCtasPerSm : kMaxCtas;
  st.ready = true;
  return RL_OK;
}

void* StaticScratchIfReady(int dev) { return g_static_state[dev].ready ? g_static_state[dev].scratch : nullptr; }

}  // namespace attn
}  // namespace rl

extern "C" int rl_launch_paged_attention_decode_static(void* out, int64_t out_row_stride, const void* q,
                                                       int64_t q_row_stride, const void* kv_pool_layer,
                                                       const int32_t* block_tables, const int32_t* seq_lens,
                                                       int32_t num_seqs, int32_t max_blocks_per_seq,
                                                       int32_t num_q_heads, int32_t num_kv_heads,
                                                       int32_t head_dim, float scale, void* stream) {
  using namespace rl;
  using namespace rl::attn;
  if (num_seqs <= 0) return RL_OK;
  int rc = CheckContract("paged_attention_decode_static", out, out_row_stride, q, q_row_stride, kv_pool_layer,
                         block_tables, seq_lens, max_blocks_per_seq, num_q_heads, num_kv_heads, head_dim);
  if (rc != RL_OK) return rc;
  if (num_seqs > kMaxSeqsPerLaunch)
    return Fail(RL_E_TOO_LARGE, "paged_attention_decode_static: %d sequences, at most %d per call", num_seqs,
                kMaxSeqsPerLaunch);
  if (num_q_heads != num_kv_heads * kGroup)
    return Fail(RL_E_BAD_SHAPE, "paged_attention_decode_static: needs 6 query heads per KV head");
  if (num_kv_heads > 8)
    return Fail(RL_E_BAD_SHAPE, "paged_attention_decode_static: at most 8 KV heads");
  if ((q_row_stride & 1) || (reinterpret_cast<uintptr_t>(q) & 3) || !Aligned16(kv_pool_layer))
    return Fail(RL_E_BAD_SHAPE, "paged_attention_decode_static: q rows 4-byte, pool slice 16-byte aligned");
  StaticState* st;
  if ((rc = EnsureStaticReady(&st)) != RL_OK) return rc;
  CUtensorMap tile_map;
  if ((rc = EncodeTileMap(kv_pool_layer, num_kv_heads, &tile_map)) != RL_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left. Partial records are fully rewritten before they
  // are read; the ticket counters must start at zero, so they are cleared here, in stream order, before
  // the kernel. The error flag (meta[0]) is NOT cleared: it stays set until rl_attention_health has
  // reported it (the array is zero when the library is loaded).
  const cudaError_t e = cudaMemsetAsync(static_cast<int*>(st->scratch) + kTicketOff, 0, sizeof(int) * kMaxCtas, s);
  if (e != cudaSuccess)
    return Fail(static_cast<int>(e), "paged_attention_decode_static: clearing the counters: %s", cudaGetErrorString(e));
  Params p;
  p.out = static_cast<half*>(out);
  p.out_stride = out_row_stride;
  p.q = static_cast<const half*>(q);
  p.q_stride = q_row_stride;
  p.tables = block_tables;
  p.seq_lens = seq_lens;
  p.num_seqs = num_seqs;
  p.max_blocks = max_blocks_per_seq;
  p.kv_heads = num_kv_heads;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.meta = static_cast<int*>(st->scratch);
  p.partials = reinterpret_cast<float*>(static_cast<int*>(st->scratch) + kMetaInts);
  p.wait_cycles = g_wait_cycles;
  p.drop_first_copy = g_drop_first_copy;
  p.timeline = nullptr;
  PagedAttentionSplitKernel<<<st->ctas, kThreads, kSmemBytes, s>>>(p, tile_map);
  return LaunchStatus("paged_attention_decode_static");
}

extern "C" int rl_launch_paged_attention_decode_check(void* out, int64_t out_row_stride, const void* q,
                                                      int64_t q_row_stride, const void* kv_pool_layer,
                                                      const int32_t* block_tables, const int32_t* seq_lens,
                                                      int32_t num_seqs, int32_t max_blocks_per_seq,
                                                      int32_t num_q_heads, int32_t num_kv_heads,
                                                      int32_t head_dim, float scale, void* stream) {
  using namespace rl;
  using namespace rl::attn;
  if (num_seqs <= 0) return RL_OK;
  const int rc = CheckContract("paged_attention_decode_check", out, out_row_stride, q, q_row_stride,
                               kv_pool_layer, block_tables, seq_lens, max_blocks_per_seq, num_q_heads,
                               num_kv_heads, head_dim);
  if (rc != RL_OK) return rc;
  PagedAttentionCheckKernel<<<dim3(num_seqs, num_q_heads), 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<half*>(out), out_row_stride, static_cast<const half*>(q), q_row_stride,
      static_cast<const half*>(kv_pool_layer), block_tables, seq_lens, max_blocks_per_seq, num_kv_heads,
      num_q_heads / num_kv_heads, scale);
  return LaunchStatus("paged_attention_decode_check");
}
