// PTX building blocks of the tensor-memory kernels (sm_100a): mbarriers with bounded waits, TMA tile
// loads with L2 policies, tcgen05 shared-memory / instruction descriptors, MMA issue and commit,
// tensor-memory loads, thread-block-cluster helpers. Every load is into the issuing CTA's own shared
// memory; nothing here addresses another GPU.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace rl {
namespace tc {

constexpr long long kWaitCycles = 2000000000LL;  // ~1 s: a wait that never completes is reported, not spun on


__device__ __forceinline__ uint32_t SmemAddr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void MbarInit(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void MbarExpectTx(uint32_t bar, int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// Bounded wait: false when the phase never completed within kWaitCycles.
__device__ __forceinline__ bool MbarWait(uint32_t bar, int parity) {
  if (MbarTryWait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!MbarTryWait(bar, parity)) {
    if (clock64() - t0 > kWaitCycles) return false;
  }
  return true;
}
__device__ __forceinline__ uint64_t L2PolicyEvictFirst() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t L2PolicyEvictNormal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t L2PolicyEvictLast() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// One box of a 2-D tensor map (x = k element, y = row) into this CTA's shared memory, completion
// counted in bytes on `bar`. x is always a multiple of 64 halves, so the copy starts 128-byte aligned.
__device__ __forceinline__ void TmaLoad2D(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar,
                                          uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 halves), written
// by TMA with the 128-byte swizzle: 8-row groups 1024 bytes apart (stride byte offset), leading
// byte offset unused for swizzled K-major tiles (encoded 1), descriptor version 1, layout type 2
// (128-byte swizzle). Fields are in 16-byte units. The tile base is 1024-byte aligned; advancing
// the start address by 32 bytes steps one K=16 slice inside the swizzle row.
__device__ __forceinline__ uint64_t TileDesc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}
// Instruction descriptor: FP32 accumulate (bits 4-5 = 1), A and B FP16 (0), both K-major (0),
// N >> 3 at bit 17, M >> 4 at bit 24 (M = 128).
__device__ __forceinline__ uint32_t InstrDesc(int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}
__device__ __forceinline__ void Umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                     uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void UmmaCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// The same two, called by ALL 32 lanes of a converged warp with identical arguments: one elected lane
// issues. Descriptors that change from one loop trip to the next then stay in the warp-uniform
// datapath; issued from inside a `lane == 0` branch they are moved there one product at a time, which
// was measured to cost 82 cycles per M = 128, N = 128 product against the tensor pipe's 64.
__device__ __forceinline__ void UmmaElected(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void UmmaCommitElected(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar)
      : "memory");
}
// 16 consecutive accumulator columns of this thread's tensor-memory lane. The load is asynchronous:
// the values may be used only after TmemWaitLoads, which takes the registers as read-write operands
// so that no use can be scheduled ahead of it.
__device__ __forceinline__ void TmemLoad16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void TmemWaitLoads(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Thread-block cluster: barrier over all threads of all CTAs (split into arrive and wait), the
// address of a peer CTA's shared memory, and a store to it.
__device__ __forceinline__ void ClusterArriveRelaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void ClusterWait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t PeerSmemAddr(uint32_t local_addr, int cta_rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(cta_rank));
  return a;
}
// 16 bytes into a peer CTA's shared memory; completion is counted in bytes on the peer's mbarrier.
__device__ __forceinline__ void StAsyncPeerF32x4(uint32_t addr, uint32_t mbar, float4 v) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1,%2,%3,%4}, [%5];" ::"r"(addr),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(mbar)
               : "memory");
}

}  // namespace tc
}  // namespace rl
