// Inline-PTX helpers for sm_100a: mbarrier, bulk (TMA) copies, tcgen05/TMEM.
// Every wait in this file is bounded: it returns false after `kSpinLimit` polls so that a
// kernel can record a status word and leave instead of spinning forever.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace mnb {
namespace ptx {

constexpr std::uint32_t kSpinLimit = 1u << 18; // polls; each failed poll backs off ~64 ns (tens of ms in all)

__device__ __forceinline__ std::uint32_t SmemAddr(const void *ptr) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(ptr));
}

__device__ __forceinline__ void MbarInit(std::uint64_t *bar, std::uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count)
               : "memory");
}

__device__ __forceinline__ void FenceMbarInit() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void FenceProxyAsyncShared() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void MbarArrive(std::uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}

__device__ __forceinline__ void MbarArriveExpectTx(std::uint64_t *bar, std::uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool MbarTryWait(std::uint64_t *bar, std::uint32_t parity) {
  std::uint32_t done;
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t"
               "}"
               : "=r"(done)
               : "r"(SmemAddr(bar)), "r"(parity)
               : "memory");
  return done != 0;
}

// Bounded wait. Returns false when the phase did not complete within the poll budget.
__device__ __forceinline__ bool MbarWait(std::uint64_t *bar, std::uint32_t parity) {
  for (std::uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (MbarTryWait(bar, parity)) {
      return true;
    }
    if (spin > 8) {
      __nanosleep(128); // try_wait already suspends for a while; keep pollers off the issue ports
    }
  }
  return false;
}

// Same bound, for waits on the critical path of a pipeline (a hand-off that is normally a few
// hundred nanoseconds away): keeps polling without backing off for longer before it sleeps.
__device__ __forceinline__ bool MbarWaitHot(std::uint64_t *bar, std::uint32_t parity) {
  for (std::uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (MbarTryWait(bar, parity)) {
      return true;
    }
    if (spin > 2048) {
      __nanosleep(128);
    }
  }
  return false;
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// Both addresses must be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void BulkLoad(void *smem_dst, const void *gmem_src, std::uint32_t bytes,
                                         std::uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(SmemAddr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(SmemAddr(bar))
      : "memory");
}

// 2-D tiled TMA load (no multicast), coordinates innermost first.
__device__ __forceinline__ void TmaLoad2D(void *smem_dst, const void *tensor_map, int x, int y,
                                          std::uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3}], [%4];" ::"r"(SmemAddr(smem_dst)),
               "l"(tensor_map), "r"(x), "r"(y), "r"(SmemAddr(bar))
               : "memory");
}

__device__ __forceinline__ void PrefetchTensorMap(const void *tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}

// ---- programmatic dependent launch ----------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start while the
// kernel before it in the stream is still draining. GridDependencyLaunch() lets the NEXT
// kernel's CTAs be scheduled as soon as SM resources free up; GridDependencyWait() blocks until
// the PREVIOUS kernel has completed and its writes are visible. Only memory the previous
// kernel cannot have written (the constant weights) may be touched before the wait.
__device__ __forceinline__ void GridDependencyLaunch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void GridDependencyWait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------------------------

// Whole-warp instruction. Writes the TMEM base address of `columns` columns to *smem_result.
__device__ __forceinline__ void TmemAlloc(std::uint32_t *smem_result, std::uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   SmemAddr(smem_result)),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void TmemRelinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void TmemDealloc(std::uint32_t taddr, std::uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}

__device__ __forceinline__ void TcFenceBefore() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void TcFenceAfter() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 x bf16 -> fp32. One thread issues.
__device__ __forceinline__ void UmmaBf16(std::uint32_t tmem_d, std::uint64_t desc_a,
                                         std::uint64_t desc_b, std::uint32_t idesc,
                                         std::uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
               "}" ::"r"(tmem_d),
               "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}

// Makes `bar` complete one arrival once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void UmmaCommit(std::uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   SmemAddr(bar))
               : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster share one MMA -------------------------------
// The MMA is issued by one thread of the even CTA; each CTA supplies its own 128 rows of the A
// operand and half of the B operand from the same offsets of its shared memory, and receives its
// 128 rows of D in its own TMEM. Allocation and release are executed by the same warp of both CTAs.

__device__ __forceinline__ std::uint32_t ClusterCtaRank() {
  std::uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

// Cluster-wide barrier over all threads of both CTAs (every thread executes both halves).
__device__ __forceinline__ void ClusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\t"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of `local` (a shared-memory address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ std::uint32_t MapToCta(std::uint32_t local, std::uint32_t rank) {
  std::uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}

// One arrival on a barrier of any CTA of the cluster (address from MapToCta). This is the form that
// hands shared memory written by a CTA's threads (followed by a proxy fence) to an MMA of the CTA
// pair; the variant with a release at cluster scope measured 0.5 us more per arrival.
__device__ __forceinline__ void MbarArriveCluster(std::uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void TmemAllocPair(std::uint32_t *smem_result, std::uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   SmemAddr(smem_result)),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void TmemRelinquishPair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void TmemDeallocPair(std::uint32_t taddr, std::uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}

// D[tmem of both CTAs] (+)= A * B over the pair: 256 x N x 16 per instruction. One thread of the
// even CTA issues; the descriptors hold offsets that are valid in both CTAs.
__device__ __forceinline__ void UmmaBf16Pair(std::uint32_t tmem_d, std::uint64_t desc_a,
                                             std::uint64_t desc_b, std::uint32_t idesc,
                                             std::uint32_t accumulate) {
  asm volatile("{\n\t"
               ".reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
               "}" ::"r"(tmem_d),
               "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
               : "memory");
}

// One arrival on `bar` in each CTA of `cta_mask` (the barrier sits at the same offset in both) once
// every pair MMA issued so far by this thread has finished.
__device__ __forceinline__ void UmmaCommitPair(std::uint64_t *bar, std::uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
                   "r"(SmemAddr(bar)),
               "h"(cta_mask)
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane (base+i).
__device__ __forceinline__ void TmemLoad32x32(std::uint32_t taddr, std::uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void TmemLoadWait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with
// the 128-byte swizzle (what a TMA box of 64 bf16 with SWIZZLE_128B produces): 8-row groups
// are 1024 bytes apart. Field layout: start address >> 4 in bits [0,14), leading byte offset
// >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in [46,48),
// layout type (2 = 128-byte swizzle) in [61,64).
__device__ __forceinline__ std::uint64_t UmmaDescKMajorSw128(std::uint32_t smem_addr) {
  std::uint64_t desc = 0;
  desc |= static_cast<std::uint64_t>((smem_addr & 0x3ffffu) >> 4);
  desc |= static_cast<std::uint64_t>(1) << 16;           // leading byte offset (unused here)
  desc |= static_cast<std::uint64_t>(1024 >> 4) << 32;   // stride between 8-row groups
  desc |= static_cast<std::uint64_t>(1) << 46;           // descriptor version
  desc |= static_cast<std::uint64_t>(2) << 61;           // SWIZZLE_128B
  return desc;
}

// Instruction descriptor for kind::f16 with bf16 A and B (both K-major), fp32 accumulate.
// c_format [4,6) = 1 (f32), a_format [7,10) = 1 (bf16), b_format [10,13) = 1 (bf16),
// a_major bit 15 = 0, b_major bit 16 = 0, n >> 3 in [17,23), m >> 4 in [24,29).
__host__ __device__ constexpr std::uint32_t UmmaIdescBf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<std::uint32_t>(n >> 3) << 17) |
         (static_cast<std::uint32_t>(m >> 4) << 24);
}

} // namespace ptx
} // namespace mnb
