// Inline-PTX wrappers for CTA pairs (a thread-block cluster of two CTAs on the two SMs of one TPC) driving
// tcgen05 with cta_group::2: one thread of the leader CTA (cluster rank 0) issues an MMA that runs on both
// SMs; each CTA holds its own 128 rows of A and of the accumulator, and one half (by N) of B.
//
// No instruction here copies with cluster-wide broadcast: every CTA loads its own operand halves with the plain
// TMA load of ptx.cuh, and a completion is made known to the other CTA with a remote mbarrier arrive or with
// a second tcgen05.commit aimed at the peer's barrier.
#pragma once

#include "ptx.cuh"

namespace ab200 {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Full barrier over all threads of the cluster (hardware barrier; every thread of both CTAs must reach it).
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cta address of this CTA -> shared::cluster address of the same offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
// Arrive on an mbarrier of any CTA of the cluster (address from mapa_shared). Default semantics (release at
// CTA scope): what the arrival reports is complete by construction (a TMA transaction count observed, a
// tcgen05.wait::ld / ::st passed), and a cluster-scope release was measured to stall the arriving thread for
// 1000-2000 cycles.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Tensor memory of the pair: the same columns are allocated in both CTAs. One warp of EACH CTA (the same
// warp index) executes these.
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Arrive on ONE mbarrier (shared::cluster address: an own shared::cta address, or a peer address from
// mapa_shared) once every cta_group::2 MMA issued so far by this thread has completed on both SMs.
__device__ __forceinline__ void tc_commit2(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}
// The same completion reported to the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void tc_commit2_both(uint64_t* bar) {
  const uint32_t a = smem_u32(bar);
  tc_commit2(mapa_shared(a, 0));
  tc_commit2(mapa_shared(a, 1));
}

// D[256 x N] (+)= A[256 x K16] * B[N x K16]^T over the pair: rows [0,128) of A and D belong to the leader,
// [128,256) to the peer; each CTA's shared memory holds N/2 rows (K-major) or columns (MN-major) of B at the
// offset the descriptor names. The instruction descriptor carries M = 256 and the full N.
__device__ __forceinline__ void umma_ss2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A from tensor memory: each CTA's TMEM holds its own 128 rows of A.
__device__ __forceinline__ void umma_ts2(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

}  // namespace ab200
