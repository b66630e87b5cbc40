// PTX wrappers for running one tile pair on a cluster of two CTAs (tcgen05 cta_group::2): the
// two CTAs sit on the two SMs of one TPC, each keeps its own 128 rows of A and HALF of the B
// tile in its shared memory, and one thread of the leader CTA (cluster rank 0) issues a single
// M=256 instruction that both tensor cores execute, each writing its 128 accumulator rows into
// its own tensor memory. Every instruction of the tcgen05 family in such a kernel carries
// cta_group::2. No load here uses cluster multicast: each CTA fetches its own half, and only
// the completion signal (the mbarrier of the leader, tcgen05.commit to both CTAs) crosses.
#pragma once
#include <cstdint>
#include <cuda.h>

#include "ptx_sm100.cuh"

namespace mono {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
// One arrival on a barrier anywhere in the cluster (address from map_to_cta). Default semantics
// (release at CTA scope): a cluster-scope release would first wait for every earlier global store of
// the thread, which is far too slow for a per-slab signal.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Hardware barrier over all threads of both CTAs.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// 2-D tiled load into THIS CTA's shared memory whose completion bytes are counted on a barrier
// that may live in the peer CTA (`bar_cluster` from map_to_cta). x is a byte coordinate, multiple of 16.
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* m, uint32_t x, uint32_t y, void* dst,
                                                 uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}

// Tensor memory of the pair: the same warp of BOTH CTAs executes these.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem of both CTAs] (+)= A * B^T with M = 256 (128 rows per CTA), issued by ONE thread of the
// leader CTA. The descriptors are shared-memory offsets valid in both CTAs: each CTA reads its own A
// rows and its own half of the N rows of B at those offsets.
__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this shared-memory offset in BOTH CTAs once every MMA issued so
// far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

}  // namespace mono
