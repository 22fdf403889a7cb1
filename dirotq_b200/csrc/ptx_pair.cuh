// Inline PTX for CTA pairs (clusters of two CTAs on neighbouring SMs driving ONE tcgen05.mma with cta_group::2):
// cluster rank and barrier, addresses in the peer's shared memory, TMA loads whose completion is counted on the
// leader's mbarrier, pair-wide TMEM allocation, pair UMMAs / scale-factor copies / commits.  Every load here brings
// its bytes into the issuing CTA's own shared memory only; the two CTAs of a pair each fetch their own halves.
#pragma once
#include <cstdint>
#include "ptx.cuh"

namespace dq {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// all threads of both CTAs; orders the shared-memory writes before it (barrier initialisation) cluster-wide
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// one arrival on an mbarrier that may live in the peer CTA (shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The same without memory ordering: for hand-offs whose payload is TENSOR memory (made complete by tcgen05.wait::ld /
// wait::st before the arrival), not shared or global memory.  A cluster-scope release has to drain the thread's
// earlier stores first and costs on the order of a microsecond per arrival on this kernel's critical path.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// 2-D tiled load into THIS CTA's shared memory; the bytes are counted on `bar`, a shared::cluster address that may
// name the leader CTA's mbarrier (the cta_group::2 form is what allows the barrier to sit in the peer).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// ---- TMEM for a pair: one full warp of EACH CTA calls these with the same arguments ----------------------------------
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// completion of all pair UMMAs issued so far by this thread -> one arrival on `bar` (shared::cluster address: own or peer)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 rows x 16 bytes of EACH CTA's shared memory -> that CTA's TMEM lanes 0..31 (4 columns), replicated to all four
// lane quarters; issued once by the leader
__device__ __forceinline__ void tmem_cp_32x128b_x4_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// E2M1 x E2M1 with UE4M3 scale factors, 256 x N x 64 over the pair: each CTA contributes its 128 rows of A, its
// N/2 rows of B and holds its 128 x N half of the accumulator
__device__ __forceinline__ void umma_nvf4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}

// The four K = 16 pair UMMAs of one 64-wide bf16 operand stage, both operands through shared-memory descriptors given as
// low words (address >> 4, advancing by 2 = 32 bytes per step) and one common high word; `accum0` = 0 clears the
// accumulator first.
__device__ __forceinline__ void umma_f16_ss_x4_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                                    uint32_t accum0) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 da, db;\n\t.reg .b32 x, y;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t"
      "add.u32 x, %1, 2;\n\tadd.u32 y, %2, 2;\n\tmov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, t;\n\t"
      "add.u32 x, %1, 4;\n\tadd.u32 y, %2, 4;\n\tmov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, t;\n\t"
      "add.u32 x, %1, 6;\n\tadd.u32 y, %2, 6;\n\tmov.b64 da, {x, %3};\n\tmov.b64 db, {y, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, t;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accum0)
      : "memory");
}

}  // namespace dq
