// The PTX instructions specific to CTA pairs (thread-block cluster of 2, tcgen05 cta_group::2), each
// behind a small function; the rest comes from ptx_tcgen05.cuh.  The CPU tests (tests/cpu_emu/) provide
// stand-ins with the same names.
#pragma once

#include "ptx_tcgen05.cuh"

#ifndef SHREWQ_CPU_EMU
namespace shrewq {
namespace {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.aligned;" ::: "memory"); }

__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); }

// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}

// arrive on a barrier of any CTA of the cluster (address from map_to_cta)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// pair TMA load: the data lands in THIS CTA's shared memory, the bytes complete on the LEADER
// CTA's barrier (same offset in CTA 0 of the cluster)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void *tmap, int c0, int c1, uint32_t bar_local) {
    const uint32_t bar_leader = map_to_cta(bar_local, 0);
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar_leader), "r"(c0), "r"(c1)
        : "memory");
}

// completion of all prior MMAs of this thread arrives once on the barrier at this shared-memory offset in
// BOTH CTAs of the pair (CTA mask 0b11)
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}

// D[256 x 256] (+)= A[256 x 16, TMEM of both CTAs] * B[256 x 16, shared memory of both CTAs]^T
__device__ __forceinline__ void tc_mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// all 512 columns in both CTAs of the pair; one warp of EACH CTA issues it, same shared-memory offset
__device__ __forceinline__ void tc_alloc_512_pair(uint32_t result_smem) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(result_smem) : "memory");
}
__device__ __forceinline__ void tc_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc_512_pair(uint32_t tmem_base) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
}

}  // namespace
}  // namespace shrewq

#define SHREWQ_CLUSTER_OF_2 __cluster_dims__(2, 1, 1)
#endif  // SHREWQ_CPU_EMU
