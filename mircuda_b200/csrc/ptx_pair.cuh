// Inline-PTX wrappers for CTA pairs (thread-block clusters of two): cluster rank and
// barriers, remote mbarrier arrivals, TMA loads whose completion is counted on the peer
// CTA's mbarrier, and the cta_group::2 forms of tensor-memory allocation, tcgen05.cp,
// tcgen05.mma and tcgen05.commit. No load in this file replicates data to several CTAs;
// only the commit (an mbarrier arrival, not a data transfer) addresses both CTAs at once.
#pragma once

#include <cstdint>

#include "ptx.cuh"

namespace mircuda_b200::ptx {

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
}

__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}

// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t shared_address, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(shared_address), "r"(rank));
  return remote;
}

__device__ __forceinline__ void mbarrier_arrive_cluster(uint32_t cluster_address) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_address)
               : "memory");
}

__device__ __forceinline__ void mbarrier_arrive_expect_tx_cluster(uint32_t cluster_address,
                                                                  uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(
                   cluster_address),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbarrier_try_wait_cluster(uint64_t* barrier, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_address(barrier)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait on a barrier of this CTA whose arrivals may come from the peer CTA.
__device__ __forceinline__ bool mbarrier_wait_cluster(uint64_t* barrier, uint32_t parity,
                                                      volatile uint32_t* abort) {
  return mbarrier_wait(barrier, parity, abort);
}

// Tiled loads into this CTA's shared memory whose byte count is reported to an mbarrier
// that may live in the peer CTA (given as a cluster-space address).
__device__ __forceinline__ void tma_load_2d_pair(void* destination, const void* tensor_map,
                                                 uint32_t barrier_cluster_address, int32_t x,
                                                 int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_address(destination)),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(barrier_cluster_address), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(void* destination, const void* tensor_map,
                                                 uint32_t barrier_cluster_address, int32_t x,
                                                 int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_address(destination)),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(barrier_cluster_address), "r"(x), "r"(y),
      "r"(z)
      : "memory");
}

__device__ __forceinline__ void tmem_allocate_pair(uint32_t* shared_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_address(shared_result)),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_deallocate_pair(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns)
               : "memory");
}

// One mbarrier arrival in each CTA named by `cta_mask` (same barrier offset) once every
// tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* barrier, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;"
      ::"r"(smem_address(barrier)),
      "h"(cta_mask)
      : "memory");
}

// Scale atom copy shared -> tensor memory in both CTAs of the pair (each from its own
// shared memory at the same offset).
__device__ __forceinline__ void tcgen05_copy_scales_pair(uint32_t tmem_address, uint64_t descriptor) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_address),
               "l"(descriptor)
               : "memory");
}

__device__ __forceinline__ void mma_mxf8f6f4_block_scale_pair(uint32_t d_tmem, uint64_t a_descriptor,
                                                              uint64_t b_descriptor, uint32_t idesc,
                                                              uint32_t scale_a_tmem,
                                                              uint32_t scale_b_tmem, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      ::"r"(d_tmem),
      "l"(a_descriptor), "l"(b_descriptor), "r"(idesc), "r"(accumulate ? 1u : 0u),
      "r"(scale_a_tmem), "r"(scale_b_tmem)
      : "memory");
}

__device__ __forceinline__ void mma_nvf4_block16_pair(uint32_t d_tmem, uint64_t a_descriptor,
                                                      uint64_t b_descriptor, uint32_t idesc,
                                                      uint32_t scale_a_tmem, uint32_t scale_b_tmem,
                                                      bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], "
      "p;\n\t"
      "}\n"
      ::"r"(d_tmem),
      "l"(a_descriptor), "l"(b_descriptor), "r"(idesc), "r"(accumulate ? 1u : 0u),
      "r"(scale_a_tmem), "r"(scale_b_tmem)
      : "memory");
}

// kind::f16 (f16 / bf16 operands) and kind::f8f6f4 without block scales, fp32 accumulator, on a
// CTA pair: M = 256 rows (128 per CTA), each CTA supplying half of the N rows of B.
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t a_descriptor, uint64_t b_descriptor,
                                             uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem),
      "l"(a_descriptor), "l"(b_descriptor), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}

__device__ __forceinline__ void mma_f8f6f4_pair(uint32_t d_tmem, uint64_t a_descriptor, uint64_t b_descriptor,
                                                uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem),
      "l"(a_descriptor), "l"(b_descriptor), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}

}  // namespace mircuda_b200::ptx
