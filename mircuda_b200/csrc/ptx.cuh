// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA
// (cp.async.bulk[.tensor]), tensor memory (tcgen05.alloc/ld/cp) and tcgen05.mma.
// Every wait is bounded: it gives up after a fixed number of polls and reports it, so a
// protocol error turns into a status code instead of a hung GPU.
#pragma once

#include <cstdint>

namespace mircuda_b200::ptx {

__device__ __forceinline__ uint32_t smem_address(const void* pointer) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t predicate = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(predicate));
  return predicate != 0;
}

// ------------------------------------------------- programmatic dependent launch
// A kernel launched with cudaLaunchAttributeProgrammaticStreamSerialization may start while the
// kernel before it on the stream still runs; it must not touch global memory that kernel (or
// anything before it) writes or reads-then-overwrites until dependency_wait() has returned.
// Launched without the attribute, both instructions do nothing.

__device__ __forceinline__ void dependency_launch_next() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---------------------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbarrier_init(uint64_t* barrier, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(barrier)),
               "r"(arrivals)
               : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbarrier_arrive(uint64_t* barrier) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(barrier))
               : "memory");
}

__device__ __forceinline__ void mbarrier_arrive_expect_tx(uint64_t* barrier, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                   smem_address(barrier)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbarrier_try_wait(uint64_t* barrier, uint32_t parity) {
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

// Release/acquire fence at device scope. `__threadfence()` is the sequentially consistent
// fence, which the hardware orders globally: hundreds of CTAs issuing it at the same moment
// (the end of a split-K kernel) were measured to queue for 10 us and more. The hand-overs in
// this library only need release/acquire ordering around an atomic counter.
__device__ __forceinline__ void fence_acq_rel_gpu() {
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
  return now;
}

// Polls until the phase with the given parity completes, `abort` becomes non-zero, or the
// time budget runs out. Returns false in the last two cases (and raises `abort` itself when
// the budget ran out), so that every role of the CTA leaves its loop and the kernel can
// finish cleanly. The bound is wall time, not a poll count: one try_wait may itself block
// for a hardware-defined slice that can be as long as a millisecond. Half a second is
// orders of magnitude beyond any legitimate wait in these kernels.
constexpr uint64_t kWaitBudgetNs = 500ull * 1000ull * 1000ull;

// PAUSE_NS > 0 puts the warp to sleep for about that long between polls: for roles that wait a
// long time beside warps that compute (a tight poll loop takes issue slots from them).
template <uint64_t BUDGET_NS = kWaitBudgetNs, uint32_t PAUSE_NS = 0>
__device__ __forceinline__ bool mbarrier_wait(uint64_t* barrier, uint32_t parity,
                                              volatile uint32_t* abort) {
  if (mbarrier_try_wait(barrier, parity)) return true;
  const uint64_t start = global_timer_ns();
  for (uint32_t poll = 1;; ++poll) {
    if (mbarrier_try_wait(barrier, parity)) return true;
    if constexpr (PAUSE_NS != 0u) __nanosleep(PAUSE_NS);
    if ((poll & 15u) == 0u) {
      if (*abort != 0u) return false;
      if (global_timer_ns() - start > BUDGET_NS) break;
    }
  }
  *abort = 1u;
  return false;
}

// --------------------------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tensor_map(const void* tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensor_map))
               : "memory");
}

// 2-D tiled load global -> shared, completion counted in bytes on an mbarrier. x is the
// innermost coordinate; x times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* destination, const void* tensor_map,
                                            uint64_t* barrier, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_address(destination)),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(smem_address(barrier)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* destination, const void* tensor_map,
                                            uint64_t* barrier, int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_address(destination)),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(smem_address(barrier)), "r"(x), "r"(y),
      "r"(z)
      : "memory");
}

// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void* destination, const void* source, uint32_t bytes,
                                          uint64_t* barrier) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_address(destination)),
      "l"(reinterpret_cast<uint64_t>(source)), "r"(bytes), "r"(smem_address(barrier))
      : "memory");
}

// 2-D tiled store shared -> global (bulk-group completion).
__device__ __forceinline__ void tma_store_2d(const void* tensor_map, const void* source, int32_t x,
                                             int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(tensor_map)),
      "r"(smem_address(source)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int Pending>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(Pending) : "memory");
}

template <int Pending>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(Pending) : "memory");
}

// ----------------------------------------------------------------------- tensor memory

__device__ __forceinline__ void tmem_allocate(uint32_t* shared_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_address(shared_result)),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_deallocate(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrive on an mbarrier once every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void tcgen05_commit(uint64_t* barrier) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_address(barrier))
               : "memory");
}

// Shared memory -> tensor memory copy of one 32-row x 16-byte block, replicated into all four
// 32-lane sub-partitions. This is how a 512-byte block-scale atom reaches the MMA.
__device__ __forceinline__ void tcgen05_copy_scales(uint32_t tmem_address, uint64_t descriptor) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_address),
               "l"(descriptor)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane base+i.
__device__ __forceinline__ void tmem_load_32x32(uint32_t address, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(address)
      : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------- MMA descriptors

// Shared-memory matrix descriptor (64 bit): start address >> 4 in bits [0,14), leading byte
// offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in
// [46,48), swizzle mode in [61,64) (0 none, 2 = 128-byte, 4 = 64-byte, 6 = 32-byte).
constexpr uint64_t kSwizzleNone = 0, kSwizzle128B = 2;

__device__ __forceinline__ uint64_t make_smem_descriptor(uint32_t shared_address,
                                                         uint32_t leading_bytes,
                                                         uint32_t stride_bytes, uint64_t swizzle) {
  uint64_t descriptor = 0;
  descriptor |= static_cast<uint64_t>((shared_address & 0x3ffffu) >> 4);
  descriptor |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3fffu) << 16;
  descriptor |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3fffu) << 32;
  descriptor |= 1ull << 46;
  descriptor |= swizzle << 61;
  return descriptor;
}

// K-major operand tile whose rows are exactly one 128-byte swizzle span: 8-row groups are
// 1024 bytes apart. Advancing along K inside the span adds the byte offset to the start.
__device__ __forceinline__ uint64_t make_k_major_sw128_descriptor(uint32_t shared_address) {
  return make_smem_descriptor(shared_address, 16, 1024, kSwizzle128B);
}

// Scale atom for tcgen05.cp: 32 rows of 16 bytes, unswizzled; 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t make_scale_descriptor(uint32_t shared_address) {
  return make_smem_descriptor(shared_address, 0, 128, kSwizzleNone);
}

// Instruction descriptor for block-scaled MMA (kind::mxf8f6f4 / mxf4nvf4), both operands
// K-major: B scale id [4,6), A format [7,10), B format [10,13), N>>3 [17,23), scale format
// bit 23 (0 = UE4M3, 1 = UE8M0), M>>4 [24,29), A scale id [29,31).
constexpr uint32_t kFormatE4M3 = 0, kFormatE2M1_in_f8f6f4 = 5, kFormatE2M1_mxf4 = 1;

__host__ __device__ constexpr uint32_t make_block_scaled_idesc(uint32_t a_format,
                                                               uint32_t b_format, uint32_t m,
                                                               uint32_t n, bool scale_is_ue8m0) {
  return (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) |
         (scale_is_ue8m0 ? (1u << 23) : 0u) | ((m >> 4) << 24);
}

__host__ __device__ constexpr uint32_t with_scale_ids(uint32_t idesc, uint32_t a_id,
                                                      uint32_t b_id) {
  return idesc | (b_id << 4) | (a_id << 29);
}

// Instruction descriptor for kind::f16 (bf16 or f16 operands, fp32 accumulator), K-major:
// C format [4,6) = 1 (f32), A format [7,10), B format [10,13) (0 f16, 1 bf16), N>>3 [17,23),
// M>>4 [24,29).
__host__ __device__ constexpr uint32_t make_f16_idesc(bool bf16, uint32_t m, uint32_t n) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem] with per-block scales read from tensor memory.
__device__ __forceinline__ void mma_mxf8f6f4_block_scale(uint32_t d_tmem, uint64_t a_descriptor,
                                                         uint64_t b_descriptor, uint32_t idesc,
                                                         uint32_t scale_a_tmem,
                                                         uint32_t scale_b_tmem, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      ::"r"(d_tmem),
      "l"(a_descriptor), "l"(b_descriptor), "r"(idesc), "r"(accumulate ? 1u : 0u),
      "r"(scale_a_tmem), "r"(scale_b_tmem)
      : "memory");
}

// NVFP4: E2M1 operands, one UE4M3 scale per 16 elements along K (K = 64 per instruction).
__device__ __forceinline__ void mma_nvf4_block16(uint32_t d_tmem, uint64_t a_descriptor,
                                                 uint64_t b_descriptor, uint32_t idesc,
                                                 uint32_t scale_a_tmem, uint32_t scale_b_tmem,
                                                 bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], "
      "p;\n\t"
      "}\n"
      ::"r"(d_tmem),
      "l"(a_descriptor), "l"(b_descriptor), "r"(idesc), "r"(accumulate ? 1u : 0u),
      "r"(scale_a_tmem), "r"(scale_b_tmem)
      : "memory");
}

// bf16 / f16 operands, fp32 accumulation (K = 16 per instruction).
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_descriptor,
                                        uint64_t b_descriptor, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem),
      "l"(a_descriptor), "l"(b_descriptor), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}

// kind::f8f6f4 without block scales: one-byte operands (here e4m3, format 0 in the descriptor
// built by make_f16_idesc(false, m, n)), fp32 accumulator, 32 bytes of K per instruction.
__device__ __forceinline__ void mma_f8f6f4(uint32_t d_tmem, uint64_t a_descriptor,
                                           uint64_t b_descriptor, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem),
      "l"(a_descriptor), "l"(b_descriptor), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}

}  // namespace mircuda_b200::ptx
