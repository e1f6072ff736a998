// 5th-generation tensor core (tcgen05) and tensor memory (TMEM) in inline PTX:
// allocation, shared-memory matrix descriptors, the instruction descriptor,
// MMA issue, commit to an mbarrier and accumulator read-back.  sm_100a only.
// Upstream's contraction is `tl.dot(a, b.T, accumulator)`
// (symm_mem_recipes/triton_all_gather_matmul.py:185), which Triton lowers to
// Hopper's warpgroup MMA; this header is its Blackwell counterpart written out.
#pragma once
#include <stdint.h>

#include "mbarrier.cuh"

namespace smr {

// ---- TMEM allocation (one warp, all 32 lanes) ------------------------------
// `ncols`: power of two in [32, 512].  The base address is written to smem.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_thread_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after_thread_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- descriptors ------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major bf16 tile whose rows are 128
// bytes (64 elements) and which TMA wrote with the 128-byte swizzle:
//   bits [0,14)  start address >> 4
//   bits [16,30) leading-dimension byte offset >> 4 (unused for swizzled K-major; 1)
//   bits [32,46) stride-dimension byte offset >> 4 = 1024 B between 8-row groups
//   bits [46,48) descriptor version = 1 on sm_100
//   bits [61,64) layout = 2 (SWIZZLE_128B)
// The tile base must be 1024-byte aligned; stepping K by 16 elements inside the
// 128-byte row adds 32 bytes (2 in descriptor units) to the start address.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1u << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1u << 46;
  d |= (uint64_t)2u << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 A and B (both K-major) and an
// fp32 accumulator:  c_format=F32 at bit 4, a_format=BF16 at bit 7,
// b_format=BF16 at bit 10, N>>3 at bit 17, M>>4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc_bf16_f32(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Instruction descriptor for kind::f8f6f4 with e4m3 A and B (format code 0 in
// both operand fields, both K-major) and an fp32 accumulator.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3_f32(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- MMA ---------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread
// has completed (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar)) : "memory");
}

// ---- accumulator read-back ----------------------------------------------------
// Each lane of the warp reads 32 consecutive fp32 columns of its own TMEM lane
// (lane = 32 * (warp_id % 4) + lane_id, encoded in bits [31:16] of taddr).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace smr
