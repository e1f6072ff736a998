// multimem (NVLS) loads / stores on a multicast address: one instruction is
// executed by the NVSwitch against the same offset of every bound GPU.
#pragma once
#include "vec.cuh"

namespace smr {

// Sum of the 8 bf16 at `mc` over all bound GPUs, accumulated in fp32 inside the
// switch and rounded to bf16 once.
__device__ __forceinline__ Vec16 multimem_ld_reduce_bf16x8(const void* mc) {
  Vec16 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
// Broadcast 16 bytes to the same offset of every bound GPU.
__device__ __forceinline__ void multimem_st_16(void* mc, const Vec16& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// fp32 x4 sum over all bound GPUs
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_red_add_u32(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

}  // namespace smr
