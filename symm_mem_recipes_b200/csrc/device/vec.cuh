// 128-bit global loads / stores and packed bf16 arithmetic.
//
// `add_bf16x8` is the arithmetic of the upstream all-reduce
// (symm_mem_recipes/triton_one_shot_all_reduce.py:32-56): four add.bf16x2,
// i.e. bf16 accumulation with one round-to-nearest-even per add.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace smr {

struct __align__(16) Vec16 {
  uint32_t x, y, z, w;
};

// Plain (weak) 16-byte load; valid on peer-mapped addresses.
__device__ __forceinline__ Vec16 ld_16(const void* p) {
  Vec16 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Streaming load that does not allocate in L1 (data read exactly once).
__device__ __forceinline__ Vec16 ld_16_stream(const void* p) {
  Vec16 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Read-only path for data that no one writes during the kernel (weights).
__device__ __forceinline__ Vec16 ld_16_nc(const void* p) {
  Vec16 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_16(void* p, const Vec16& v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
  uint32_t c;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(c) : "r"(a), "r"(b));
  return c;
}
__device__ __forceinline__ Vec16 add_bf16x8(const Vec16& a, const Vec16& b) {
  Vec16 c;
  c.x = add_bf16x2(a.x, b.x);
  c.y = add_bf16x2(a.y, b.y);
  c.z = add_bf16x2(a.z, b.z);
  c.w = add_bf16x2(a.w, b.w);
  return c;
}

__device__ __forceinline__ float bf16lo_to_f32(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
// two floats -> packed bf16x2 (lo in the low half), round to nearest even
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// four floats -> four e4m3 bytes (f0 in the lowest byte), round to nearest
// even, values beyond +-448 saturate.  The two-input cvt puts its FIRST source
// in the upper byte of the pair.
__device__ __forceinline__ uint32_t pack_e4m3x4(float f0, float f1, float f2, float f3) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(f1), "f"(f0));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(f3), "f"(f2));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ void st_8(void* p, uint32_t a, uint32_t b) {
  asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

}  // namespace smr
