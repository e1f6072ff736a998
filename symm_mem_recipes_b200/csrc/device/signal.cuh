// Cross-GPU signalling primitives: scoped loads / stores / atomics in inline
// PTX and bounded spin loops built on them.
//
// Upstream writes these qualifiers inline where it needs them and spins
// without a bound (symm_mem_recipes/triton_barrier.py:112-139,
// triton_all_gather_matmul.py:72-95).
//
// Every wait takes a deadline in nanoseconds of %globaltimer plus a hard
// iteration cap.  When either runs out the wait records a Status and returns
// false; the caller unwinds (frees TMEM, drains copies) and returns.
#pragma once
#include <stdint.h>
#include "status.h"

namespace smr {

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t cas_release_sys(uint32_t* p, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.global.release.sys.cas.b32 %0, [%1], %2, %3;"
               : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t cas_acquire_sys(uint32_t* p, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.global.acquire.sys.cas.b32 %0, [%1], %2, %3;"
               : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ void fence_acq_rel_gpu() {
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
}
// Orders generic-proxy accesses against async-proxy (TMA) accesses.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// First reporter wins; the record is read by the host after the launch.
__device__ __forceinline__ void report_status(Status* st, uint32_t code, uint32_t rank,
                                              uint32_t block, uint32_t peer, uint32_t where,
                                              uint32_t aux = 0) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->rank = rank;
    st->block = block;
    st->peer = peer;
    st->where = where;
    st->aux = aux;
    __threadfence();
  }
}

// A deadline that is armed lazily: the clock is read only every 64 spins.
struct Deadline {
  uint64_t timeout_ns;
  uint64_t end;
  uint32_t spins;
  __device__ __forceinline__ explicit Deadline(uint64_t t) : timeout_ns(t), end(0), spins(0) {}
  // true while the caller may keep spinning
  __device__ __forceinline__ bool alive() {
    ++spins;
    if ((spins & 63u) != 0u) return true;
    if (spins >= (1u << 30)) return false;  // hard cap, clock or no clock
    uint64_t now = globaltimer_ns();
    if (end == 0) {
      end = now + timeout_ns;
      return true;
    }
    return now < end;
  }
};

// Spin until *p >= target (acquire, system scope).  Returns false on timeout.
__device__ __forceinline__ bool wait_ge_acquire_sys(const uint32_t* p, uint32_t target,
                                                    uint64_t timeout_ns) {
  Deadline d(timeout_ns);
  while (ld_acquire_sys(p) < target) {
    if (!d.alive()) return false;
  }
  return true;
}
// The same for a counter that only grows and may wrap: waits until it has reached `target`
// (difference taken modulo 2^32; the counter is never more than 2^31 ahead or behind).
__device__ __forceinline__ bool wait_reached_acquire_sys(const uint32_t* p, uint32_t target,
                                                         uint64_t timeout_ns) {
  Deadline d(timeout_ns);
  while ((int32_t)(ld_acquire_sys(p) - target) < 0) {
    if (!d.alive()) return false;
  }
  return true;
}
__device__ __forceinline__ bool wait_ge_acquire_gpu(const uint32_t* p, uint32_t target,
                                                    uint64_t timeout_ns) {
  Deadline d(timeout_ns);
  while (ld_acquire_gpu(p) < target) {
    if (!d.alive()) return false;
  }
  return true;
}
__device__ __forceinline__ bool wait_eq_acquire_sys(const uint32_t* p, uint32_t target,
                                                    uint64_t timeout_ns) {
  Deadline d(timeout_ns);
  while (ld_acquire_sys(p) != target) {
    if (!d.alive()) return false;
  }
  return true;
}

}  // namespace smr
