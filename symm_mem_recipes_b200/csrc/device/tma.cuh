// TMA: tiled tensor loads (cp.async.bulk.tensor) and untiled bulk copies
// (cp.async.bulk) in inline PTX.  No load here carries a cluster-multicast
// qualifier: a remote tile is fetched by the CTA that needs it.
//
// Upstream reaches TMA through Triton's descriptor loads and stores
// (symm_mem_recipes/triton_all_gather_matmul.py:166-193, descriptors built at :255-286).
//
// Alignment rule for every tiled copy: the innermost coordinate times the
// element size must be a multiple of 16 bytes (8 elements for bf16).
#pragma once
#include <cuda.h>
#include <stdint.h>

#include "mbarrier.cuh"

namespace smr {

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tile global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(x), "r"(y)
      : "memory");
}

// 2-D tile shared -> global, tracked by bulk async-groups.  Parts of the box outside the tensor
// are not written.  The shared-memory writes that filled the tile must be followed by
// fence_proxy_async_smem() before the issuing thread is signalled.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
// Makes this thread's earlier shared-memory writes visible to the async proxy (TMA stores).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void st_shared_16(uint32_t smem_addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(smem_addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// Untiled bulk copy global -> shared (both 16-byte aligned, size % 16 == 0).
// The source may be a peer GPU's memory mapped into this process.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// Untiled bulk copy shared -> global, tracked by bulk async-groups.
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// At most N most recent groups may still be READING their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// At most N most recent groups may still be incomplete (writes not yet done).
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

}  // namespace smr
