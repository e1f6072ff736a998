// blockwise_barrier: a cross-GPU barrier among the CTAs that carry the same
// `block_id` on every rank, over the zero-filled signal pad.
//
// Behaviour follows symm_mem_recipes/triton_barrier.py:50-153: thread t < WS
// (1) flips slot pad[t][block_id*WS + rank] of peer t from 0 to 1, spinning
// while the peer has not consumed the previous signal, then (2) flips slot
// pad[rank][block_id*WS + t] of its own pad from 1 back to 0, spinning until
// peer t has arrived.  Every slot is 0 again afterwards, so the barrier needs
// no host-side epoch and can be replayed from a CUDA graph.
//
// Differences from upstream, on purpose:
//  * the consuming CAS itself is `.acquire.sys` and the sending CAS is
//    `.release.sys`, so signal -> wait is a proper synchronises-with edge; the
//    CTA-wide bar.sync then extends it to every thread of the CTA.  Upstream
//    instead re-reads its own pad with ld.acquire after the bar.sync
//    (triton_barrier.py:145-153).
//  * both spins are bounded; on expiry the barrier records a Status and every
//    thread of the CTA gets `false`.
//
// Usage patterns (what the barrier orders):
//  * entry:  writes made by peers BEFORE their kernel are visible to every
//    thread of this CTA AFTER the barrier.
//  * middle: writes made by any thread of the peer CTAs before the barrier are
//    visible after it, provided the writer CTA calls __syncthreads() first
//    (the barrier does; see `sync_before`).
//  * exit:   with kRelaxed the barrier only proves arrival (peers finished
//    reading our memory) and carries no data.
#pragma once
#include "pad_layout.h"
#include "signal.cuh"

namespace smr {

__device__ __forceinline__ uint32_t flat_tid() {
  return threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
}
__device__ __forceinline__ uint32_t flat_block_id() {
  return blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
}

// One thread's half of the protocol against peer `peer`.
__device__ __forceinline__ bool barrier_signal_wait(uint32_t* const* pads, uint32_t slot_base,
                                                    int rank, int world_size, int peer,
                                                    uint64_t timeout_ns, Status* st,
                                                    uint32_t block_id, uint32_t where) {
  uint32_t* send = pads[peer] + slot_base + rank;
  uint32_t* wait = pads[rank] + slot_base + peer;
  Deadline d(timeout_ns);
  while (cas_release_sys(send, 0u, 1u) != 0u) {
    if (!d.alive()) {
      report_status(st, kTimeoutBarrierSend, rank, block_id, peer, where);
      return false;
    }
  }
  Deadline d2(timeout_ns);
  while (cas_acquire_sys(wait, 1u, 0u) != 1u) {
    if (!d2.alive()) {
      report_status(st, kTimeoutBarrierWait, rank, block_id, peer, where);
      return false;
    }
  }
  return true;
}

// Must be called by every thread of the CTA.  `pads` is the device table of
// the WS signal-pad base pointers (pads[rank] is the local one).
__device__ __forceinline__ bool blockwise_barrier(uint32_t* const* pads, uint32_t block_id,
                                                  int rank, int world_size,
                                                  uint64_t timeout_ns, Status* st,
                                                  uint32_t where) {
  __syncthreads();  // sync_before: the CTA's earlier writes precede the release
  bool ok = true;
  uint32_t tid = flat_tid();
  if (tid < (uint32_t)world_size) {
    ok = barrier_signal_wait(pads, block_id * (uint32_t)world_size, rank, world_size, (int)tid,
                             timeout_ns, st, block_id, where);
  }
  return __syncthreads_and(ok) != 0;
}

}  // namespace smr
