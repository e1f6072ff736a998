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

// ---------------------------------------------------------------------------
// Epoch barrier: the low-latency barrier of the all-reduce kernels.
//
// blockwise_barrier above pays a remote atomic round trip (CAS to the peer's
// pad) before it can start waiting.  Here arrival is a plain store: thread
// t < WS writes this block's barrier count e into slot [16 + rank] of peer t
// (st.release.sys, one way over NVLink) and polls its OWN slot [16 + t] until
// it reads a count >= e.  The count lives in the pad (slot [0] of the block's
// group), is read when the kernel starts and written back when it ends, so no
// launch parameter changes between calls and a captured graph replays.  A peer
// can be at most one barrier ahead, hence the signed comparison.
// ---------------------------------------------------------------------------
struct EpochBarrier {
  uint32_t* const* pads;
  uint32_t* mine;      // this rank's group of kArFlagStride slots for this block id
  uint32_t slot_base;  // offset of that group inside any rank's pad
  uint32_t count;      // barriers passed so far by this block id
  int rank, world_size;

  __device__ __forceinline__ EpochBarrier(uint32_t* const* pads_, uint32_t block_id, int rank_, int ws)
      : pads(pads_), rank(rank_), world_size(ws) {
    slot_base = kArFlagBase + block_id * kArFlagStride;
    mine = pads[rank] + slot_base;
    count = ld_relaxed_gpu(mine);     // written by the previous kernel of this stream
  }

  // All threads of the CTA call it.  false on timeout (Status recorded).
  __device__ __forceinline__ bool sync(uint64_t timeout_ns, Status* st, uint32_t where) {
    ++count;
    __syncthreads();   // the CTA's earlier writes precede the release
    bool ok = true;
    const uint32_t tid = flat_tid();
    if (tid < (uint32_t)world_size) {
      st_release_sys(pads[tid] + slot_base + 16u + (uint32_t)rank, count);
      const uint32_t* wait = mine + 16u + tid;
      Deadline d(timeout_ns);
      while ((int32_t)(ld_acquire_sys(wait) - count) < 0) {
        if (!d.alive()) {
          report_status(st, kTimeoutBarrierWait, rank, slot_base, tid, where, count);
          ok = false;
          break;
        }
      }
    }
    return __syncthreads_and(ok) != 0;
  }

  // Once, by every thread, after the kernel's last sync.
  __device__ __forceinline__ void finish() {
    if (flat_tid() == 0) *mine = count;
  }
};

// ---------------------------------------------------------------------------
// NVLS barrier: arrival is ONE `multimem.red.add` on a counter in the multicast
// mapping of the signal pad, which the NVSwitch applies to the copy of that
// counter on every rank; each rank then polls its own copy until it reads
// (barriers so far) x world_size.  One instruction on the wire per rank and
// barrier instead of world_size stores.  Needs a multicast mapping that covers
// the pad (the allocator binds the whole block).  Slots of the block's group:
// [1] = arrivals (sum over ranks and barriers), [2] = this rank's barrier count;
// they do not overlap the epoch barrier's slots, and like them they only grow.
// ---------------------------------------------------------------------------
struct MulticastBarrier {
  uint32_t* mine;        // this rank's group of kArFlagStride slots for this block id
  uint32_t* mc_arrivals; // multicast address of slot [1] of that group
  uint32_t slot_base;
  uint32_t count;
  int rank, world_size;

  // `buffers[rank]` / `pads[rank]`: local payload and pad base; `multicast`: multicast payload base.
  __device__ __forceinline__ MulticastBarrier(uint32_t* const* pads, void* const* buffers, void* multicast,
                                              uint32_t block_id, int rank_, int ws)
      : rank(rank_), world_size(ws) {
    slot_base = kArFlagBase + block_id * kArFlagStride;
    mine = pads[rank] + slot_base;
    const size_t pad_offset = reinterpret_cast<const char*>(pads[rank]) - static_cast<const char*>(buffers[rank]);
    mc_arrivals = reinterpret_cast<uint32_t*>(static_cast<char*>(multicast) + pad_offset) + slot_base + 1u;
    count = ld_relaxed_gpu(mine + 2);
  }

  // All threads of the CTA call it.  false on timeout (Status recorded).
  __device__ __forceinline__ bool sync(uint64_t timeout_ns, Status* st, uint32_t where) {
    ++count;
    __syncthreads();   // the CTA's earlier writes precede the release
    bool ok = true;
    if (flat_tid() == 0) {
      asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_arrivals), "r"(1u) : "memory");
      const uint32_t target = count * (uint32_t)world_size;
      Deadline d(timeout_ns);
      while ((int32_t)(ld_acquire_sys(mine + 1) - target) < 0) {
        if (!d.alive()) {
          report_status(st, kTimeoutBarrierWait, rank, slot_base, 0, where, count);
          ok = false;
          break;
        }
      }
    }
    return __syncthreads_and(ok) != 0;
  }

  // Once, by every thread, after the kernel's last sync.
  __device__ __forceinline__ void finish() {
    if (flat_tid() == 0) mine[2] = count;
  }
};

}  // namespace smr
