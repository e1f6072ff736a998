// Symmetric memory on the CPU: POSIX shared memory blocks (payload + signal
// pad) mapped by every rank of the host, and the same barrier / all-reduce
// protocols executed with host atomics.  It exists so that the allocator API,
// the rendezvous, the dispatcher and the barrier state machine can be tested
// with `gloo` ranks on a machine without a GPU.  No upstream counterpart: the
// upstream recipes are only exercised by GPU drivers
// (symm_mem_recipes/triton_barrier.py:173-200, triton_one_shot_all_reduce.py:128-164).
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "../device/pad_layout.h"
#include "../device/status.h"

namespace smr {

class HostSymmAllocation {
 public:
  // Creates /dev/shm/<name> of payload + pad bytes, zero-filled.
  HostSymmAllocation(const std::string& shm_name, size_t payload_bytes);
  ~HostSymmAllocation();
  HostSymmAllocation(const HostSymmAllocation&) = delete;
  HostSymmAllocation& operator=(const HostSymmAllocation&) = delete;

  const std::string& shm_name() const { return name_; }
  size_t payload_bytes() const { return payload_bytes_; }
  size_t pad_offset() const { return pad_offset_; }
  size_t block_bytes() const { return block_bytes_; }
  void* local_ptr() const { return base_; }

  // Maps the peers' blocks by name (names[rank] must be this block's name).
  void rendezvous(int rank, const std::vector<std::string>& names);
  bool rendezvoused() const { return rendezvoused_; }
  int rank() const { return rank_; }
  int world_size() const { return world_size_; }
  void* peer_ptr(int r) const { return peers_.at(r); }
  uint32_t* peer_pad(int r) const {
    return reinterpret_cast<uint32_t*>(static_cast<char*>(peers_.at(r)) + pad_offset_);
  }
  void release();

  // Same slot protocol as the device barrier; `slot_base` selects block or
  // channel slots.  Returns a StatusCode (kOk on success) and fills `peer`.
  uint32_t barrier(uint32_t slot_base, uint64_t timeout_ns, int* failed_peer);
  // The two halves of that protocol on their own, towards ONE peer: `put_signal` flips slot
  // [slot_base + this rank] of `dst`'s pad from 0 to 1 (release; waits while an earlier signal is
  // unconsumed), `wait_signal` flips slot [slot_base + src] of the own pad from 1 to 0 (acquire).
  uint32_t put_signal(int dst, uint32_t slot_base, uint64_t timeout_ns);
  uint32_t wait_signal(int src, uint32_t slot_base, uint64_t timeout_ns);

 private:
  std::string name_;
  size_t payload_bytes_, pad_offset_, block_bytes_;
  void* base_ = nullptr;
  int rank_ = -1, world_size_ = 0;
  std::vector<void*> peers_;
  bool rendezvoused_ = false, released_ = false;
};

// Barrier protocol on bare pads (used by the multi-threaded protocol tests).
uint32_t host_barrier_signal_wait(uint32_t* const* pads, uint32_t slot_base, int rank,
                                  int world_size, uint64_t timeout_ns, int* failed_peer);

// Epoch barrier of the all-reduce kernels (store the barrier count into the peers' slots, poll
// the own ones), same slot layout as the device version: group of kArFlagStride slots per
// block id at kArFlagBase, [0] = own count, [16 + s] = last count announced by rank s.
// `count` is the caller's running barrier count for this block id.
uint32_t host_epoch_barrier(uint32_t* const* pads, uint32_t block_id, int rank, int world_size,
                            uint32_t* count, uint64_t timeout_ns, int* failed_peer);

// Low-latency all-reduce protocol on host memory (see ll_all_reduce_kernel): tagged 8-byte
// words pushed into every rank's inbox, two parities, call number in the workspace header.
// `workspaces[r]` is rank r's workspace base as mapped here.  Returns a StatusCode.
uint32_t host_ll_all_reduce(void* const* workspaces, int rank, int world_size, const uint16_t* in,
                            uint16_t* out, size_t numel, size_t capacity_numel, uint64_t timeout_ns,
                            int* failed_peer);

}  // namespace smr
