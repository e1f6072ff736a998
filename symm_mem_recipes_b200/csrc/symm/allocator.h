// Symmetric allocation on a CUDA device: one physical VMM block holding the
// payload followed by a zero-filled signal pad, exportable to the other ranks
// of the host as a POSIX file descriptor, with the peers' blocks mapped into
// this process and (optionally) all of them bound to one NVLink multicast
// object for NVLS.
//
// Plays the role that torch's C++ `_SymmetricMemory` plays for the upstream
// recipes (`empty_strided_p2p` / `rendezvous`, used at
// symm_mem_recipes/triton_all_gather_matmul.py:226, 369-375 and
// symm_mem_recipes/triton_one_shot_all_reduce.py:111, 145-151).
#pragma once
#include <cuda.h>
#include <stdint.h>

#include <memory>
#include <string>
#include <vector>

#include "../device/pad_layout.h"
#include "ipc.h"

namespace smr {

class CudaSymmAllocation {
 public:
  // Allocates and maps the local block on `device`, zero-fills it.
  CudaSymmAllocation(int device, size_t payload_bytes);
  ~CudaSymmAllocation();
  CudaSymmAllocation(const CudaSymmAllocation&) = delete;
  CudaSymmAllocation& operator=(const CudaSymmAllocation&) = delete;

  int device() const { return device_; }
  size_t payload_bytes() const { return payload_bytes_; }
  size_t pad_offset() const { return pad_offset_; }
  size_t block_bytes() const { return block_bytes_; }
  void* local_ptr() const { return reinterpret_cast<void*>(va_); }

  // ---- rendezvous, phase by phase (the Python layer puts a Store barrier
  //      between phases and supplies the socket names) ----
  void begin_rendezvous(int rank, int world_size);
  // Sends this block's FD to every peer and maps the WS-1 blocks received.
  void exchange_and_map(const FdChannel& chan, const std::vector<std::string>& names,
                        int timeout_ms);
  // Multicast: rank 0 creates the object and sends it round; every rank adds
  // its device.  Returns false when the device or driver cannot do multicast.
  bool multicast_create_and_add(const FdChannel& chan, const std::vector<std::string>& names,
                                int timeout_ms);
  // After all ranks have added their device: bind local memory and map.
  void multicast_bind_and_map();
  void multicast_teardown();
  // Builds the device pointer tables.  Call last.
  void finish_rendezvous();
  bool rendezvoused() const { return rendezvoused_; }

  int rank() const { return rank_; }
  int world_size() const { return world_size_; }
  void* peer_ptr(int r) const { return reinterpret_cast<void*>(peer_va_.at(r)); }
  uint32_t* peer_pad(int r) const {
    return reinterpret_cast<uint32_t*>(peer_va_.at(r) + pad_offset_);
  }
  void* multicast_ptr() const { return reinterpret_cast<void*>(mc_va_); }
  void* const* buffers_dev() const { return buffers_dev_; }
  uint32_t* const* pads_dev() const { return pads_dev_; }

  // Unmaps everything (multicast first).  Idempotent; the device must be idle.
  void release();

  static bool multicast_supported(int device);

 private:
  int device_;
  size_t payload_bytes_, pad_offset_, block_bytes_;
  size_t granularity_ = 0;   // of the physical allocation; every mapping of it is aligned to this
  CUmemGenericAllocationHandle handle_ = 0;
  CUdeviceptr va_ = 0;
  int rank_ = -1, world_size_ = 0;
  std::vector<CUmemGenericAllocationHandle> peer_handles_;
  std::vector<CUdeviceptr> peer_va_;
  CUmemGenericAllocationHandle mc_handle_ = 0;
  CUdeviceptr mc_va_ = 0;
  bool mc_device_added_ = false, mc_bound_ = false;
  void** buffers_dev_ = nullptr;
  uint32_t** pads_dev_ = nullptr;
  bool rendezvoused_ = false, released_ = false;
};

}  // namespace smr
