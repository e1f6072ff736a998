#include "allocator.h"

#include <cuda_runtime_api.h>
#include <unistd.h>

#include <stdexcept>

#include "driver_api.h"

namespace smr {

namespace {

constexpr int32_t kTagBlock = 1;
constexpr int32_t kTagMulticast = 2;

void rt_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

CUmemAllocationProp block_prop(int device) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

CUmulticastObjectProp mc_prop(int world_size, size_t bytes) {
  CUmulticastObjectProp p{};
  p.numDevices = (unsigned)world_size;
  p.size = bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  p.flags = 0;
  return p;
}

void set_rw_access(CUdeviceptr va, size_t bytes, int device) {
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  SMR_CU_CHECK(DriverApi::get().cuMemSetAccess(va, bytes, &acc, 1));
}

}  // namespace

bool CudaSymmAllocation::multicast_supported(int device) {
  int v = 0;
  const DriverApi& d = DriverApi::get();
  CUdevice dev;
  if (d.cuDeviceGet(&dev, device) != CUDA_SUCCESS) return false;
  if (d.cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS)
    return false;
  return v != 0;
}

CudaSymmAllocation::CudaSymmAllocation(int device, size_t payload_bytes)
    : device_(device), payload_bytes_(payload_bytes) {
  const DriverApi& d = DriverApi::get();
  rt_check(cudaSetDevice(device), "cudaSetDevice");
  rt_check(cudaFree(nullptr), "context creation");
  CUmemAllocationProp prop = block_prop(device);
  size_t gran = 0;
  SMR_CU_CHECK(d.cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  if (multicast_supported(device)) {
    // A block can only be bound to a multicast object in units of the
    // multicast granularity; size for the largest world we support.
    CUmulticastObjectProp mp = mc_prop(2, gran);
    size_t mgran = 0;
    if (d.cuMulticastGetGranularity(&mgran, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS &&
        mgran > gran)
      gran = round_up(mgran, gran);
  }
  granularity_ = gran;
  pad_offset_ = round_up(payload_bytes_ == 0 ? 16 : payload_bytes_, 256);
  block_bytes_ = round_up(pad_offset_ + kSignalPadBytes, gran);
  try {
    SMR_CU_CHECK(d.cuMemCreate(&handle_, block_bytes_, &prop, 0));
    SMR_CU_CHECK(d.cuMemAddressReserve(&va_, block_bytes_, gran, 0, 0));
    SMR_CU_CHECK(d.cuMemMap(va_, block_bytes_, 0, handle_, 0));
    set_rw_access(va_, block_bytes_, device_);
    rt_check(cudaMemset(reinterpret_cast<void*>(va_), 0, block_bytes_), "cudaMemset(block)");
    rt_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  } catch (...) {
    // a constructor that throws runs no destructor: give back what was obtained so far
    release();
    throw;
  }
}

CudaSymmAllocation::~CudaSymmAllocation() {
  try {
    release();
  } catch (...) {
  }
}

void CudaSymmAllocation::begin_rendezvous(int rank, int world_size) {
  if (rendezvoused_) throw std::runtime_error("allocation is already rendezvoused");
  if (world_size < 1 || world_size > kMaxWorldSize || rank < 0 || rank >= world_size)
    throw std::runtime_error("bad rank / world size");
  rank_ = rank;
  world_size_ = world_size;
  peer_handles_.assign(world_size, 0);
  peer_va_.assign(world_size, 0);
  peer_va_[rank] = va_;
}

void CudaSymmAllocation::exchange_and_map(const FdChannel& chan,
                                          const std::vector<std::string>& names, int timeout_ms) {
  const DriverApi& d = DriverApi::get();
  rt_check(cudaSetDevice(device_), "cudaSetDevice");
  if ((int)names.size() != world_size_) throw std::runtime_error("names.size() != world_size");
  if (world_size_ == 1) return;
  int fd = -1;
  SMR_CU_CHECK(d.cuMemExportToShareableHandle(&fd, handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  try {
    for (int step = 1; step < world_size_; ++step) {
      int peer = (rank_ + step) % world_size_;
      chan.send_fd(names[peer], fd, rank_, kTagBlock, timeout_ms);
    }
  } catch (...) {
    close(fd);
    throw;
  }
  close(fd);
  for (int i = 1; i < world_size_; ++i) {
    FdMessage m = chan.recv_fd(timeout_ms);
    if (m.tag != kTagBlock || m.src_rank < 0 || m.src_rank >= world_size_ || m.src_rank == rank_ ||
        peer_handles_[m.src_rank] != 0) {
      close(m.fd);
      throw std::runtime_error("rendezvous: unexpected message from rank " + std::to_string(m.src_rank));
    }
    CUmemGenericAllocationHandle h = 0;
    CUresult r = d.cuMemImportFromShareableHandle(&h, reinterpret_cast<void*>((uintptr_t)m.fd),
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(m.fd);
    SMR_CU_CHECK(r);
    peer_handles_[m.src_rank] = h;
    CUdeviceptr va = 0;
    // aligned to the allocation granularity so that the mapping can use large pages
    SMR_CU_CHECK(d.cuMemAddressReserve(&va, block_bytes_, granularity_, 0, 0));
    peer_va_[m.src_rank] = va;          // recorded at once: release() returns it if a later step throws
    SMR_CU_CHECK(d.cuMemMap(va, block_bytes_, 0, h, 0));
    set_rw_access(va, block_bytes_, device_);
  }
}

bool CudaSymmAllocation::multicast_create_and_add(const FdChannel& chan,
                                                  const std::vector<std::string>& names,
                                                  int timeout_ms) {
  const DriverApi& d = DriverApi::get();
  rt_check(cudaSetDevice(device_), "cudaSetDevice");
  if (world_size_ < 2 || !multicast_supported(device_)) return false;
  CUmulticastObjectProp prop = mc_prop(world_size_, block_bytes_);
  size_t mgran = 0;
  if (d.cuMulticastGetGranularity(&mgran, &prop, CU_MULTICAST_GRANULARITY_MINIMUM) != CUDA_SUCCESS ||
      mgran == 0 || block_bytes_ % mgran != 0)
    return false;  // same answer on every rank: sizes and devices are identical
  if (rank_ == 0) {
    SMR_CU_CHECK(d.cuMulticastCreate(&mc_handle_, &prop));
    int fd = -1;
    SMR_CU_CHECK(d.cuMemExportToShareableHandle(&fd, mc_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    try {
      for (int peer = 1; peer < world_size_; ++peer)
        chan.send_fd(names[peer], fd, rank_, kTagMulticast, timeout_ms);
    } catch (...) {
      close(fd);
      throw;
    }
    close(fd);
  } else {
    FdMessage m = chan.recv_fd(timeout_ms);
    if (m.tag != kTagMulticast || m.src_rank != 0) {
      close(m.fd);
      throw std::runtime_error("rendezvous: expected the multicast handle from rank 0");
    }
    CUresult r = d.cuMemImportFromShareableHandle(&mc_handle_, reinterpret_cast<void*>((uintptr_t)m.fd),
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(m.fd);
    SMR_CU_CHECK(r);
  }
  CUdevice dev;
  SMR_CU_CHECK(d.cuDeviceGet(&dev, device_));
  SMR_CU_CHECK(d.cuMulticastAddDevice(mc_handle_, dev));
  mc_device_added_ = true;
  return true;
}

void CudaSymmAllocation::multicast_bind_and_map() {
  const DriverApi& d = DriverApi::get();
  rt_check(cudaSetDevice(device_), "cudaSetDevice");
  if (mc_handle_ == 0) throw std::runtime_error("no multicast object");
  SMR_CU_CHECK(d.cuMulticastBindMem(mc_handle_, 0, handle_, 0, block_bytes_, 0));
  mc_bound_ = true;
  SMR_CU_CHECK(d.cuMemAddressReserve(&mc_va_, block_bytes_, granularity_, 0, 0));
  SMR_CU_CHECK(d.cuMemMap(mc_va_, block_bytes_, 0, mc_handle_, 0));
  set_rw_access(mc_va_, block_bytes_, device_);
}

void CudaSymmAllocation::multicast_teardown() {
  if (mc_handle_ == 0) return;
  const DriverApi& d = DriverApi::get();
  cudaSetDevice(device_);
  if (mc_va_ != 0) {
    d.cuMemUnmap(mc_va_, block_bytes_);
    d.cuMemAddressFree(mc_va_, block_bytes_);
    mc_va_ = 0;
  }
  if (mc_bound_) {
    CUdevice dev;
    if (d.cuDeviceGet(&dev, device_) == CUDA_SUCCESS)
      d.cuMulticastUnbind(mc_handle_, dev, 0, block_bytes_);
    mc_bound_ = false;
  }
  d.cuMemRelease(mc_handle_);
  mc_handle_ = 0;
}

void CudaSymmAllocation::finish_rendezvous() {
  rt_check(cudaSetDevice(device_), "cudaSetDevice");
  std::vector<void*> bufs(world_size_);
  std::vector<uint32_t*> pads(world_size_);
  for (int r = 0; r < world_size_; ++r) {
    if (peer_va_[r] == 0) throw std::runtime_error("rendezvous: rank " + std::to_string(r) + " was never mapped");
    bufs[r] = reinterpret_cast<void*>(peer_va_[r]);
    pads[r] = reinterpret_cast<uint32_t*>(peer_va_[r] + pad_offset_);
  }
  rt_check(cudaMalloc(reinterpret_cast<void**>(&buffers_dev_), sizeof(void*) * kMaxWorldSize), "cudaMalloc");
  rt_check(cudaMalloc(reinterpret_cast<void**>(&pads_dev_), sizeof(void*) * kMaxWorldSize), "cudaMalloc");
  rt_check(cudaMemcpy(buffers_dev_, bufs.data(), sizeof(void*) * world_size_, cudaMemcpyHostToDevice), "cudaMemcpy");
  rt_check(cudaMemcpy(pads_dev_, pads.data(), sizeof(void*) * world_size_, cudaMemcpyHostToDevice), "cudaMemcpy");
  rendezvoused_ = true;
}

void CudaSymmAllocation::release() {
  if (released_) return;
  released_ = true;
  const DriverApi& d = DriverApi::get();
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  multicast_teardown();
  for (int r = 0; r < (int)peer_va_.size(); ++r) {
    if (r == rank_ || peer_va_[r] == 0) continue;
    d.cuMemUnmap(peer_va_[r], block_bytes_);
    d.cuMemAddressFree(peer_va_[r], block_bytes_);
    if (peer_handles_[r] != 0) d.cuMemRelease(peer_handles_[r]);
    peer_va_[r] = 0;
  }
  if (buffers_dev_ != nullptr) cudaFree(buffers_dev_);
  if (pads_dev_ != nullptr) cudaFree(pads_dev_);
  buffers_dev_ = nullptr;
  pads_dev_ = nullptr;
  if (va_ != 0) {
    d.cuMemUnmap(va_, block_bytes_);
    d.cuMemAddressFree(va_, block_bytes_);
    va_ = 0;
  }
  if (handle_ != 0) {
    d.cuMemRelease(handle_);
    handle_ = 0;
  }
}

}  // namespace smr
