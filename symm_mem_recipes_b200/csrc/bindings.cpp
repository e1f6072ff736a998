// Python bindings (pybind11 through torch/extension.h).  This is the only
// translation unit that sees framework headers; everything it calls takes raw
// pointers and a stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>
#include <torch/extension.h>

#include <map>
#include <memory>
#include <atomic>
#include <mutex>
#include <thread>

#include "kernels/launch.h"
#include "oracle/cpu_reference.h"
#include "symm/allocator.h"
#include "symm/driver_api.h"
#include "symm/host_backend.h"
#include "symm/ipc.h"

namespace py = pybind11;
using namespace smr;

namespace {

void rt_check(int e, const char* what) {
  TORCH_CHECK(e == 0, what, ": ", cudaGetErrorString((cudaError_t)e));
}

// ---- per-device status record ----------------------------------------------
std::mutex g_status_mu;
std::map<int, Status*> g_status;

Status* status_for(int device) {
  std::lock_guard<std::mutex> lock(g_status_mu);
  auto it = g_status.find(device);
  if (it != g_status.end()) return it->second;
  c10::cuda::CUDAGuard guard(device);
  Status* s = nullptr;
  rt_check(cudaMalloc(reinterpret_cast<void**>(&s), sizeof(Status)), "cudaMalloc(status)");
  rt_check(cudaMemset(s, 0, sizeof(Status)), "cudaMemset(status)");
  g_status[device] = s;
  return s;
}

// Synchronises the device, returns (code, rank, block, peer, where, aux) and
// clears the record.
py::tuple read_status(int device) {
  Status* s = status_for(device);
  c10::cuda::CUDAGuard guard(device);
  Status h{};
  rt_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  rt_check(cudaMemcpy(&h, s, sizeof(Status), cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
  if (h.code != 0) rt_check(cudaMemset(s, 0, sizeof(Status)), "cudaMemset(status)");
  return py::make_tuple(h.code, h.rank, h.block, h.peer, h.where, h.aux);
}

cudaStream_t current_stream(int device) { return c10::cuda::getCurrentCUDAStream(device).stream(); }

PeerView view_of(const CudaSymmAllocation& a) {
  TORCH_CHECK(a.rendezvoused(), "symmetric allocation has not been rendezvoused");
  PeerView pv;
  pv.buffers = a.buffers_dev();
  pv.pads = a.pads_dev();
  pv.multicast = a.multicast_ptr();
  pv.rank = a.rank();
  pv.world_size = a.world_size();
  return pv;
}

PeerPtrs ptrs_of(const CudaSymmAllocation& a) {
  TORCH_CHECK(a.rendezvoused(), "symmetric allocation has not been rendezvoused");
  TORCH_CHECK(a.world_size() <= 8, "this kernel takes its peers by value: at most 8 ranks");
  PeerPtrs p{};
  for (int r = 0; r < a.world_size(); ++r) {
    p.buffers[r] = a.peer_ptr(r);
    p.pads[r] = a.peer_pad(r);
  }
  return p;
}

torch::Tensor cuda_view(const std::shared_ptr<CudaSymmAllocation>& a, int rank,
                        std::vector<int64_t> sizes, torch::ScalarType dtype, int64_t offset_bytes,
                        bool multicast) {
  int64_t numel = 1;
  for (auto s : sizes) numel *= s;
  int64_t bytes = numel * (int64_t)c10::elementSize(dtype);
  TORCH_CHECK(offset_bytes >= 0 && (size_t)(offset_bytes + bytes) <= a->payload_bytes(),
              "view exceeds the symmetric allocation");
  char* base;
  if (multicast) {
    TORCH_CHECK(a->multicast_ptr() != nullptr, "allocation has no multicast mapping");
    base = static_cast<char*>(a->multicast_ptr());
  } else if (rank < 0 || !a->rendezvoused()) {
    base = static_cast<char*>(a->local_ptr());
  } else {
    base = static_cast<char*>(a->peer_ptr(rank));
  }
  auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, a->device());
  // The deleter keeps the allocation alive for as long as a view exists.  A
  // peer or multicast mapping reports the peer's device to the pointer query;
  // target_device pins the view to the device that maps it.
  return at::for_blob(base + offset_bytes, sizes)
      .deleter([a](void*) {})
      .options(opts)
      .target_device(c10::Device(c10::kCUDA, a->device()))
      .make_tensor();
}

torch::Tensor cuda_pad_view(const std::shared_ptr<CudaSymmAllocation>& a, int rank) {
  char* base = (rank < 0 || !a->rendezvoused()) ? static_cast<char*>(a->local_ptr())
                                                : static_cast<char*>(a->peer_ptr(rank));
  auto opts = torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, a->device());
  return at::for_blob(base + a->pad_offset(), {(int64_t)kSignalPadSlots})
      .deleter([a](void*) {})
      .options(opts)
      .target_device(c10::Device(c10::kCUDA, a->device()))
      .make_tensor();
}

torch::Tensor host_view(const std::shared_ptr<HostSymmAllocation>& a, int rank,
                        std::vector<int64_t> sizes, torch::ScalarType dtype, int64_t offset_bytes) {
  int64_t numel = 1;
  for (auto s : sizes) numel *= s;
  int64_t bytes = numel * (int64_t)c10::elementSize(dtype);
  TORCH_CHECK(offset_bytes >= 0 && (size_t)(offset_bytes + bytes) <= a->payload_bytes(),
              "view exceeds the symmetric allocation");
  char* base = (rank < 0 || !a->rendezvoused()) ? static_cast<char*>(a->local_ptr())
                                                : static_cast<char*>(a->peer_ptr(rank));
  auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCPU);
  return torch::from_blob(base + offset_bytes, sizes, [a](void*) {}, opts);
}

torch::Tensor host_pad_view(const std::shared_ptr<HostSymmAllocation>& a, int rank) {
  char* base = (rank < 0 || !a->rendezvoused()) ? static_cast<char*>(a->local_ptr())
                                                : static_cast<char*>(a->peer_ptr(rank));
  auto opts = torch::TensorOptions().dtype(torch::kInt32).device(torch::kCPU);
  return torch::from_blob(base + a->pad_offset(), {(int64_t)kSignalPadSlots}, [a](void*) {}, opts);
}

const uint16_t* bf16_ptr(const torch::Tensor& t) {
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16 && t.is_contiguous() && t.device().is_cpu(),
              "expected a contiguous CPU bf16 tensor");
  return reinterpret_cast<const uint16_t*>(t.data_ptr());
}

// Host all-reduce over shared memory: barrier, then the oracle's arithmetic.
// algo: 0 one-shot (ordered bf16), 1 two-shot (ordered bf16, in place),
//       2 "multimem" stand-in (fp32 accumulate, in place).
py::tuple host_all_reduce(const std::shared_ptr<HostSymmAllocation>& a, int64_t offset_bytes,
                          torch::Tensor out, int64_t numel, int algo, uint64_t timeout_ns) {
  TORCH_CHECK(a->rendezvoused(), "symmetric allocation has not been rendezvoused");
  const int ws = a->world_size(), rank = a->rank();
  int peer = -1;
  uint32_t code;
  {
    py::gil_scoped_release nogil;
    code = a->barrier(0, timeout_ns, &peer);
  }
  if (code != kOk) return py::make_tuple(code, rank, 0, peer, (int)kWhereOneShotEntry, 0);
  std::vector<const uint16_t*> srcs(ws);
  for (int r = 0; r < ws; ++r)
    srcs[r] = reinterpret_cast<const uint16_t*>(static_cast<char*>(a->peer_ptr(r)) + offset_bytes);
  if (algo == 0) {
    TORCH_CHECK(out.numel() == numel, "output size mismatch");
    ordered_sum_bf16(srcs.data(), ws, reinterpret_cast<uint16_t*>(out.data_ptr()), (size_t)numel);
    return py::make_tuple(0, rank, 0, 0, 0, 0);
  }
  // in-place algorithms: reduce own slice, publish to every peer, exit barrier
  size_t n_vec = (size_t)numel / 8, q = n_vec / ws, rem = n_vec % ws;
  size_t begin = (size_t)rank * q + std::min((size_t)rank, rem);
  size_t end = begin + q + ((size_t)rank < rem ? 1 : 0);
  std::vector<uint16_t> tmp((end - begin) * 8);
  std::vector<const uint16_t*> sl(ws);
  for (int r = 0; r < ws; ++r) sl[r] = srcs[r] + begin * 8;
  if (algo == 1) ordered_sum_bf16(sl.data(), ws, tmp.data(), tmp.size());
  else fp32_sum_bf16(sl.data(), ws, tmp.data(), tmp.size());
  for (int r = 0; r < ws; ++r)
    memcpy(const_cast<uint16_t*>(srcs[r]) + begin * 8, tmp.data(), tmp.size() * 2);
  {
    py::gil_scoped_release nogil;
    code = a->barrier(0, timeout_ns, &peer);
  }
  return py::make_tuple(code, rank, 0, peer, (int)kWhereTwoShotExit, 0);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "symm_mem_recipes_b200 native module (sm_100a kernels + symmetric memory runtime)";
  m.attr("SIGNAL_PAD_BYTES") = (int)kSignalPadBytes;
  m.attr("BLOCK_SLOTS") = (int)kBlockSlots;
  m.attr("CHANNEL_SLOTS") = (int)kChannelSlots;
  m.attr("FLAG_SLOTS_BASE") = (int)kFlagSlotsBase;
  m.attr("MAX_WORLD_SIZE") = (int)kMaxWorldSize;

  py::class_<FdChannel, std::shared_ptr<FdChannel>>(m, "FdChannel")
      .def(py::init<const std::string&>())
      .def_property_readonly("name", &FdChannel::name)
      .def("send_fd", &FdChannel::send_fd, py::call_guard<py::gil_scoped_release>())
      .def("recv_fd",
           [](const FdChannel& c, int timeout_ms) {
             FdMessage msg;
             {
               py::gil_scoped_release nogil;
               msg = c.recv_fd(timeout_ms);
             }
             return py::make_tuple(msg.fd, msg.src_rank, msg.tag);
           });

  py::class_<CudaSymmAllocation, std::shared_ptr<CudaSymmAllocation>>(m, "CudaSymmAllocation")
      .def(py::init<int, size_t>())
      .def_property_readonly("device", &CudaSymmAllocation::device)
      .def_property_readonly("payload_bytes", &CudaSymmAllocation::payload_bytes)
      .def_property_readonly("block_bytes", &CudaSymmAllocation::block_bytes)
      .def_property_readonly("pad_offset", &CudaSymmAllocation::pad_offset)
      .def_property_readonly("rank", &CudaSymmAllocation::rank)
      .def_property_readonly("world_size", &CudaSymmAllocation::world_size)
      .def_property_readonly("rendezvoused", &CudaSymmAllocation::rendezvoused)
      .def_property_readonly("local_ptr", [](const CudaSymmAllocation& a) { return (uintptr_t)a.local_ptr(); })
      .def_property_readonly("multicast_ptr", [](const CudaSymmAllocation& a) { return (uintptr_t)a.multicast_ptr(); })
      .def_property_readonly("buffer_ptrs_dev", [](const CudaSymmAllocation& a) { return (uintptr_t)a.buffers_dev(); })
      .def_property_readonly("signal_pad_ptrs_dev", [](const CudaSymmAllocation& a) { return (uintptr_t)a.pads_dev(); })
      .def("peer_ptr", [](const CudaSymmAllocation& a, int r) { return (uintptr_t)a.peer_ptr(r); })
      .def("begin_rendezvous", &CudaSymmAllocation::begin_rendezvous)
      .def("exchange_and_map", &CudaSymmAllocation::exchange_and_map, py::call_guard<py::gil_scoped_release>())
      .def("multicast_create_and_add", &CudaSymmAllocation::multicast_create_and_add,
           py::call_guard<py::gil_scoped_release>())
      .def("multicast_bind_and_map", &CudaSymmAllocation::multicast_bind_and_map)
      .def("multicast_teardown", &CudaSymmAllocation::multicast_teardown)
      .def("finish_rendezvous", &CudaSymmAllocation::finish_rendezvous)
      .def("release", &CudaSymmAllocation::release)
      .def_static("multicast_supported", &CudaSymmAllocation::multicast_supported);
  // flags[offset] = value, ordered after the work already queued on the current stream and preceded by a
  // system-scope fence (cuStreamWriteValue32: what upstream's host-driven all-gather publishes progress
  // with, symm_mem_recipes/triton_all_gather_matmul.py:51-55).  False when the driver lacks the call.
  m.def("stream_write_value32", [](torch::Tensor flags, int64_t offset, uint32_t value) {
    TORCH_CHECK(flags.is_cuda() && flags.is_contiguous() && flags.element_size() == 4 &&
                offset >= 0 && offset < flags.numel(), "need a contiguous 32-bit CUDA tensor and an offset inside it");
    const DriverApi& d = DriverApi::get();
    if (d.cuStreamWriteValue32 == nullptr) return false;
    int dev = flags.get_device();
    c10::cuda::CUDAGuard guard(dev);
    CUdeviceptr addr = reinterpret_cast<CUdeviceptr>(flags.data_ptr()) + (CUdeviceptr)offset * 4;
    SMR_CU_CHECK(d.cuStreamWriteValue32(current_stream(dev), addr, value, CU_STREAM_WRITE_VALUE_DEFAULT));
    return true;
  });
  m.def("cuda_view", &cuda_view, py::arg("alloc"), py::arg("rank"), py::arg("sizes"), py::arg("dtype"),
        py::arg("offset_bytes"), py::arg("multicast") = false);
  m.def("cuda_pad_view", &cuda_pad_view);

  py::class_<HostSymmAllocation, std::shared_ptr<HostSymmAllocation>> host_cls(m, "HostSymmAllocation");
  host_cls.def(py::init<const std::string&, size_t>())
      .def_property_readonly("shm_name", &HostSymmAllocation::shm_name)
      .def_property_readonly("payload_bytes", &HostSymmAllocation::payload_bytes)
      .def_property_readonly("block_bytes", &HostSymmAllocation::block_bytes)
      .def_property_readonly("pad_offset", &HostSymmAllocation::pad_offset)
      .def_property_readonly("rank", &HostSymmAllocation::rank)
      .def_property_readonly("world_size", &HostSymmAllocation::world_size)
      .def_property_readonly("rendezvoused", &HostSymmAllocation::rendezvoused)
      .def_property_readonly("local_ptr", [](const HostSymmAllocation& a) { return (uintptr_t)a.local_ptr(); })
      .def("rendezvous", &HostSymmAllocation::rendezvous)
      .def("release", &HostSymmAllocation::release)
      .def("barrier",
           [](HostSymmAllocation& a, uint32_t slot_base, uint64_t timeout_ns) {
             int peer = -1;
             uint32_t code;
             {
               py::gil_scoped_release nogil;
               code = a.barrier(slot_base, timeout_ns, &peer);
             }
             return py::make_tuple(code, peer);
           });
  host_cls
      .def("put_signal",
           [](HostSymmAllocation& a, int dst, uint32_t slot_base, uint64_t timeout_ns) {
             py::gil_scoped_release nogil;
             return a.put_signal(dst, slot_base, timeout_ns);
           })
      .def("wait_signal", [](HostSymmAllocation& a, int src, uint32_t slot_base, uint64_t timeout_ns) {
        py::gil_scoped_release nogil;
        return a.wait_signal(src, slot_base, timeout_ns);
      });
  m.def("host_view", &host_view);
  m.def("host_pad_view", &host_pad_view);
  m.def("host_all_reduce", &host_all_reduce);
  m.def("host_ll_all_reduce", [](const std::shared_ptr<HostSymmAllocation>& workspace, torch::Tensor in,
                                 torch::Tensor out, int64_t capacity_numel, uint64_t timeout_ns) {
    TORCH_CHECK(workspace->rendezvoused(), "workspace has not been rendezvoused");
    TORCH_CHECK(in.numel() == out.numel() && in.numel() % 8 == 0 && in.numel() <= capacity_numel, "bad sizes");
    const int ws = workspace->world_size();
    TORCH_CHECK(256 + (size_t)2 * ws * (capacity_numel / 8) * 32 <= workspace->payload_bytes(), "workspace too small");
    std::vector<void*> bases(ws);
    for (int r = 0; r < ws; ++r) bases[r] = workspace->peer_ptr(r);
    int peer = -1;
    uint32_t code;
    const uint16_t* src = bf16_ptr(in);
    uint16_t* dst = reinterpret_cast<uint16_t*>(out.data_ptr());
    {
      py::gil_scoped_release nogil;
      code = host_ll_all_reduce(bases.data(), workspace->rank(), ws, src, dst, (size_t)in.numel(),
                                (size_t)capacity_numel, timeout_ns, &peer);
    }
    return py::make_tuple(code, workspace->rank(), 0, peer, (int)kWhereOneShotEntry, 0);
  });
  // Epoch barrier hammered by threads (same protocol as the device EpochBarrier): returns
  // (codes per rank, max skew seen).
  m.def("host_epoch_barrier_stress", [](int world_size, int blocks, int iters, uint64_t timeout_ns) {
    TORCH_CHECK(world_size >= 1 && world_size <= kMaxWorldSize && blocks >= 1 && (uint32_t)blocks <= kArMaxBlocks,
                "bad stress configuration");
    std::vector<std::vector<uint32_t>> pads(world_size, std::vector<uint32_t>(kSignalPadSlots, 0u));
    std::vector<uint32_t*> pad_ptrs(world_size);
    for (int r = 0; r < world_size; ++r) pad_ptrs[r] = pads[r].data();
    std::vector<uint32_t> codes(world_size, 0);
    std::vector<std::atomic<int64_t>> progress(world_size);
    for (auto& c : progress) c.store(0);
    std::atomic<int64_t> max_skew{0};
    {
      py::gil_scoped_release nogil;
      std::vector<std::thread> threads;
      for (int r = 0; r < world_size; ++r) {
        threads.emplace_back([&, r] {
          std::vector<uint32_t> counts(blocks, 0);
          for (int it = 0; it < iters && codes[r] == 0; ++it) {
            for (int b = 0; b < blocks; ++b) {
              progress[r].fetch_add(1);
              int peer = -1;
              uint32_t code = host_epoch_barrier(pad_ptrs.data(), (uint32_t)b, r, world_size, &counts[b],
                                                 timeout_ns, &peer);
              if (code != kOk) {
                codes[r] = code;
                break;
              }
              int64_t mine = progress[r].load();
              for (int q = 0; q < world_size; ++q) {
                int64_t skew = mine - progress[q].load();
                int64_t cur = max_skew.load();
                while (skew > cur && !max_skew.compare_exchange_weak(cur, skew)) {
                }
              }
            }
          }
        });
      }
      for (auto& t : threads) t.join();
    }
    return py::make_tuple(codes, max_skew.load());
  });

  // Barrier protocol hammered by threads: `world_size` threads act as ranks over
  // private pads, each running `iters` barriers on each of `blocks` block ids.
  // `dead_rank` >= 0 never arrives.  Returns (codes per rank, sum of |pad|, max
  // counter skew seen), so a test can check completion, the all-zero pad and
  // that no rank ever ran ahead of a rank that had not arrived.
  m.def("host_barrier_stress", [](int world_size, int blocks, int iters, uint64_t timeout_ns, int dead_rank) {
    TORCH_CHECK(world_size >= 1 && world_size <= kMaxWorldSize && blocks >= 1 &&
                (uint32_t)blocks * world_size <= kBlockSlots, "bad stress configuration");
    std::vector<std::vector<uint32_t>> pads(world_size, std::vector<uint32_t>(kSignalPadSlots, 0u));
    std::vector<uint32_t*> pad_ptrs(world_size);
    for (int r = 0; r < world_size; ++r) pad_ptrs[r] = pads[r].data();
    std::vector<uint32_t> codes(world_size, 0);
    std::vector<std::atomic<int64_t>> progress(world_size);
    for (auto& c : progress) c.store(0);
    std::atomic<int64_t> max_skew{0};
    {
      py::gil_scoped_release nogil;
      std::vector<std::thread> threads;
      for (int r = 0; r < world_size; ++r) {
        if (r == dead_rank) continue;
        threads.emplace_back([&, r] {
          for (int it = 0; it < iters && codes[r] == 0; ++it) {
            for (int b = 0; b < blocks; ++b) {
              progress[r].fetch_add(1);
              int peer = -1;
              uint32_t code = host_barrier_signal_wait(pad_ptrs.data(), (uint32_t)b * world_size, r, world_size,
                                                       timeout_ns, &peer);
              if (code != kOk) {
                codes[r] = code;
                break;
              }
              // after a barrier nobody can be more than one barrier behind me
              int64_t mine = progress[r].load();
              for (int q = 0; q < world_size; ++q) {
                if (q == dead_rank) continue;
                int64_t skew = mine - progress[q].load();
                int64_t cur = max_skew.load();
                while (skew > cur && !max_skew.compare_exchange_weak(cur, skew)) {
                }
              }
            }
          }
        });
      }
      for (auto& t : threads) t.join();
    }
    uint64_t pad_sum = 0;
    for (auto& pad : pads)
      for (uint32_t v : pad) pad_sum += v;
    return py::make_tuple(codes, pad_sum, max_skew.load());
  });

  // ---- status ----
  m.def("read_status", &read_status);

  // ---- device ops ----
  m.def("barrier_test", [](const std::shared_ptr<CudaSymmAllocation>& a, int blocks, int threads,
                           uint64_t timeout_ns, int kind) {
    c10::cuda::CUDAGuard guard(a->device());
    rt_check(launch_barrier_test(view_of(*a), blocks, threads, timeout_ns, status_for(a->device()),
                                 current_stream(a->device()), kind), "barrier_test");
  }, py::arg("alloc"), py::arg("blocks"), py::arg("threads"), py::arg("timeout_ns"), py::arg("kind") = 0);
  m.def("channel_barrier", [](const std::shared_ptr<CudaSymmAllocation>& a, int channel,
                              uint64_t timeout_ns) {
    c10::cuda::CUDAGuard guard(a->device());
    rt_check(launch_channel_barrier(view_of(*a), channel, timeout_ns, status_for(a->device()),
                                    current_stream(a->device())), "channel_barrier");
  });
  m.def("put_signal", [](const std::shared_ptr<CudaSymmAllocation>& a, int dst, int channel, uint64_t timeout_ns) {
    c10::cuda::CUDAGuard guard(a->device());
    rt_check(launch_put_signal(view_of(*a), dst, channel, timeout_ns, status_for(a->device()),
                               current_stream(a->device())), "put_signal");
  });
  m.def("wait_signal", [](const std::shared_ptr<CudaSymmAllocation>& a, int src, int channel, uint64_t timeout_ns) {
    c10::cuda::CUDAGuard guard(a->device());
    rt_check(launch_wait_signal(view_of(*a), src, channel, timeout_ns, status_for(a->device()),
                                current_stream(a->device())), "wait_signal");
  });
  m.def("wait_flag", [](torch::Tensor flag, uint32_t target, uint64_t timeout_ns) {
    TORCH_CHECK(flag.is_cuda() && flag.element_size() == 4, "flag must be a 32-bit CUDA tensor");
    int dev = flag.get_device();
    c10::cuda::CUDAGuard guard(dev);
    rt_check(launch_wait_flag(reinterpret_cast<const uint32_t*>(flag.data_ptr()), target, timeout_ns, 0,
                              status_for(dev), current_stream(dev)), "wait_flag");
  });
  m.def("one_shot_all_reduce", [](const std::shared_ptr<CudaSymmAllocation>& a, int64_t offset_bytes,
                                  torch::Tensor out, int64_t numel, int max_blocks, bool exit_barrier,
                                  uint64_t timeout_ns, bool write_back) {
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == torch::kBFloat16 &&
                out.numel() == numel, "bad output tensor");
    c10::cuda::CUDAGuard guard(a->device());
    rt_check(launch_one_shot_all_reduce(view_of(*a), ptrs_of(*a), (size_t)offset_bytes, out.data_ptr(),
                                        (size_t)numel, max_blocks, exit_barrier, write_back, timeout_ns,
                                        status_for(a->device()), current_stream(a->device())),
             "one_shot_all_reduce");
  }, py::arg("alloc"), py::arg("offset_bytes"), py::arg("out"), py::arg("numel"), py::arg("max_blocks"),
     py::arg("exit_barrier"), py::arg("timeout_ns"), py::arg("write_back") = false);
  m.def("ll_all_reduce_workspace_bytes", &ll_all_reduce_workspace_bytes);
  m.def("ll_all_reduce", [](const std::shared_ptr<CudaSymmAllocation>& workspace, torch::Tensor in,
                            torch::Tensor out, int64_t capacity_numel, int max_blocks, uint64_t timeout_ns) {
    auto okt = [](const torch::Tensor& t) {
      return t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kBFloat16;
    };
    TORCH_CHECK(okt(in) && okt(out) && in.numel() == out.numel(), "in / out must be contiguous bf16 CUDA tensors");
    TORCH_CHECK(((uintptr_t)in.data_ptr() | (uintptr_t)out.data_ptr()) % 16 == 0, "in / out must be 16-byte aligned");
    c10::cuda::CUDAGuard guard(workspace->device());
    PeerView pv = view_of(*workspace);
    TORCH_CHECK(ll_all_reduce_workspace_bytes((size_t)capacity_numel, pv.world_size) <= workspace->payload_bytes(),
                "workspace too small");
    rt_check(launch_ll_all_reduce(pv, in.data_ptr(), out.data_ptr(), (size_t)in.numel(), (size_t)capacity_numel,
                                  max_blocks, timeout_ns, status_for(workspace->device()),
                                  current_stream(workspace->device())), "ll_all_reduce");
  });
  m.def("two_shot_all_reduce", [](const std::shared_ptr<CudaSymmAllocation>& a, int64_t offset_bytes,
                                  int64_t numel, int max_blocks, uint64_t timeout_ns) {
    c10::cuda::CUDAGuard guard(a->device());
    rt_check(launch_two_shot_all_reduce(view_of(*a), (size_t)offset_bytes, (size_t)numel, max_blocks,
                                        timeout_ns, status_for(a->device()),
                                        current_stream(a->device())), "two_shot_all_reduce");
  });
  m.def("multimem_all_reduce", [](const std::shared_ptr<CudaSymmAllocation>& a, int64_t offset_bytes,
                                  int64_t numel, int max_blocks, uint64_t timeout_ns) {
    c10::cuda::CUDAGuard guard(a->device());
    rt_check(launch_multimem_all_reduce(view_of(*a), (size_t)offset_bytes, (size_t)numel, max_blocks,
                                        timeout_ns, status_for(a->device()),
                                        current_stream(a->device())), "multimem_all_reduce");
  }, py::arg("alloc"), py::arg("offset_bytes"), py::arg("numel"), py::arg("max_blocks"), py::arg("timeout_ns"));

  // a: own shard (or all of A when mode == 0), b: [N, K], c: [M, N]
  // mode 2 (push): `aout_alloc` holds a_out; a is any CUDA tensor.
  m.def("ag_matmul", [](torch::Tensor a, torch::Tensor b, torch::Tensor c, int mode,
                        std::shared_ptr<CudaSymmAllocation> aout_alloc, int64_t aout_offset,
                        c10::optional<torch::Tensor> a_out, int block_n, int num_sms, uint64_t timeout_ns,
                        c10::optional<torch::Tensor> tail_scratch, int epilogue,
                        c10::optional<torch::Tensor> trace, int lead, int push_ahead,
                        bool push_plain_stores, int push_pieces, int panel_w) {
    const auto dtype = a.scalar_type();
    const bool fp8 = dtype == at::kFloat8_e4m3fn;
    TORCH_CHECK(fp8 || dtype == torch::kBFloat16, "a must be bfloat16 or float8_e4m3fn");
    auto ok2d = [dtype](const torch::Tensor& t) {
      return t.is_cuda() && t.dim() == 2 && t.is_contiguous() && t.scalar_type() == dtype;
    };
    TORCH_CHECK(ok2d(a) && ok2d(b) && ok2d(c), "a, b, c must be contiguous 2-D CUDA tensors of one dtype");
    TORCH_CHECK(a.size(1) == b.size(1), "A[*, K] and B[N, K] disagree on K");
    int dev = a.get_device();
    TORCH_CHECK(b.get_device() == dev && c.get_device() == dev, "a, b and c must live on one GPU");
    c10::cuda::CUDAGuard guard(dev);
    cudaStream_t stream = current_stream(dev);
    AgMatmulArgs args{};
    args.a_local = a.data_ptr();
    args.b = b.data_ptr();
    args.c = c.data_ptr();
    args.N = (int)b.size(0);
    args.K = (int)a.size(1);
    args.elem_bytes = fp8 ? 1 : 2;
    args.epilogue = epilogue;
    TORCH_CHECK(epilogue == 0 || (epilogue == 1 && !fp8), "the SwiGLU epilogue is a bfloat16 epilogue");
    args.block_n = block_n;
    args.num_sms = num_sms;
    args.timeout_ns = timeout_ns;
    args.status = status_for(dev);
    args.mode = mode;
    if (mode != 0) {
      TORCH_CHECK(mode == 2, "mode must be 0 (no gather) or 2 (push)");
      TORCH_CHECK(aout_alloc != nullptr && a_out.has_value(), "the gather needs a symmetric a_out");
      PeerView pv = view_of(*aout_alloc);
      args.rank = pv.rank;
      args.world_size = pv.world_size;
      args.rows_per_rank = (int)a.size(0);
      args.M = args.rows_per_rank * pv.world_size;
      args.pads = pv.pads;
      args.barrier_block_base = 1024;
      TORCH_CHECK(ok2d(*a_out) && a_out->size(0) == args.M && a_out->size(1) == args.K, "a_out must be [M, K] of a's dtype");
      args.a_out = a_out->data_ptr();
      TORCH_CHECK((char*)a_out->data_ptr() == (char*)aout_alloc->local_ptr() + aout_offset,
                  "a_out does not sit at aout_offset of its allocation");
      args.aout_buffers = pv.buffers;
      args.aout_mc = pv.multicast;
      args.aout_offset = (size_t)aout_offset;
      args.local_pad = aout_alloc->peer_pad(pv.rank);
    } else {
      args.M = (int)a.size(0);
    }
    TORCH_CHECK(c.size(0) == args.M && c.size(1) == (epilogue == 1 ? args.N / 2 : args.N),
                "c must be [M, N] ([M, N / 2] with the SwiGLU epilogue)");
    if (tail_scratch.has_value()) {
      // first 4 KiB: arrival counters; the rest: fp32 partial accumulators
      TORCH_CHECK(tail_scratch->is_cuda() && tail_scratch->is_contiguous() && tail_scratch->nbytes() > 8192,
                  "tail_scratch must be a contiguous CUDA tensor");
      char* base = static_cast<char*>(tail_scratch->data_ptr());
      args.tail_counters = reinterpret_cast<uint32_t*>(base);
      args.tail_counter_slots = 1024;
      args.tail_scratch = base + 4096;
      args.tail_scratch_bytes = tail_scratch->nbytes() - 4096;
    }
    args.lead = lead;
    args.push_ahead = push_ahead;
    args.push_plain_stores = push_plain_stores ? 1 : 0;
    args.push_pieces = push_pieces;
    args.panel_w = panel_w;
    if (trace.has_value()) {
      TORCH_CHECK(trace->is_cuda() && trace->get_device() == dev && trace->is_contiguous() &&
                  trace->scalar_type() == torch::kInt64 && trace->numel() >= (int64_t)num_sms * 12,
                  "trace must be a contiguous int64 CUDA tensor of num_sms x 12 words");
      args.trace = reinterpret_cast<uint64_t*>(trace->data_ptr());
    }
    rt_check(launch_ag_matmul_2cta(args, stream), "ag_matmul");
  }, py::arg("a"), py::arg("b"), py::arg("c"), py::arg("mode"), py::arg("aout_alloc"), py::arg("aout_offset"),
     py::arg("a_out"), py::arg("block_n"), py::arg("num_sms"), py::arg("timeout_ns"),
     py::arg("tail_scratch") = py::none(), py::arg("epilogue") = 0,
     py::arg("trace") = py::none(), py::arg("lead") = -1,
     py::arg("push_ahead") = 0, py::arg("push_plain_stores") = false,
     py::arg("push_pieces") = 0, py::arg("panel_w") = 0);

  m.def("check_push_schedule", &check_push_schedule);
  m.def("check_pair_work", &check_pair_work);
  m.def("check_rs_pair_schedule", &check_rs_pair_schedule);
  m.def("check_rs_progress", &check_rs_progress);
  m.def("gemv_batch_tile", &gemv_batch_tile);
  m.def("gemv_workspace_bytes", [](int batch_tile, int N, int world_size) {
    return gemv_workspace_bytes(batch_tile, N, world_size, nullptr, nullptr, nullptr);
  });
  m.def("gemv_tc_workspace_bytes", [](int N, int K, int world_size, int num_sms, bool tagged) {
    return gemv_tc_workspace_bytes(N, K, world_size, num_sms, nullptr, nullptr, nullptr, nullptr, tagged);
  }, py::arg("N"), py::arg("K"), py::arg("world_size"), py::arg("num_sms"), py::arg("tagged") = false);
  m.def("gemv_all_reduce", [](torch::Tensor x, torch::Tensor w, torch::Tensor out,
                              const std::shared_ptr<CudaSymmAllocation>& workspace, int64_t ws_offset,
                              uint64_t timeout_ns, bool tensor_core, int num_sms, bool tagged, bool weights_nk) {
    auto ok2d = [](const torch::Tensor& t) {
      return t.is_cuda() && t.dim() == 2 && t.is_contiguous() && t.scalar_type() == torch::kBFloat16;
    };
    TORCH_CHECK(ok2d(x) && ok2d(w) && ok2d(out), "x, w, out must be contiguous 2-D bf16 CUDA tensors");
    TORCH_CHECK(!weights_nk || tensor_core, "weights stored [N, K] are read by the tcgen05 kernel only");
    const int64_t w_k = weights_nk ? w.size(1) : w.size(0), w_n = weights_nk ? w.size(0) : w.size(1);
    TORCH_CHECK(x.size(1) == w_k && out.size(0) == x.size(0) && out.size(1) == w_n,
                "need x[B, K], w[K, N] (or [N, K] with weights_nk), out[B, N]");
    int dev = x.get_device();
    TORCH_CHECK(w.get_device() == dev && out.get_device() == dev && workspace->device() == dev,
                "x, w, out and the workspace must live on one GPU");
    c10::cuda::CUDAGuard guard(dev);
    GemvArgs args{};
    args.x = x.data_ptr();
    args.w = w.data_ptr();
    args.out = out.data_ptr();
    args.batch = (int)x.size(0);
    args.K = (int)x.size(1);
    args.N = (int)w_n;
    args.pv = view_of(*workspace);
    args.ws_offset = (size_t)ws_offset;
    args.timeout_ns = timeout_ns;
    args.status = status_for(dev);
    int bt = gemv_batch_tile(args.batch);
    TORCH_CHECK(bt > 0, "batch must be between 1 and 16");
    TORCH_CHECK(!tagged || tensor_core, "the tagged exchange belongs to the tcgen05 kernel");
    if (tensor_core) {
      TORCH_CHECK(gemv_tc_workspace_bytes(args.N, args.K, args.pv.world_size, num_sms, nullptr, nullptr, nullptr,
                                          nullptr, tagged) <= workspace->payload_bytes(), "workspace too small");
      rt_check(launch_gemv_all_reduce_tc(args, num_sms, current_stream(dev), tagged, weights_nk),
               "gemv_all_reduce (tcgen05)");
      return;
    }
    TORCH_CHECK(gemv_workspace_bytes(bt, args.N, args.pv.world_size, nullptr, nullptr, nullptr) + (size_t)ws_offset
                    <= workspace->payload_bytes(), "workspace too small");
    rt_check(launch_gemv_all_reduce(args, current_stream(dev)), "gemv_all_reduce");
  }, py::arg("x"), py::arg("w"), py::arg("out"), py::arg("workspace"), py::arg("ws_offset"),
     py::arg("timeout_ns"), py::arg("tensor_core") = false, py::arg("num_sms") = 148, py::arg("tagged") = false,
     py::arg("weights_nk") = false);

  m.def("matmul_rs_workspace_bytes", &matmul_rs_workspace_bytes);
  m.def("matmul_reduce_scatter", [](torch::Tensor a, torch::Tensor b, torch::Tensor out,
                                    const std::shared_ptr<CudaSymmAllocation>& workspace, int num_sms,
                                    uint64_t timeout_ns, c10::optional<torch::Tensor> trace, int panel_w) {
    auto ok2d = [](const torch::Tensor& t) {
      return t.is_cuda() && t.dim() == 2 && t.is_contiguous() && t.scalar_type() == torch::kBFloat16;
    };
    TORCH_CHECK(ok2d(a) && ok2d(b) && ok2d(out), "a, b, out must be contiguous 2-D bf16 CUDA tensors");
    TORCH_CHECK(a.size(1) == b.size(1), "A[M, K] and B[N, K] disagree on K");
    int dev = a.get_device();
    TORCH_CHECK(b.get_device() == dev && out.get_device() == dev && workspace->device() == dev,
                "a, b, out and the workspace must live on one GPU");
    c10::cuda::CUDAGuard guard(dev);
    MatmulRsArgs args{};
    args.a = a.data_ptr();
    args.b = b.data_ptr();
    args.out = out.data_ptr();
    args.M = (int)a.size(0);
    args.N = (int)b.size(0);
    args.K = (int)a.size(1);
    args.pv = view_of(*workspace);
    TORCH_CHECK(out.size(0) * args.pv.world_size == args.M && out.size(1) == args.N, "out must be [M / WS, N]");
    TORCH_CHECK(matmul_rs_workspace_bytes(args.M, args.N) <= workspace->payload_bytes(), "workspace too small");
    args.inbox_offset = 0;
    for (int r = 0; r < args.pv.world_size; ++r) args.peer_base[r] = workspace->peer_ptr(r);
    args.local_pad = workspace->peer_pad(args.pv.rank);
    args.num_sms = num_sms;
    args.timeout_ns = timeout_ns;
    args.status = status_for(dev);
    args.panel_w = panel_w;
    if (trace.has_value()) {
      TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == torch::kInt64 && trace->numel() >= 4 * num_sms,
                  "trace must be an int64 CUDA tensor of at least 4 * num_sms elements");
      args.trace = reinterpret_cast<uint64_t*>(trace->data_ptr());
    }
    rt_check(launch_matmul_reduce_scatter(args, current_stream(dev)), "matmul_reduce_scatter");
  }, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("workspace"), py::arg("num_sms"),
     py::arg("timeout_ns"), py::arg("trace") = py::none(), py::arg("panel_w") = 0);

  // all-reduce form: `out` [M, N] lives in the symmetric allocation `out_alloc` at `out_offset`
  m.def("matmul_all_reduce", [](torch::Tensor a, torch::Tensor b, torch::Tensor out,
                                const std::shared_ptr<CudaSymmAllocation>& out_alloc, int64_t out_offset,
                                const std::shared_ptr<CudaSymmAllocation>& workspace, int num_sms,
                                uint64_t timeout_ns, int panel_w) {
    auto ok2d = [](const torch::Tensor& t) {
      return t.is_cuda() && t.dim() == 2 && t.is_contiguous() && t.scalar_type() == torch::kBFloat16;
    };
    TORCH_CHECK(ok2d(a) && ok2d(b) && ok2d(out), "a, b, out must be contiguous 2-D bf16 CUDA tensors");
    TORCH_CHECK(a.size(1) == b.size(1), "A[M, K] and B[N, K] disagree on K");
    TORCH_CHECK(out.size(0) == a.size(0) && out.size(1) == b.size(0), "out must be [M, N]");
    TORCH_CHECK((char*)out.data_ptr() == (char*)out_alloc->local_ptr() + out_offset,
                "out does not sit at out_offset of its allocation");
    int dev = a.get_device();
    TORCH_CHECK(b.get_device() == dev && out.get_device() == dev && workspace->device() == dev &&
                out_alloc->device() == dev, "a, b, out and the workspace must live on one GPU");
    c10::cuda::CUDAGuard guard(dev);
    MatmulRsArgs args{};
    args.a = a.data_ptr();
    args.b = b.data_ptr();
    args.out = nullptr;
    args.M = (int)a.size(0);
    args.N = (int)b.size(0);
    args.K = (int)a.size(1);
    args.pv = view_of(*workspace);
    PeerView ov = view_of(*out_alloc);
    TORCH_CHECK(ov.world_size == args.pv.world_size && ov.rank == args.pv.rank, "out and workspace: different groups");
    TORCH_CHECK(matmul_rs_workspace_bytes(args.M, args.N) <= workspace->payload_bytes(), "workspace too small");
    args.inbox_offset = 0;
    for (int r = 0; r < args.pv.world_size; ++r) args.peer_base[r] = workspace->peer_ptr(r);
    args.local_pad = workspace->peer_pad(args.pv.rank);
    args.num_sms = num_sms;
    args.timeout_ns = timeout_ns;
    args.status = status_for(dev);
    args.all_reduce = true;
    args.panel_w = panel_w;
    args.ar_peers = ov.buffers;
    args.ar_mc = ov.multicast;
    args.ar_offset = (size_t)out_offset;
    rt_check(launch_matmul_reduce_scatter(args, current_stream(dev)), "matmul_all_reduce");
  }, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("out_alloc"), py::arg("out_offset"), py::arg("workspace"),
     py::arg("num_sms"), py::arg("timeout_ns"), py::arg("panel_w") = 0);

  // ---- rank-local layer glue ----
  m.def("rms_norm", [](torch::Tensor x, c10::optional<torch::Tensor> residual, torch::Tensor w,
                       c10::optional<torch::Tensor> sum_out, torch::Tensor out, double eps) {
    auto ok = [](const torch::Tensor& t) {
      return t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kBFloat16;
    };
    TORCH_CHECK(ok(x) && ok(w) && ok(out) && x.dim() == 2 && w.dim() == 1 && w.size(0) == x.size(1) &&
                out.sizes() == x.sizes(), "rms_norm: x[rows, H], w[H], out[rows, H], contiguous bf16 on the GPU");
    TORCH_CHECK(!residual.has_value() || (ok(*residual) && residual->sizes() == x.sizes()), "residual must match x");
    TORCH_CHECK(!sum_out.has_value() || (residual.has_value() && ok(*sum_out) && sum_out->sizes() == x.sizes()),
                "sum_out needs a residual and must match x");
    int dev = x.get_device();
    c10::cuda::CUDAGuard guard(dev);
    rt_check(launch_rms_norm(x.data_ptr(), residual ? residual->data_ptr() : nullptr, w.data_ptr(),
                             sum_out ? sum_out->data_ptr() : nullptr, out.data_ptr(), (int)x.size(0),
                             (int)x.size(1), (float)eps, current_stream(dev)), "rms_norm");
  }, py::arg("x"), py::arg("residual"), py::arg("w"), py::arg("sum_out"), py::arg("out"), py::arg("eps"));
  // `pos` (optional): int32 CUDA tensor of one element that holds the first position; read on the device
  m.def("rope_inplace", [](torch::Tensor qkv, int n_heads, int head_dim, int seq, int pos0, double theta,
                           int num_sms, c10::optional<torch::Tensor> pos) {
    TORCH_CHECK(qkv.is_cuda() && qkv.is_contiguous() && qkv.dim() == 2 && qkv.scalar_type() == torch::kBFloat16,
                "rope_inplace: qkv[tokens, row] contiguous bf16 on the GPU");
    int dev = qkv.get_device();
    TORCH_CHECK(!pos.has_value() || (pos->is_cuda() && pos->get_device() == dev && pos->numel() == 1 &&
                                     pos->scalar_type() == torch::kInt32),
                "rope_inplace: pos must be an int32 tensor of one element on qkv's GPU");
    c10::cuda::CUDAGuard guard(dev);
    rt_check(launch_rope_inplace(qkv.data_ptr(), qkv.size(0), (int)qkv.size(1), n_heads, head_dim, seq, pos0,
                                 pos ? static_cast<const int*>(pos->data_ptr()) : nullptr, (float)theta, num_sms,
                                 current_stream(dev)), "rope_inplace");
  }, py::arg("qkv"), py::arg("n_heads"), py::arg("head_dim"), py::arg("seq"), py::arg("pos0"), py::arg("theta"),
     py::arg("num_sms"), py::arg("pos") = py::none());
  m.def("silu_mul", [](torch::Tensor gate_up, torch::Tensor out, int num_sms) {
    auto ok = [](const torch::Tensor& t) {
      return t.is_cuda() && t.is_contiguous() && t.dim() == 2 && t.scalar_type() == torch::kBFloat16;
    };
    TORCH_CHECK(ok(gate_up) && ok(out) && gate_up.size(1) == 2 * out.size(1) && gate_up.size(0) == out.size(0),
                "silu_mul: gate_up[rows, 2F], out[rows, F], contiguous bf16 on the GPU");
    int dev = gate_up.get_device();
    c10::cuda::CUDAGuard guard(dev);
    rt_check(launch_silu_mul(gate_up.data_ptr(), out.data_ptr(), gate_up.size(0), (int)out.size(1), num_sms,
                             current_stream(dev)), "silu_mul");
  });

  m.def("decode_attention_scratch_bytes", [](int batch, int hkv, int head_dim, int s_max) {
    return decode_attention_scratch_bytes(batch, hkv, head_dim, s_max, nullptr);
  });
  // `pos` (optional): int32 CUDA tensor of one element holding the position; read on the device
  m.def("decode_attention", [](torch::Tensor qkv, torch::Tensor k_cache, torch::Tensor v_cache, torch::Tensor out,
                               torch::Tensor scratch, int hq, int hkv, int pos0, c10::optional<torch::Tensor> pos,
                               double rope_theta) {
    auto ok = [](const torch::Tensor& t) {
      return t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kBFloat16;
    };
    TORCH_CHECK(ok(qkv) && ok(k_cache) && ok(v_cache) && ok(out) && qkv.dim() == 2 && k_cache.dim() == 4 &&
                v_cache.sizes() == k_cache.sizes(), "decode_attention: contiguous bf16 CUDA tensors, caches [B, S, hkv, D]");
    const int B = (int)qkv.size(0), s_max = (int)k_cache.size(1), D = (int)k_cache.size(3);
    TORCH_CHECK(k_cache.size(0) == B && k_cache.size(2) == hkv && qkv.size(1) == (int64_t)(hq + 2 * hkv) * D &&
                out.dim() == 2 && out.size(0) == B && out.size(1) == (int64_t)hq * D,
                "decode_attention: qkv [B, (hq + 2 hkv) D], out [B, hq D]");
    TORCH_CHECK(scratch.is_cuda() && scratch.is_contiguous() && scratch.scalar_type() == torch::kUInt8,
                "scratch must be a uint8 CUDA tensor");
    int dev = qkv.get_device();
    TORCH_CHECK(!pos.has_value() || (pos->is_cuda() && pos->get_device() == dev && pos->numel() == 1 &&
                                     pos->scalar_type() == torch::kInt32),
                "decode_attention: pos must be an int32 tensor of one element on the same GPU");
    c10::cuda::CUDAGuard guard(dev);
    rt_check(launch_decode_attention(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                     scratch.data_ptr(), (size_t)scratch.nbytes(), B, hq, hkv, D, s_max, pos0,
                                     pos ? static_cast<const int*>(pos->data_ptr()) : nullptr, (float)rope_theta,
                                     current_stream(dev)),
             "decode_attention");
  }, py::arg("qkv"), py::arg("k_cache"), py::arg("v_cache"), py::arg("out"), py::arg("scratch"), py::arg("hq"),
     py::arg("hkv"), py::arg("pos0"), py::arg("pos") = py::none(), py::arg("rope_theta") = 0.0);

  // ---- oracles (CPU tensors) ----
  m.def("oracle_rms_norm_bf16", [](torch::Tensor x, c10::optional<torch::Tensor> residual, torch::Tensor w,
                                   double eps) {
    TORCH_CHECK(x.dim() == 2 && w.dim() == 1 && w.size(0) == x.size(1), "x[rows, H], w[H]");
    torch::Tensor out = torch::empty_like(x), sum = torch::empty_like(x);
    rms_norm_bf16(bf16_ptr(x), residual ? bf16_ptr(*residual) : nullptr, bf16_ptr(w),
                  residual ? reinterpret_cast<uint16_t*>(sum.data_ptr()) : nullptr,
                  reinterpret_cast<uint16_t*>(out.data_ptr()), (int)x.size(0), (int)x.size(1), (float)eps);
    return std::make_pair(out, residual ? sum : x);
  });
  m.def("oracle_rope_bf16", [](torch::Tensor qkv, int n_heads, int head_dim, int seq, int pos0, double theta) {
    TORCH_CHECK(qkv.dim() == 2 && (int64_t)n_heads * head_dim <= qkv.size(1) && head_dim % 2 == 0, "qkv[tokens, row]");
    bf16_ptr(qkv);   // dtype / device / contiguity check
    torch::Tensor out = qkv.clone();
    rope_bf16(reinterpret_cast<uint16_t*>(out.data_ptr()), out.size(0), (int)out.size(1), n_heads, head_dim, seq,
              pos0, (float)theta);
    return out;
  });
  m.def("oracle_silu_mul_bf16", [](torch::Tensor gu) {
    TORCH_CHECK(gu.dim() == 2 && gu.size(1) % 2 == 0, "gate_up[rows, 2F]");
    torch::Tensor out = torch::empty({gu.size(0), gu.size(1) / 2}, gu.options());
    silu_mul_bf16(bf16_ptr(gu), reinterpret_cast<uint16_t*>(out.data_ptr()), gu.size(0), (int)gu.size(1) / 2);
    return out;
  });
  // the caches are updated in place (CPU tensors), as the kernel does
  m.def("oracle_decode_attention_bf16", [](torch::Tensor qkv, torch::Tensor k_cache, torch::Tensor v_cache, int hq,
                                           int hkv, int pos) {
    TORCH_CHECK(qkv.dim() == 2 && k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes() && hkv > 0 &&
                k_cache.size(2) == hkv && k_cache.size(0) == qkv.size(0) && hq % hkv == 0, "bad shapes");
    const int D = (int)k_cache.size(3), s_max = (int)k_cache.size(1), B = (int)qkv.size(0);
    TORCH_CHECK(qkv.size(1) == (int64_t)(hq + 2 * hkv) * D && pos >= 0 && pos < s_max, "bad qkv row or position");
    TORCH_CHECK(k_cache.is_contiguous() && v_cache.is_contiguous() && qkv.is_contiguous(), "contiguous tensors");
    bf16_ptr(k_cache);
    bf16_ptr(v_cache);
    torch::Tensor out = torch::empty({B, (int64_t)hq * D}, qkv.options());
    decode_attention_bf16(bf16_ptr(qkv), reinterpret_cast<uint16_t*>(k_cache.data_ptr()),
                          reinterpret_cast<uint16_t*>(v_cache.data_ptr()),
                          reinterpret_cast<uint16_t*>(out.data_ptr()), B, hq, hkv, D, s_max, pos);
    return out;
  });
  m.def("oracle_ordered_sum_bf16", [](std::vector<torch::Tensor> srcs) {
    TORCH_CHECK(!srcs.empty(), "need at least one source");
    std::vector<const uint16_t*> p;
    for (auto& t : srcs) p.push_back(bf16_ptr(t));
    torch::Tensor out = torch::empty_like(srcs[0]);
    ordered_sum_bf16(p.data(), (int)p.size(), reinterpret_cast<uint16_t*>(out.data_ptr()), (size_t)out.numel());
    return out;
  });
  m.def("oracle_fp32_sum_bf16", [](std::vector<torch::Tensor> srcs) {
    TORCH_CHECK(!srcs.empty(), "need at least one source");
    std::vector<const uint16_t*> p;
    for (auto& t : srcs) p.push_back(bf16_ptr(t));
    torch::Tensor out = torch::empty_like(srcs[0]);
    fp32_sum_bf16(p.data(), (int)p.size(), reinterpret_cast<uint16_t*>(out.data_ptr()), (size_t)out.numel());
    return out;
  });
  m.def("oracle_gemm_nt_bf16", [](torch::Tensor a, torch::Tensor b) {
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "A[M,K], B[N,K]");
    torch::Tensor c = torch::empty({a.size(0), b.size(0)}, a.options());
    gemm_nt_bf16(bf16_ptr(a), bf16_ptr(b), reinterpret_cast<uint16_t*>(c.data_ptr()), (int)a.size(0),
                 (int)b.size(0), (int)a.size(1));
    return c;
  });
  m.def("oracle_gemv_f32", [](torch::Tensor x, torch::Tensor w) {
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(0), "x[B,K], w[K,N]");
    torch::Tensor y = torch::empty({x.size(0), w.size(1)}, x.options().dtype(torch::kFloat32));
    gemv_f32(bf16_ptr(x), bf16_ptr(w), y.data_ptr<float>(), (int)x.size(0), (int)x.size(1), (int)w.size(1));
    return y;
  });
}
