// Launch-time check that every CTA of a grid can be resident at once.
//
// The CTAs of the fused kernels wait for one another (arrival counters of a
// split-K tail, flags written by the CTAs of a peer rank that run the same grid,
// the K splits of a GEMV tile).  A grid that does not fit on the GPU in one wave
// would leave the first wave waiting for CTAs that cannot start; the bounded
// waits would turn that into a timeout seconds later.  The launchers call this
// first and refuse such a grid with cudaErrorCooperativeLaunchTooLarge instead.
// It is the occupancy arithmetic of an otherwise idle GPU: a kernel of another
// stream that holds SMs at the time of the launch is not seen (the bounded
// waits remain the backstop for that).  No upstream counterpart: the upstream
// kernels never wait for a CTA of their own grid.
#pragma once
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

namespace smr {

// 0 when `grid` CTAs of `threads` threads and `smem` bytes of dynamic shared memory (in clusters of
// `cluster` CTAs) fit on the current device at once, else a cudaError_t.  Answers are cached per
// (kernel, launch shape, device): the occupancy queries are host-side arithmetic, but a decode
// step launches these kernels every few microseconds.
template <class Kernel>
inline int check_co_resident(Kernel kernel, int grid, int threads, size_t smem, int cluster = 1) {
  static std::mutex mu;
  static std::unordered_map<unsigned long long, int> cache;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  unsigned long long key = reinterpret_cast<unsigned long long>(reinterpret_cast<const void*>(kernel));
  key = key * 1000003ull + (unsigned long long)grid;
  key = key * 1000003ull + (unsigned long long)threads;
  key = key * 1000003ull + (unsigned long long)smem;
  key = key * 1000003ull + (unsigned long long)(cluster * 64 + dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  int verdict = 0;
  if (cluster <= 1) {
    int sms = 0, per_sm = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
    if (e != cudaSuccess) return (int)e;
    verdict = (long long)per_sm * sms >= grid ? 0 : (int)cudaErrorCooperativeLaunchTooLarge;
  } else {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
    if (e != cudaSuccess) return (int)e;
    verdict = (long long)clusters * cluster >= grid ? 0 : (int)cudaErrorCooperativeLaunchTooLarge;
  }
  std::lock_guard<std::mutex> lock(mu);
  cache[key] = verdict;
  return verdict;
}

}  // namespace smr
