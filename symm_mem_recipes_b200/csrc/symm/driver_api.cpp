#include "driver_api.h"

#include <dlfcn.h>

#include <mutex>

namespace smr {

namespace {
DriverApi g_api;
std::once_flag g_once;
std::string g_load_error;

void load() {
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (lib == nullptr) lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
  if (lib == nullptr) {
    g_load_error = std::string("cannot load the CUDA driver library: ") + dlerror();
    return;
  }
#define SMR_LOAD(name)                                                     \
  g_api.name = reinterpret_cast<decltype(g_api.name)>(dlsym(lib, #name)); \
  if (g_api.name == nullptr) {                                             \
    g_load_error = "CUDA driver lacks symbol " #name;                      \
    return;                                                                \
  }
  SMR_LOAD(cuGetErrorString)
  SMR_LOAD(cuDeviceGet)
  SMR_LOAD(cuDeviceGetAttribute)
  SMR_LOAD(cuCtxGetCurrent)
  SMR_LOAD(cuCtxSetCurrent)
  SMR_LOAD(cuDevicePrimaryCtxRetain)
  SMR_LOAD(cuMemGetAllocationGranularity)
  SMR_LOAD(cuMemCreate)
  SMR_LOAD(cuMemRelease)
  SMR_LOAD(cuMemAddressReserve)
  SMR_LOAD(cuMemAddressFree)
  SMR_LOAD(cuMemMap)
  SMR_LOAD(cuMemUnmap)
  SMR_LOAD(cuMemSetAccess)
  SMR_LOAD(cuMemExportToShareableHandle)
  SMR_LOAD(cuMemImportFromShareableHandle)
  SMR_LOAD(cuMulticastCreate)
  SMR_LOAD(cuMulticastAddDevice)
  SMR_LOAD(cuMulticastBindMem)
  SMR_LOAD(cuMulticastUnbind)
  SMR_LOAD(cuMulticastGetGranularity)
  SMR_LOAD(cuTensorMapEncodeTiled)
#undef SMR_LOAD
  // cuda.h maps the name to its _v2 entry point (per-stream memory-operation ordering)
  g_api.cuStreamWriteValue32 =
      reinterpret_cast<decltype(g_api.cuStreamWriteValue32)>(dlsym(lib, "cuStreamWriteValue32_v2"));
}
}  // namespace

const DriverApi& DriverApi::get() {
  std::call_once(g_once, load);
  if (!g_load_error.empty()) throw std::runtime_error(g_load_error);
  return g_api;
}

std::string driver_error_string(CUresult r) {
  const char* s = nullptr;
  try {
    if (DriverApi::get().cuGetErrorString(r, &s) == CUDA_SUCCESS && s != nullptr) return s;
  } catch (...) {
  }
  return "CUresult " + std::to_string((int)r);
}

}  // namespace smr
