// CUDA driver entry points, resolved at first use with dlopen("libcuda.so.1").
// The library therefore loads on a machine without a GPU driver (the CPU
// backend and the oracles still work there); every GPU entry point fails with
// a clear message instead.
#pragma once
#include <cuda.h>

#include <stdexcept>
#include <string>

namespace smr {

struct DriverApi {
#define SMR_DRIVER_FN(name) decltype(&::name) name = nullptr;
  SMR_DRIVER_FN(cuGetErrorString)
  SMR_DRIVER_FN(cuDeviceGet)
  SMR_DRIVER_FN(cuDeviceGetAttribute)
  SMR_DRIVER_FN(cuCtxGetCurrent)
  SMR_DRIVER_FN(cuCtxSetCurrent)
  SMR_DRIVER_FN(cuDevicePrimaryCtxRetain)
  SMR_DRIVER_FN(cuMemGetAllocationGranularity)
  SMR_DRIVER_FN(cuMemCreate)
  SMR_DRIVER_FN(cuMemRelease)
  SMR_DRIVER_FN(cuMemAddressReserve)
  SMR_DRIVER_FN(cuMemAddressFree)
  SMR_DRIVER_FN(cuMemMap)
  SMR_DRIVER_FN(cuMemUnmap)
  SMR_DRIVER_FN(cuMemSetAccess)
  SMR_DRIVER_FN(cuMemExportToShareableHandle)
  SMR_DRIVER_FN(cuMemImportFromShareableHandle)
  SMR_DRIVER_FN(cuMulticastCreate)
  SMR_DRIVER_FN(cuMulticastAddDevice)
  SMR_DRIVER_FN(cuMulticastBindMem)
  SMR_DRIVER_FN(cuMulticastUnbind)
  SMR_DRIVER_FN(cuMulticastGetGranularity)
  SMR_DRIVER_FN(cuTensorMapEncodeTiled)
  // optional (nullptr when the driver lacks it): stream-ordered 32-bit write with a system-scope fence before it
  SMR_DRIVER_FN(cuStreamWriteValue32)
#undef SMR_DRIVER_FN
  // Throws std::runtime_error when no driver library can be loaded.
  static const DriverApi& get();
};

std::string driver_error_string(CUresult r);

#define SMR_CU_CHECK(expr)                                                            \
  do {                                                                                \
    CUresult _r = (expr);                                                             \
    if (_r != CUDA_SUCCESS)                                                           \
      throw std::runtime_error(std::string(#expr) + " failed: " +                     \
                               ::smr::driver_error_string(_r));                       \
  } while (0)

}  // namespace smr
