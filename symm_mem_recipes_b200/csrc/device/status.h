// Status word shared by every kernel of the library.
//
// No device wait in this library is unbounded: a spin that runs out of time
// records WHY in a `Status` record that lives in device memory and makes the
// kernel return.  The host reads the record back (`check_status`) and raises a
// Python exception; the CUDA context stays usable.  The upstream recipes spin
// forever instead (symm_mem_recipes/triton_barrier.py:112-139,
// symm_mem_recipes/triton_all_gather_matmul.py:72-95).
#pragma once
#include <stdint.h>

namespace smr {

enum StatusCode : uint32_t {
  kOk = 0,
  kTimeoutBarrierSend = 1,   // peer never consumed our previous signal
  kTimeoutBarrierWait = 2,   // peer never arrived
  kTimeoutFlag = 3,          // a progress / arrival flag never reached its value
  kTimeoutMbarrier = 4,      // an mbarrier phase never completed (pipeline bug)
  kBadArgument = 5,
};

// 32 bytes; the first reporter wins (CAS on `code`), later ones are dropped.
struct Status {
  uint32_t code;
  uint32_t rank;
  uint32_t block;
  uint32_t peer;
  uint32_t where;   // call-site tag chosen by the kernel
  uint32_t aux;
  uint32_t pad[2];
};

// Call-site tags (the `where` field).
enum Where : uint32_t {
  kWhereBarrierKernel = 1,
  kWhereOneShotEntry = 10,
  kWhereOneShotExit = 11,
  kWhereTwoShotEntry = 12,
  kWhereTwoShotExit = 13,
  kWhereMultimemEntry = 14,
  kWhereMultimemExit = 15,
  kWhereGemmFull = 20,
  kWhereGemmEmpty = 21,
  kWhereGemmTmemFull = 22,
  kWhereGemmTmemEmpty = 23,
  kWhereGemmProgress = 24,
  kWhereCopierEntry = 25,
  kWhereCopierExit = 26,
  kWhereGemvArrive = 30,
  kWhereGemvEpoch = 31,
  kWhereRsArrive = 40,
  kWhereRsEntry = 41,
  kWhereRsExit = 42,
  kWhereTest = 99,
};

}  // namespace smr
