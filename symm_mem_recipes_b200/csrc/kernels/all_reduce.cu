// Barrier and all-reduce kernels over symmetric memory (bf16).
//
//  * one-shot:  every rank reads all WS peer buffers and sums them, in rank
//    order 0..WS-1 starting from +0 with bf16 adds.  Same arithmetic, hence
//    same bits on every rank, as
//    symm_mem_recipes/triton_one_shot_all_reduce.py:59-93; the loads are issued
//    starting at the rank's own neighbour so that the WS-1 links are busy at
//    once (upstream loads peer 0 first on every rank, :86-88).
//  * two-shot:  rank r reduces slice r (reduce-scatter by peer loads) and
//    stores the result into slice r of every peer (all-gather by peer stores).
//  * multimem:  rank r reduces slice r inside the NVSwitch
//    (multimem.ld_reduce, fp32 accumulate) and broadcasts it (multimem.st).
//
// None of them has a counterpart launch parameter that must change between
// calls: barriers return the pad to zero, so a captured graph replays.
#include <cuda_runtime.h>
#include <stdlib.h>

#include "../device/barrier.cuh"
#include "../device/multimem.cuh"
#include "../device/vec.cuh"
#include "launch.h"

namespace smr {

namespace {

constexpr int kArThreads = 512;

__global__ void barrier_test_kernel(PeerView pv, uint64_t timeout_ns, Status* st) {
  blockwise_barrier(pv.pads, flat_block_id(), pv.rank, pv.world_size, timeout_ns, st, kWhereTest);
}

// The two counting barriers behind one constructor signature.
struct EpochBar : EpochBarrier {
  __device__ __forceinline__ EpochBar(const PeerView& pv, uint32_t block_id)
      : EpochBarrier(pv.pads, block_id, pv.rank, pv.world_size) {}
};
struct NvlsBar : MulticastBarrier {
  __device__ __forceinline__ NvlsBar(const PeerView& pv, uint32_t block_id)
      : MulticastBarrier(pv.pads, pv.buffers, pv.multicast, block_id, pv.rank, pv.world_size) {}
};

// Same smoke test for the counting barriers (two rounds, so that the count written back is used).
template <class Bar>
__global__ void counting_barrier_test_kernel(PeerView pv, uint64_t timeout_ns, Status* st) {
  Bar bar(pv, flat_block_id());
  if (!bar.sync(timeout_ns, st, kWhereTest)) return;
  bar.sync(timeout_ns, st, kWhereTest);
  bar.finish();
}

// One CTA; slot = kBlockSlots + channel * WS + sender.
__global__ void channel_barrier_kernel(PeerView pv, int channel, uint64_t timeout_ns, Status* st) {
  int t = threadIdx.x;
  if (t < pv.world_size) {
    barrier_signal_wait(pv.pads, kBlockSlots + (uint32_t)channel * (uint32_t)pv.world_size,
                        pv.rank, pv.world_size, t, timeout_ns, st, (uint32_t)channel,
                        kWhereBarrierKernel);
  }
}

// One thread, one peer: the two halves of the channel barrier on their own.
__global__ void put_signal_kernel(PeerView pv, int dst, int channel, uint64_t timeout_ns, Status* st) {
  if (threadIdx.x != 0) return;
  uint32_t* slot = pv.pads[dst] + kBlockSlots + (uint32_t)channel * (uint32_t)pv.world_size + pv.rank;
  Deadline d(timeout_ns);
  while (cas_release_sys(slot, 0u, 1u) != 0u) {
    if (!d.alive()) {
      report_status(st, kTimeoutBarrierSend, pv.rank, (uint32_t)channel, dst, kWhereBarrierKernel);
      return;
    }
  }
}
__global__ void wait_signal_kernel(PeerView pv, int src, int channel, uint64_t timeout_ns, Status* st) {
  if (threadIdx.x != 0) return;
  uint32_t* slot = pv.pads[pv.rank] + kBlockSlots + (uint32_t)channel * (uint32_t)pv.world_size + src;
  Deadline d(timeout_ns);
  while (cas_acquire_sys(slot, 1u, 0u) != 1u) {
    if (!d.alive()) {
      report_status(st, kTimeoutBarrierWait, pv.rank, (uint32_t)channel, src, kWhereBarrierKernel);
      return;
    }
  }
}

__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t target, uint64_t timeout_ns,
                                 int rank, Status* st) {
  if (threadIdx.x == 0) {
    if (!wait_ge_acquire_sys(flag, target, timeout_ns)) {
      report_status(st, kTimeoutFlag, rank, blockIdx.x, 0, kWhereTest, target);
    }
  }
}

__device__ __forceinline__ Vec16 ld_16_relaxed_sys(const void* p) {
  Vec16 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// U elements (16-byte vectors) per thread and iteration: U x WS peer loads in flight per thread,
// up to 128 CTAs (measured on 2 and 4 GPUs: 32 CTAs with one element per thread leave the links
// two to four times under-used).  The peers' addresses arrive by value in the kernel's parameters,
// not through the device table: no dependent load sits in front of the barrier's first store.
// Epoch barrier (one release store per peer) on entry; the sum of an element is rank-ordered:
// same bits on every rank (symm_mem_recipes/triton_one_shot_all_reduce.py:84-89).
template <int WS, int U>
__global__ void __launch_bounds__(kArThreads)
one_shot_all_reduce_kernel(PeerPtrs ptrs, int rank, size_t offset_bytes, Vec16* __restrict__ out,
                           size_t n_vec, bool exit_barrier, bool write_back, uint64_t timeout_ns, Status* st) {
  EpochBarrier bar(ptrs.pads, blockIdx.x, rank, WS);
  if (!bar.sync(timeout_ns, st, kWhereOneShotEntry)) return;

  const Vec16* src[WS];
#pragma unroll
  for (int r = 0; r < WS; ++r)
    src[r] = reinterpret_cast<const Vec16*>(static_cast<const char*>(ptrs.buffers[r]) + offset_bytes);

  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < n_vec; k += (size_t)U * stride) {
    Vec16 v[U][WS];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = k + (size_t)u * stride;
      if (i < n_vec) {
#pragma unroll
        for (int r = 0; r < WS; ++r) v[u][r] = ld_16(src[r] + i);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = k + (size_t)u * stride;
      if (i < n_vec) {
        Vec16 acc = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int r = 0; r < WS; ++r) acc = add_bf16x8(acc, v[u][r]);
        st_16(out + i, acc);
      }
    }
  }

  if (exit_barrier) {
    // proves that every peer has finished reading this rank's buffer
    if (bar.sync(timeout_ns, st, kWhereOneShotExit) && write_back) {
      // in-place form: now the sum may replace this rank's input; every thread
      // copies back exactly the vectors it produced above
      Vec16* self = reinterpret_cast<Vec16*>(static_cast<char*>(ptrs.buffers[rank]) + offset_bytes);
      for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride)
        st_16(self + i, ld_16(out + i));
    }
  }
  bar.finish();
}

// Slice of 16-byte vectors owned by `r`: [begin, end)
__device__ __forceinline__ void slice_of(size_t n_vec, int ws, int r, size_t& begin, size_t& end) {
  size_t q = n_vec / ws, rem = n_vec % ws;
  begin = (size_t)r * q + ((size_t)r < rem ? (size_t)r : rem);
  end = begin + q + ((size_t)r < rem ? 1 : 0);
}

template <int WS, int RANK>
__global__ void __launch_bounds__(kArThreads)
two_shot_all_reduce_kernel(PeerView pv, size_t offset_bytes, size_t n_vec, uint64_t timeout_ns,
                           Status* st) {
  EpochBarrier bar(pv.pads, blockIdx.x, RANK, WS);
  if (!bar.sync(timeout_ns, st, kWhereTwoShotEntry)) return;

  Vec16* buf[WS];
#pragma unroll
  for (int r = 0; r < WS; ++r)
    buf[r] = reinterpret_cast<Vec16*>(static_cast<char*>(pv.buffers[r]) + offset_bytes);

  size_t begin, end;
  slice_of(n_vec, WS, RANK, begin, end);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = begin + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < end; i += stride) {
    Vec16 v[WS];
#pragma unroll
    for (int j = 0; j < WS; ++j) {
      const int r = (RANK + 1 + j) % WS;
      v[r] = ld_16(buf[r] + i);
    }
    Vec16 acc = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int r = 0; r < WS; ++r) acc = add_bf16x8(acc, v[r]);
    // Element i of every peer is read by this thread only (above), so the
    // in-place push cannot overtake a reader.
#pragma unroll
    for (int j = 0; j < WS; ++j) {
      const int r = (RANK + 1 + j) % WS;
      st_16(buf[r] + i, acc);
    }
  }
  // All pushes of all ranks have landed once every CTA has passed this.
  bar.sync(timeout_ns, st, kWhereTwoShotExit);
  bar.finish();
}

// Eight independent in-switch reductions in flight per thread and few CTAs (eight to sixteen: more
// measured slower at every size on 4 and 8 GPUs, and so did barriers by multimem.red).
__global__ void __launch_bounds__(kArThreads)
multimem_all_reduce_kernel(PeerView pv, size_t offset_bytes, size_t n_vec, uint64_t timeout_ns,
                           Status* st) {
  constexpr int U = 8;
  const int rank = pv.rank, ws = pv.world_size;
  EpochBar bar(pv, blockIdx.x);
  if (!bar.sync(timeout_ns, st, kWhereMultimemEntry)) return;
  Vec16* mc = reinterpret_cast<Vec16*>(static_cast<char*>(pv.multicast) + offset_bytes);
  size_t begin, end;
  slice_of(n_vec, ws, rank, begin, end);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = begin + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (U - 1) * stride < end; i += U * stride) {
    Vec16 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = multimem_ld_reduce_bf16x8(mc + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) multimem_st_16(mc + i + u * stride, v[u]);
  }
  for (; i < end; i += stride) {
    Vec16 a = multimem_ld_reduce_bf16x8(mc + i);
    multimem_st_16(mc + i, a);
  }
  bar.sync(timeout_ns, st, kWhereMultimemExit);
  bar.finish();
}

// ---------------------------------------------------------------------------
// Low-latency all-reduce for small messages: no barrier and no peer loads.
// Every rank PUSHES its input into an inbox on every rank, each 8 bytes on the
// wire carrying 4 bytes of data and a 4-byte tag (the call number), then polls
// its OWN inbox until every peer's words carry the tag and sums them in rank
// order (bf16 adds: same bits on every rank, same arithmetic as one-shot).
// One NVLink crossing instead of a barrier round trip plus a load round trip.
// A peer can be at most one call ahead (it needs this rank's data to finish a
// call), so two inbox parities suffice; the call number lives in the workspace
// and is advanced by the last CTA to finish.
//   workspace: [0] call number, [1] CTAs done; inbox at +256:
//   [2 parity][WS src][capacity_vec] x 32 bytes
// ---------------------------------------------------------------------------
template <int WS>
__global__ void __launch_bounds__(kArThreads)
ll_all_reduce_kernel(PeerView pv, const Vec16* __restrict__ in, Vec16* __restrict__ out, size_t n_vec,
                     size_t capacity_vec, uint64_t timeout_ns, Status* st) {
  const int rank = pv.rank;
  char* my_ws = static_cast<char*>(pv.buffers[rank]);
  uint32_t* header = reinterpret_cast<uint32_t*>(my_ws);
  const uint32_t tag = ld_relaxed_gpu(&header[0]) + 1u;
  const size_t parity_off = 256 + (size_t)(tag & 1u) * WS * capacity_vec * 32;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  bool ok = true;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec && ok; i += stride) {
    const Vec16 x = ld_16(in + i);
    const Vec16 p0{x.x, tag, x.y, tag}, p1{x.z, tag, x.w, tag};
    const size_t slot = parity_off + ((size_t)rank * capacity_vec + i) * 32;
#pragma unroll
    for (int j = 1; j <= WS; ++j) {             // own inbox last
      const int peer = (rank + j) % WS;
      char* dst = static_cast<char*>(pv.buffers[peer]) + slot;
      st_16(dst, p0);
      st_16(dst + 16, p1);
    }
    Vec16 a[WS], b[WS];
    uint32_t pending = (1u << WS) - 1u;
    Deadline d(timeout_ns);
    while (pending != 0u) {
#pragma unroll
      for (int r = 0; r < WS; ++r) {
        if (pending & (1u << r)) {
          const char* src = my_ws + parity_off + ((size_t)r * capacity_vec + i) * 32;
          a[r] = ld_16_relaxed_sys(src);
          b[r] = ld_16_relaxed_sys(src + 16);
        }
      }
#pragma unroll
      for (int r = 0; r < WS; ++r)
        if ((pending & (1u << r)) && a[r].y == tag && a[r].w == tag && b[r].y == tag && b[r].w == tag)
          pending &= ~(1u << r);
      if (pending != 0u && !d.alive()) {
        report_status(st, kTimeoutFlag, rank, blockIdx.x, __ffs(pending) - 1, kWhereOneShotEntry, tag);
        ok = false;
        break;
      }
    }
    if (!ok) break;
    Vec16 acc = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int r = 0; r < WS; ++r) acc = add_bf16x8(acc, Vec16{a[r].x, a[r].z, b[r].x, b[r].z});
    st_16(out + i, acc);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t done = atomicAdd(&header[1], 1u);
    if (done == gridDim.x - 1) {
      header[1] = 0u;
      __threadfence();
      st_release_gpu(&header[0], tag);
    }
  }
}

int blocks_for(size_t n_vec, int max_blocks) {
  size_t b = (n_vec + kArThreads - 1) / kArThreads;
  if (b < 1) b = 1;
  if (b > (size_t)max_blocks) b = max_blocks;
  return (int)b;
}

int last_error() { return (int)cudaGetLastError(); }

}  // namespace

int launch_barrier_test(const PeerView& pv, int num_blocks, int threads, uint64_t timeout_ns,
                        Status* status, cudaStream_t stream, int kind) {
  if (num_blocks < 1 || (uint32_t)num_blocks * pv.world_size > kBlockSlots) return cudaErrorInvalidValue;
  if (threads < pv.world_size) return cudaErrorInvalidValue;
  if (kind != 0 && (uint32_t)num_blocks > kArMaxBlocks) return cudaErrorInvalidValue;
  switch (kind) {
    case 0: barrier_test_kernel<<<num_blocks, threads, 0, stream>>>(pv, timeout_ns, status); break;
    case 1: counting_barrier_test_kernel<EpochBar><<<num_blocks, threads, 0, stream>>>(pv, timeout_ns, status); break;
    case 2:
      if (pv.multicast == nullptr) return cudaErrorNotSupported;
      counting_barrier_test_kernel<NvlsBar><<<num_blocks, threads, 0, stream>>>(pv, timeout_ns, status);
      break;
    default: return cudaErrorInvalidValue;
  }
  return last_error();
}

int launch_channel_barrier(const PeerView& pv, int channel, uint64_t timeout_ns, Status* status,
                           cudaStream_t stream) {
  if (channel < 0 || (uint32_t)(channel + 1) * pv.world_size > kChannelSlots) return cudaErrorInvalidValue;
  channel_barrier_kernel<<<1, 32, 0, stream>>>(pv, channel, timeout_ns, status);
  return last_error();
}

int launch_put_signal(const PeerView& pv, int dst, int channel, uint64_t timeout_ns, Status* status,
                      cudaStream_t stream) {
  if (dst < 0 || dst >= pv.world_size || channel < 0 || (uint32_t)(channel + 1) * pv.world_size > kChannelSlots)
    return cudaErrorInvalidValue;
  put_signal_kernel<<<1, 32, 0, stream>>>(pv, dst, channel, timeout_ns, status);
  return last_error();
}

int launch_wait_signal(const PeerView& pv, int src, int channel, uint64_t timeout_ns, Status* status,
                       cudaStream_t stream) {
  if (src < 0 || src >= pv.world_size || channel < 0 || (uint32_t)(channel + 1) * pv.world_size > kChannelSlots)
    return cudaErrorInvalidValue;
  wait_signal_kernel<<<1, 32, 0, stream>>>(pv, src, channel, timeout_ns, status);
  return last_error();
}

int launch_wait_flag(const uint32_t* flag, uint32_t target, uint64_t timeout_ns, int rank,
                     Status* status, cudaStream_t stream) {
  wait_flag_kernel<<<1, 32, 0, stream>>>(flag, target, timeout_ns, rank, status);
  return last_error();
}

#define SMR_RANK_CASE(r, ...) case r: { constexpr int RANK = r; __VA_ARGS__; break; }
#define SMR_DISPATCH_WS_RANK(ws, rank, ...)                                                     \
  switch (ws) {                                                                                 \
    case 1: { constexpr int WS = 1; switch (rank) { SMR_RANK_CASE(0, __VA_ARGS__) default: return cudaErrorInvalidValue; } break; } \
    case 2: { constexpr int WS = 2; switch (rank) { SMR_RANK_CASE(0, __VA_ARGS__) SMR_RANK_CASE(1, __VA_ARGS__) default: return cudaErrorInvalidValue; } break; } \
    case 4: { constexpr int WS = 4; switch (rank) { SMR_RANK_CASE(0, __VA_ARGS__) SMR_RANK_CASE(1, __VA_ARGS__) SMR_RANK_CASE(2, __VA_ARGS__) SMR_RANK_CASE(3, __VA_ARGS__) default: return cudaErrorInvalidValue; } break; } \
    case 8: { constexpr int WS = 8; switch (rank) { SMR_RANK_CASE(0, __VA_ARGS__) SMR_RANK_CASE(1, __VA_ARGS__) SMR_RANK_CASE(2, __VA_ARGS__) SMR_RANK_CASE(3, __VA_ARGS__) SMR_RANK_CASE(4, __VA_ARGS__) SMR_RANK_CASE(5, __VA_ARGS__) SMR_RANK_CASE(6, __VA_ARGS__) SMR_RANK_CASE(7, __VA_ARGS__) default: return cudaErrorInvalidValue; } break; } \
    default: return cudaErrorInvalidValue;                                                      \
  }

int launch_one_shot_all_reduce(const PeerView& pv, const PeerPtrs& ptrs, size_t offset_bytes, void* out,
                               size_t numel, int max_blocks, bool exit_barrier, bool write_back,
                               uint64_t timeout_ns, Status* status, cudaStream_t stream) {
  if (write_back && !exit_barrier) return cudaErrorInvalidValue;
  if (numel % 8 != 0 || offset_bytes % 16 != 0) return cudaErrorInvalidValue;
  size_t n_vec = numel / 8;
  if (max_blocks < 1) max_blocks = 1;
  if ((uint32_t)max_blocks > kArMaxBlocks) max_blocks = (int)kArMaxBlocks;     // one epoch-barrier group per CTA
  // Two vectors per thread once the message is worth it (U x WS vectors live in registers: at most 16),
  // and always from four ranks on: the one-vector instantiation for eight ranks compiles to 38 registers, too
  // few to hold eight loaded vectors, i.e. its peer loads are consumed one after the other (measured on eight
  // ranks: 15.7 µs at 64 KiB with one vector per thread, 11.3 µs at 128 KiB with two).
  const int unroll = (pv.world_size >= 4 || n_vec >= (size_t)2 * kArThreads * 8) ? 2 : 1;
  size_t per_block = (size_t)kArThreads * unroll;
  size_t want = (n_vec + per_block - 1) / per_block;
  int blocks = (int)(want < 1 ? 1 : (want > (size_t)max_blocks ? (size_t)max_blocks : want));
#define SMR_ONE_SHOT(WS_)                                                                                    \
  if (unroll == 2)                                                                                           \
    one_shot_all_reduce_kernel<WS_, 2><<<blocks, kArThreads, 0, stream>>>(                                   \
        ptrs, pv.rank, offset_bytes, static_cast<Vec16*>(out), n_vec, exit_barrier, write_back, timeout_ns, status); \
  else                                                                                                       \
    one_shot_all_reduce_kernel<WS_, 1><<<blocks, kArThreads, 0, stream>>>(                                   \
        ptrs, pv.rank, offset_bytes, static_cast<Vec16*>(out), n_vec, exit_barrier, write_back, timeout_ns, status)
  switch (pv.world_size) {
    case 1: SMR_ONE_SHOT(1); break;
    case 2: SMR_ONE_SHOT(2); break;
    case 4: SMR_ONE_SHOT(4); break;
    case 8: SMR_ONE_SHOT(8); break;
    default: return cudaErrorInvalidValue;
  }
#undef SMR_ONE_SHOT
  return last_error();
}

size_t ll_all_reduce_workspace_bytes(size_t max_numel, int world_size) {
  return 256 + (size_t)2 * world_size * (max_numel / 8) * 32;
}

int launch_ll_all_reduce(const PeerView& pv, const void* in, void* out, size_t numel, size_t capacity_numel,
                         int max_blocks, uint64_t timeout_ns, Status* status, cudaStream_t stream) {
  if (numel % 8 != 0 || numel > capacity_numel || capacity_numel % 8 != 0) return cudaErrorInvalidValue;
  size_t n_vec = numel / 8;
  // small CTAs on many SMs: one SM sustains only ~30 GB/s of NVLink stores
  constexpr int kLlThreads = 128;
  size_t want = (n_vec + kLlThreads - 1) / kLlThreads;
  int blocks = (int)(want < 1 ? 1 : (want > (size_t)max_blocks ? (size_t)max_blocks : want));
#define SMR_LL_CASE(n) case n: ll_all_reduce_kernel<n><<<blocks, kLlThreads, 0, stream>>>( \
      pv, static_cast<const Vec16*>(in), static_cast<Vec16*>(out), n_vec, capacity_numel / 8, timeout_ns, status); break;
  switch (pv.world_size) {
    SMR_LL_CASE(1) SMR_LL_CASE(2) SMR_LL_CASE(4) SMR_LL_CASE(8)
    default: return cudaErrorInvalidValue;
  }
#undef SMR_LL_CASE
  return last_error();
}

int launch_two_shot_all_reduce(const PeerView& pv, size_t offset_bytes, size_t numel,
                               int max_blocks, uint64_t timeout_ns, Status* status,
                               cudaStream_t stream) {
  if (numel % 8 != 0 || offset_bytes % 16 != 0) return cudaErrorInvalidValue;
  size_t n_vec = numel / 8;
  if ((uint32_t)max_blocks > kArMaxBlocks) max_blocks = (int)kArMaxBlocks;
  int blocks = blocks_for((n_vec + pv.world_size - 1) / pv.world_size, max_blocks);
  SMR_DISPATCH_WS_RANK(pv.world_size, pv.rank,
                       (two_shot_all_reduce_kernel<WS, RANK><<<blocks, kArThreads, 0, stream>>>(
                           pv, offset_bytes, n_vec, timeout_ns, status)));
  return last_error();
}

int launch_multimem_all_reduce(const PeerView& pv, size_t offset_bytes, size_t numel,
                               int max_blocks, uint64_t timeout_ns, Status* status,
                               cudaStream_t stream) {
  if (numel % 8 != 0 || offset_bytes % 16 != 0) return cudaErrorInvalidValue;
  if (pv.multicast == nullptr) return cudaErrorNotSupported;
  size_t n_vec = numel / 8;
  if (max_blocks < 1) max_blocks = 1;
  if ((uint32_t)max_blocks > kArMaxBlocks) max_blocks = (int)kArMaxBlocks;
  int blocks = blocks_for((n_vec + pv.world_size - 1) / pv.world_size, max_blocks);
  multimem_all_reduce_kernel<<<blocks, kArThreads, 0, stream>>>(pv, offset_bytes, n_vec, timeout_ns, status);
  return last_error();
}

}  // namespace smr
