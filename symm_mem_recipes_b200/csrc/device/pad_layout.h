// Layout of the signal pad that sits behind every symmetric allocation.
//
// The pad is zero-filled at allocation and every protocol in the library
// returns it to all-zero (the property that makes the upstream barrier usable
// inside CUDA graphs, symm_mem_recipes/triton_barrier.py:57-65).
//
//   [0, kBlockSlots)                      blockwise-barrier slots, u32,
//                                         slot = block_id * world_size + sender
//   [kBlockSlots, +kChannelSlots)         host-launched barrier channels,
//                                         slot = channel * world_size + sender
//   [kFlagSlotsBase, +kFusedFlagSlots)    call counters and per-tile arrival
//                                         counters of the fused GEMM kernels
//   [kArFlagBase, end)                    epoch barrier of the all-reduce
//                                         kernels: 32 slots per block id,
//                                         [0] = this rank's barrier count,
//                                         [16 + s] = last count announced by rank s
// The first two regions return to all-zero after every operation; the last two
// hold monotonically increasing counters (no reset, no host-side state).
#pragma once
#include <stdint.h>

namespace smr {
constexpr uint32_t kSignalPadBytes = 128u * 1024u;
constexpr uint32_t kSignalPadSlots = kSignalPadBytes / 4u;        // 32768 u32
constexpr uint32_t kBlockSlots = 16384u;                          // 2048 blocks x 8 ranks
constexpr uint32_t kChannelSlots = 2048u;                         // 128 channels x 16 ranks
constexpr uint32_t kFlagSlotsBase = kBlockSlots + kChannelSlots;  // 18432
constexpr uint32_t kFlagSlots = kSignalPadSlots - kFlagSlotsBase; // 14336
constexpr uint32_t kFusedFlagSlots = 8192u;
constexpr uint32_t kArFlagBase = kFlagSlotsBase + kFusedFlagSlots;          // 26624
constexpr uint32_t kArFlagStride = 32u;
constexpr uint32_t kArMaxBlocks = (kSignalPadSlots - kArFlagBase) / kArFlagStride;   // 192
constexpr int kMaxWorldSize = 16;
}  // namespace smr
