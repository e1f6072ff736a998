// Fused GEMM + reduce-scatter for sm_100a (row-parallel linear layer, prefill):
//     out_r[M/WS, N] = sum over ranks s of ( A_s[M, K_s] * B_s[N, K_s]^T )[rows of rank r]
// No upstream counterpart (the upstream package has the all-gather half only).
//
//  * The GEMM is the tcgen05 / TMEM pipeline of ag_matmul_sm100.cu (TMA
//    producer warp, MMA warp, four epilogue warps, two TMEM accumulators).
//  * Tiles are visited by destination rank: rank+1 first, ..., own rows last,
//    so the links are busy from the first tile and nothing waits on the wire
//    at the end.
//  * Epilogue: accumulator -> bf16 -> a shared-memory strip of [128 rows x 64
//    columns] (16 KB, 16-byte chunks XOR-swizzled by row so that the writes do
//    not collide on banks) -> ONE bulk copy (cp.async.bulk, shared -> global)
//    of 16 contiguous KB into the DESTINATION rank's inbox.  The inbox is
//    internal scratch, so it is laid out strip by strip,
//    [src][row block][N tile][strip][16 KB], exactly as the strips sit in
//    shared memory: every store is one long contiguous write over NVLink (a
//    row-major inbox would turn it into 128-byte fragments 16 KB apart, which
//    measured 400 GB/s).  Two strips alternate, so the next one is converted
//    while the previous one is on the wire.  A tile's arrival counter on the
//    destination gets +1 (red.release.sys) once the tile's stores have
//    completed, which is checked one tile later so the epilogue never waits
//    for the wire.
//  * Reduce: after its GEMM tiles every CTA takes output tiles of its own rank,
//    waits (bounded) until WS partials have arrived, sums them in rank order in
//    fp32 and writes bf16.  All ranks thus produce identical bits.
//  * An entry barrier over the signal pad proves that every rank has finished
//    reducing the previous call before its inbox is overwritten.  Counters
//    count calls (epoch word in the pad), so nothing is reset between calls.
#include "matmul_rs_common.cuh"

namespace smr {

using namespace rs;

namespace {

template <int kStages, int kNStrips>
struct RsSmem {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = kBN * kBK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kRingBytes = kStageBytes * kStages;
  static constexpr uint32_t kStripOffset = kRingBytes;
  static constexpr uint32_t kStripBytes = kNStrips * kStripBytesOne;   // strips in flight on the wire
  static constexpr uint32_t kBarOffset = kStripOffset + kStripBytes;
  static constexpr uint32_t kNumBars = 2 * kStages + 4;
  static constexpr uint32_t kMiscOffset = kBarOffset + 8 * kNumBars;
  static constexpr uint32_t kTotal = kMiscOffset + 16 + 1024;
};
static_assert(RsSmem<4, 2>::kTotal <= 232448 && RsSmem<3, 5>::kTotal <= 232448, "shared memory limit exceeded");

// tile index -> destination rank, 128-row block inside the destination, N tile
__device__ __forceinline__ void tile_coords(const RsParams& p, int t, int& dest, int& mb, int& ni) {
  const int per_dest = p.blocks_per_rank * p.n_tiles_n;
  int step = t / per_dest, rem = t - step * per_dest;
  dest = p.rank + 1 + step;
  if (dest >= p.world_size) dest -= p.world_size;
  mb = rem / p.n_tiles_n;
  ni = rem - mb * p.n_tiles_n;
}

// kStages: depth of the operand ring; kNStrips: epilogue strips that may be on the wire at once.
// <4, 2> is the default; <3, 5> trades a stage for three more strips in flight (short-K shapes,
// where the wire, not the main loop, is the limit).
// kThreadStores: a strip leaves shared memory by coalesced 16-byte loads and stores of the 128
// epilogue threads (512 contiguous bytes per warp instruction) instead of one bulk store by one
// thread.  Stores issued by threads are not capped at kNStrips per SM on the wire, the buffer is
// free as soon as it has been read, and the tile's counter is bumped right after its last strip.
template <int kStages, int kNStrips, bool kAllReduce = false, bool kThreadStores = false>
__global__ void __launch_bounds__(kThreads, 1)
matmul_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const RsParams p) {
  using Smem = RsSmem<kStages, kNStrips>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* strip = smem + Smem::kStripOffset;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBarOffset);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Smem::kMiscOffset);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* header = p.local_pad + kFlagSlotsBase;        // [0] epoch, [1] CTAs done
  const uint32_t epoch = ld_relaxed_gpu(&header[0]) + 1u;
  const uint32_t target = epoch * (uint32_t)p.world_size;
  uint32_t* my_counters = p.local_pad + kFlagSlotsBase + 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[blockIdx.x * 4 + 0] = globaltimer_ns();
  // every rank has entered this call: its reduce of the previous call is done
  bool entered = blockwise_barrier(p.pads, 1024u + blockIdx.x, p.rank, p.world_size, p.timeout_ns,
                                   p.status, kWhereRsEntry);
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[blockIdx.x * 4 + 1] = globaltimer_ns();
  tcgen05_fence_before_thread_sync();
  __syncthreads();
  tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.world_size * p.blocks_per_rank * p.n_tiles_n;
  const int k_blocks = (p.K + kBK - 1) / kBK;
  const int rows_per_rank = p.blocks_per_rank * kBM;
  bool failed = !entered;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
        int dest, mb, ni;
        tile_coords(p, t, dest, mb, ni);
        const int row0 = dest * rows_per_rank + mb * kBM;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.timeout_ns)) {
            report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, stage, kWhereGemmEmpty);
            failed = true;
            break;
          }
          uint8_t* sa = smem + (size_t)stage * Smem::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], Smem::kStageBytes);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * kBK, row0);
          tma_load_2d(sa + Smem::kABytes, &tmap_b, &full_bar[stage], kb * kBK, ni * kBN);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(kBM, kBN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.timeout_ns)) {
          report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, acc, kWhereGemmTmemEmpty);
          failed = true;
          break;
        }
        tcgen05_fence_after_thread_sync();
        const uint32_t d_tmem = tmem_base + acc * 256u;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.timeout_ns)) {
            report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, stage, kWhereGemmFull);
            failed = true;
            break;
          }
          tcgen05_fence_after_thread_sync();
          const uint32_t sa = smem_u32(smem + (size_t)stage * Smem::kStageBytes);
          const uint64_t da = umma_smem_desc_sw128(sa);
          const uint64_t db = umma_smem_desc_sw128(sa + Smem::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_bf16_ss(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                         (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> bf16 strip -> TMA store into the destination ----------------
    const int quarter = warp & 3;
    const int etid = (int)threadIdx.x - 64;
    const int r = quarter * 32 + lane;                  // row of the tile owned by this thread
    uint32_t acc = 0, acc_phase = 0, strip_ctr = 0;
    uint32_t* prev_counter = nullptr;                   // tile whose stores are issued but not yet signalled
    for (int t = blockIdx.x; t < total_tiles && !failed; t += gridDim.x) {
      int dest, mb, ni;
      tile_coords(p, t, dest, mb, ni);
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.timeout_ns)) {
        if (lane == 0)
          report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, acc, kWhereGemmTmemFull);
        failed = true;
        break;
      }
      tcgen05_fence_after_thread_sync();
      const uint32_t taddr = tmem_base + acc * 256u + ((uint32_t)(quarter * 32) << 16);
      int strips = 0;
#pragma unroll 1
      for (int sidx = 0; sidx < kBN / kStripCols; ++sidx) {
        const int col0 = ni * kBN + sidx * kStripCols;
        if (col0 >= p.N) break;                          // uniform over the CTA
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(taddr + (uint32_t)(sidx * kStripCols), v0);
        tmem_ld_32x32b_x32(taddr + (uint32_t)(sidx * kStripCols + 32), v1);
        tmem_ld_wait();
        // the store issued two strips ago has finished reading the buffer we are about to fill
        if constexpr (!kThreadStores) {
          if (etid == 0) bulk_wait_group_read<kNStrips - 1>();
        }
        epilogue_sync();
        uint8_t* buf = strip + (size_t)(strip_ctr % (uint32_t)kNStrips) * kStripBytesOne;
        strip_row_to_smem(buf, r, v0, v1);
        if constexpr (kThreadStores) {
          epilogue_sync();                               // the strip is complete in shared memory
          char* dst = static_cast<char*>(p.buffers[dest]) + p.inbox_offset +
                      strip_offset(p.rank, mb, ni, sidx, p.blocks_per_rank, p.n_tiles_n);
          strip_copy_out(dst, buf, etid);
        } else {
        fence_proxy_async();                             // generic writes to smem, async-proxy read
        epilogue_sync();
        if (etid == 0) {
          char* dst = static_cast<char*>(p.buffers[dest]) + p.inbox_offset +
                      strip_offset(p.rank, mb, ni, sidx, p.blocks_per_rank, p.n_tiles_n);
          bulk_store(dst, buf, kStripBytesOne);
          bulk_commit_group();
        }
        }
        ++strip_ctr;
        ++strips;
      }
      // the accumulator has been read: hand it back
      tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if constexpr (kThreadStores) {
        epilogue_sync();                                 // every thread has issued its stores of this tile
        if (etid == 0 && strips > 0)
          red_add_release_sys(p.pads[dest] + kFlagSlotsBase + 2 + mb * p.n_tiles_n + ni, 1u);
      } else if (etid == 0) {
        if (prev_counter != nullptr) {
          // everything older than this tile's groups has completed
          if (strips == 4) bulk_wait_group<4>();
          else bulk_wait_group<0>();
          fence_proxy_async();
          red_add_release_sys(prev_counter, 1u);
        }
        prev_counter = p.pads[dest] + kFlagSlotsBase + 2 + mb * p.n_tiles_n + ni;
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (etid == 0) {
      bulk_wait_group<0>();
      if (prev_counter != nullptr && !failed) {
        fence_proxy_async();
        red_add_release_sys(prev_counter, 1u);
      }
    }
  }

  // ---------------- GEMM teardown ----------------
  if (__any_sync(0xffffffffu, failed)) {
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  tcgen05_fence_before_thread_sync();
  failed = __syncthreads_or(failed) != 0;
  tcgen05_fence_after_thread_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[blockIdx.x * 4 + 2] = globaltimer_ns();

  // ---------------- reduce the tiles of this rank ----------------
  if (!failed) {
    const int my_tiles = p.blocks_per_rank * p.n_tiles_n;
    const char* inbox = static_cast<const char*>(p.buffers[p.rank]) + p.inbox_offset;
    for (int t = blockIdx.x; t < my_tiles; t += gridDim.x) {
      const int mb = t / p.n_tiles_n, ni = t - mb * p.n_tiles_n;
      bool ok = true;
      if (threadIdx.x == 0 && !wait_ge_acquire_sys(&my_counters[t], target, p.timeout_ns)) {
        report_status(p.status, kTimeoutFlag, p.rank, blockIdx.x, t, kWhereRsArrive, target);
        ok = false;
      }
      if (!__syncthreads_and(ok)) break;
      switch (p.world_size) {
        case 2: reduce_tile<2, kAllReduce>(p, inbox, mb, ni); break;
        case 4: reduce_tile<4, kAllReduce>(p, inbox, mb, ni); break;
        case 8: reduce_tile<8, kAllReduce>(p, inbox, mb, ni); break;
        default: reduce_tile<0, kAllReduce>(p, inbox, mb, ni); break;
      }
    }
  }

  if constexpr (kAllReduce) {
    // CTA i of every rank has finished broadcasting its rows: when all CTAs of this rank have passed
    // here, the whole [M, N] output of this rank is complete
    blockwise_barrier(p.pads, 1024u + blockIdx.x, p.rank, p.world_size, p.timeout_ns, p.status, kWhereRsArrive);
  }

  // ---------------- the last CTA to finish publishes this call's number ----------------
  __syncthreads();
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[blockIdx.x * 4 + 3] = globaltimer_ns();
  if (threadIdx.x == 0) {
    uint32_t done = atomicAdd(&header[1], 1u);
    if (done == gridDim.x - 1) {
      header[1] = 0u;
      __threadfence();
      st_release_gpu(&header[0], epoch);
    }
  }
}

}  // namespace

size_t matmul_rs_workspace_bytes(int M, int N) {
  // strip-major inbox: every [128 x 256] tile occupies four 16 KB strips, also at the N edge
  return (size_t)((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN) * kStripsPerTile * kStripBytesOne;
}

int launch_matmul_reduce_scatter(const MatmulRsArgs& a, cudaStream_t stream) {
  if (a.cta_pair) return launch_matmul_reduce_scatter_2cta(a, stream);
  const int ws = a.pv.world_size;
  if (a.M <= 0 || a.N % 8 != 0 || a.K % 8 != 0 || a.M % (ws * kBM) != 0) return cudaErrorInvalidValue;
  RsParams p{};
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.rank = a.pv.rank; p.world_size = ws;
  p.blocks_per_rank = a.M / ws / kBM;
  p.n_tiles_n = (a.N + kBN - 1) / kBN;
  if ((uint32_t)(p.blocks_per_rank * p.n_tiles_n) + 2u > kFusedFlagSlots) return cudaErrorInvalidValue;
  p.buffers = a.pv.buffers;
  p.inbox_offset = a.inbox_offset;
  p.pads = a.pv.pads;
  p.local_pad = a.local_pad;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.timeout_ns = a.timeout_ns;
  p.status = a.status;
  p.trace = a.trace;
  if (a.all_reduce) {
    if (a.ar_peers == nullptr || a.deep_strips || a.ar_offset % 16 != 0) return cudaErrorInvalidValue;
    p.ar_peers = a.ar_peers;
    p.ar_mc = a.ar_mc;
    p.ar_offset = a.ar_offset;
  } else if (a.out == nullptr) {
    return cudaErrorInvalidValue;
  }
  CUtensorMap ta, tb;
  if (make_tmap(&ta, a.a, (uint64_t)a.M, (uint64_t)a.K, kBM)) return cudaErrorInvalidValue;
  if (make_tmap(&tb, a.b, (uint64_t)a.N, (uint64_t)a.K, kBN)) return cudaErrorInvalidValue;
  int total_tiles = ws * p.blocks_per_rank * p.n_tiles_n;
  int grid = a.num_sms < total_tiles ? a.num_sms : total_tiles;
  if (grid < 1 || (uint32_t)(1024 + grid) * (uint32_t)ws > kBlockSlots) return cudaErrorInvalidValue;
  if (a.deep_strips) {
    auto kern = matmul_rs_kernel<3, 5>;
    constexpr int smem = (int)RsSmem<3, 5>::kTotal;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    kern<<<grid, kThreads, smem, stream>>>(ta, tb, p);
  } else if (a.thread_stores && !a.all_reduce) {
    auto kern = matmul_rs_kernel<4, 2, false, true>;
    constexpr int smem = (int)RsSmem<4, 2>::kTotal;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    kern<<<grid, kThreads, smem, stream>>>(ta, tb, p);
  } else if (a.all_reduce) {
    auto kern = matmul_rs_kernel<4, 2, true>;
    constexpr int smem = (int)RsSmem<4, 2>::kTotal;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    kern<<<grid, kThreads, smem, stream>>>(ta, tb, p);
  } else {
    auto kern = matmul_rs_kernel<4, 2>;
    constexpr int smem = (int)RsSmem<4, 2>::kTotal;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    kern<<<grid, kThreads, smem, stream>>>(ta, tb, p);
  }
  return (int)cudaGetLastError();
}

}  // namespace smr
