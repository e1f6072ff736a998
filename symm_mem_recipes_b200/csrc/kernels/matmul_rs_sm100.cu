// Fused GEMM + reduce-scatter for sm_100a (row-parallel linear layer, prefill):
//     out_r[M/WS, N] = sum over ranks s of ( A_s[M, K_s] * B_s[N, K_s]^T )[rows of rank r]
// No upstream counterpart (the upstream package has the all-gather half only).
//
//  * Main loop on CTA pairs (tcgen05 `cta_group::2`), as in ag_matmul_2cta_sm100.cu: two CTAs
//    on neighbouring SMs multiply one [256 x 256] tile, each staging its own 128 rows of A and
//    its own half of the B tile (ordinary TMA loads, no multicast qualifier); the leader's MMA
//    thread issues one MMA per 16 elements of K and each CTA finds its 128 accumulator rows in
//    its own TMEM.  Six 32 KB stages.
//  * Row blocks are visited by destination rank: rank+1 first, ..., own rows last, so the links
//    are busy from the first tile and nothing waits on the wire at the end.  The two row blocks
//    of a pair are consecutive entries of that list, so they may belong to different
//    destinations; each CTA converts, ships and signals its own block.  With an odd number of
//    row blocks the last pair's second CTA multiplies zero rows (out-of-range TMA coordinates
//    read as zero) and ships nothing.
//  * Epilogue: accumulator -> bf16 -> a shared-memory strip of [128 rows x 64 columns] (16 KB,
//    16-byte chunks XOR-swizzled by row so that the writes do not collide on banks) -> the
//    128 epilogue threads copy it with coalesced 16-byte stores (512 contiguous bytes per warp
//    instruction) into the DESTINATION rank's inbox.  The inbox is internal scratch, so it is
//    laid out strip by strip, [src][row block][N tile][strip][16 KB], exactly as the strips sit
//    in shared memory: every strip is one contiguous 16 KB write over NVLink.  Two strip
//    buffers alternate.  A tile's arrival counter on the destination gets +1 (red.release.sys)
//    after its last strip.  Measured on 4 GPUs against the other forms this kernel has had
//    (one CTA per tile; strips leaving by bulk copies, two to five in flight): 1.21x cuBLAS +
//    NCCL at the down-projection shape where those reached 0.82x to 1.17x, and within 3 % of
//    the best of them at the o-projection shape.
//  * Reduce: the tiles of the rank's OWN rows come last in the visiting order, when the peers'
//    partials for them have long arrived.  Their epilogue does not ship the accumulator: it waits
//    (bounded) for the tile's WS - 1 arrivals, reads the peers' bf16 partials out of the inbox
//    (row by row, 28 independent 16-byte loads in flight per thread), adds them and its own
//    accumulator (rounded to bf16 as if it had travelled) in rank order in fp32, and writes the
//    final bf16 rows.  There is no separate reduction pass and the own partial never touches
//    memory.
//  * An entry barrier over the signal pad proves that every rank has finished reducing the
//    previous call before its inbox is overwritten.  Counters count calls (epoch word in the
//    pad), so nothing is reset between calls.
//  * All-reduce form (kAllReduce): each rank reduces its rows and broadcasts them into a
//    symmetric [M, N] output on every rank; an exit barrier proves that all rows have landed.
//
// Barriers inside the pair: full[] on the leader, empty[] / tmem_full[] by multicast commit,
// tmem_empty[] on the leader with 8 arrivals.
#include "../device/tcgen05_pair.cuh"
#include "matmul_rs_common.cuh"
#include "residency.h"

namespace smr {

using namespace rs;

namespace {

constexpr int kStages = 6;
constexpr int kNStrips = 2;

struct PairRsSmem {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = (kBN / 2) * kBK * 2;       // this CTA's half of the B tile
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kRingBytes = kStageBytes * kStages;
  static constexpr uint32_t kStripOffset = kRingBytes;
  static constexpr uint32_t kStripBytes = kNStrips * kStripBytesOne;
  static constexpr uint32_t kBarOffset = kStripOffset + kStripBytes;
  static constexpr uint32_t kNumBars = 2 * kStages + 4;
  static constexpr uint32_t kMiscOffset = kBarOffset + 8 * kNumBars;
  static constexpr uint32_t kTotal = kMiscOffset + 16 + 1024;
  static_assert(kStageBytes % 1024 == 0, "stage bases must stay 1024-byte aligned");
};
static_assert(PairRsSmem::kTotal <= 232448, "shared memory limit exceeded");

template <bool kAllReduce = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
matmul_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const RsParams p) {
  using L = PairRsSmem;
  extern __shared__ uint8_t smem_raw[];
  // same offset in both CTAs: the dynamic window starts at the same shared address
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* strip = smem + L::kStripOffset;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOffset);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  uint32_t* header = p.local_pad + kFlagSlotsBase;        // [0] epoch, [1] CTAs done
  const uint32_t epoch = ld_relaxed_gpu(&header[0]) + 1u;
  const uint32_t target = epoch * (uint32_t)(p.world_size - 1);   // arrivals from the peers, per call
  uint32_t* my_counters = p.local_pad + kFlagSlotsBase + 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 8);   // 4 epilogue warps x 2 CTAs (used in the leader)
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[blockIdx.x * 4 + 0] = globaltimer_ns();
  // every rank has entered this call: its reduce of the previous call is done
  bool entered = blockwise_barrier(p.pads, 1024u + blockIdx.x, p.rank, p.world_size, p.timeout_ns,
                                   p.status, kWhereRsEntry);
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[blockIdx.x * 4 + 1] = globaltimer_ns();
  tcgen05_fence_before_thread_sync();
  __syncthreads();
  cluster_sync_all();                 // barriers of both CTAs initialised, TMEM allocated
  tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int pair = (int)blockIdx.x >> 1;
  const int n_pairs = (int)gridDim.x >> 1;
  const int n_rb = p.world_size * p.blocks_per_rank;       // 128-row blocks over all destinations
  const int n_pair_rows = (n_rb + 1) >> 1;
  const int total_tiles = n_pair_rows * p.n_tiles_n;
  const int k_blocks = (p.K + kBK - 1) / kBK;
  const int rows_per_rank = p.blocks_per_rank * kBM;
  bool failed = !entered;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int t = pair; t < total_tiles && !failed; t += n_pairs) {
        int pr, ni;
        panel_tile_coords(p.n_tiles_n, p.panel_w, n_pair_rows, t, pr, ni);
        const int rb = 2 * pr + (int)cta_rank;
        int row0 = p.M;                                    // past the end: reads as zero
        if (rb < n_rb) {
          int dest, mb;
          row_block_coords(p, rb, dest, mb);
          row0 = dest * rows_per_rank + mb * kBM;
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.timeout_ns)) {
            report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, stage, kWhereGemmEmpty);
            failed = true;
            break;
          }
          uint8_t* sa = smem + (size_t)stage * L::kStageBytes;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2u * L::kStageBytes);
          const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, &tmap_a, full_leader, kb * kBK, row0);
          tma_load_2d_pair(sa + L::kABytes, &tmap_b, full_leader, kb * kBK, ni * kBN + (int)cta_rank * (kBN / 2));
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(2 * kBM, kBN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      for (int t = pair; t < total_tiles && !failed; t += n_pairs) {
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
          const uint32_t sa = smem_u32(smem + (size_t)stage * L::kStageBytes);
          const uint64_t da = umma_smem_desc_sw128(sa);
          const uint64_t db = umma_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_bf16_ss_pair(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                              (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit_pair(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------- epilogue (warps 2..5 of both CTAs): TMEM -> bf16 strip -> coalesced stores into the destination -------
    const int quarter = warp & 3;
    const int etid = (int)threadIdx.x - 64;
    const int r = quarter * 32 + lane;                  // row of this CTA's block owned by this thread
    uint32_t acc = 0, acc_phase = 0, strip_ctr = 0;
    __shared__ int own_ok;
    for (int t = pair; t < total_tiles && !failed; t += n_pairs) {
      int pr, ni;
      panel_tile_coords(p.n_tiles_n, p.panel_w, n_pair_rows, t, pr, ni);
      const int rb = 2 * pr + (int)cta_rank;
      const bool valid = rb < n_rb;
      int dest = 0, mb = 0;
      if (valid) row_block_coords(p, rb, dest, mb);
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.timeout_ns)) {
        if (lane == 0)
          report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, acc, kWhereGemmTmemFull);
        failed = true;
        break;
      }
      tcgen05_fence_after_thread_sync();
      const uint32_t taddr = tmem_base + acc * 256u + ((uint32_t)(quarter * 32) << 16);
      int strips = 0;
      if (valid && dest == p.rank) {
        // ---- own rows: every peer's partial of this tile is (about to be) in the inbox ----
        if (etid == 0) {
          own_ok = 1;
          if (!wait_reached_acquire_sys(&my_counters[mb * p.n_tiles_n + ni], target, p.timeout_ns)) {
            report_status(p.status, kTimeoutFlag, p.rank, blockIdx.x, mb * p.n_tiles_n + ni, kWhereRsArrive, target);
            own_ok = 0;
          }
        }
        epilogue_sync();
        if (!own_ok) { failed = true; break; }
        switch (p.world_size) {
          case 2: reduce_own_tile<2, kAllReduce>(p, taddr, mb, ni, r, etid, strip, kNStrips, strip_ctr); break;
          case 4: reduce_own_tile<4, kAllReduce>(p, taddr, mb, ni, r, etid, strip, kNStrips, strip_ctr); break;
          case 8: reduce_own_tile<8, kAllReduce>(p, taddr, mb, ni, r, etid, strip, kNStrips, strip_ctr); break;
          default: reduce_own_tile<0, kAllReduce>(p, taddr, mb, ni, r, etid, strip, kNStrips, strip_ctr); break;
        }
      } else if (valid) {
#pragma unroll 1
        for (int sidx = 0; sidx < kStripsPerTile; ++sidx) {
          const int col0 = ni * kBN + sidx * kStripCols;
          if (col0 >= p.N) break;                          // uniform over the CTA
          uint32_t v0[32], v1[32];
          tmem_ld_32x32b_x32(taddr + (uint32_t)(sidx * kStripCols), v0);
          tmem_ld_32x32b_x32(taddr + (uint32_t)(sidx * kStripCols + 32), v1);
          tmem_ld_wait();
          // every thread has copied the strip before last out of the buffer we are about to fill
          epilogue_sync();
          uint8_t* buf = strip + (size_t)(strip_ctr % (uint32_t)kNStrips) * kStripBytesOne;
          strip_row_to_smem(buf, r, v0, v1);
          epilogue_sync();                                 // the strip is complete in shared memory
          char* dst = static_cast<char*>(p.buffers[dest]) + p.inbox_offset +
                      strip_offset(p.rank, mb, ni, sidx, p.blocks_per_rank, p.n_tiles_n);
          strip_copy_out(dst, buf, etid);
          ++strip_ctr;
          ++strips;
        }
      }
      // the accumulator has been read (or holds nothing to ship): hand it back to the leader's MMA thread
      tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
      epilogue_sync();                                   // every thread has issued its stores of this tile
      if (etid == 0 && strips > 0)                       // (own tiles ship nothing: strips stays 0)
        red_add_release_sys(p.pads[dest] + kFlagSlotsBase + 2 + mb * p.n_tiles_n + ni, 1u);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ---------------- GEMM teardown ----------------
  if (__any_sync(0xffffffffu, failed)) {
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  tcgen05_fence_before_thread_sync();
  failed = __syncthreads_or(failed) != 0;
  cluster_sync_all();   // the peer may still read this CTA's smem / signal its barriers until here
  tcgen05_fence_after_thread_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
  if (p.trace != nullptr && threadIdx.x == 0) p.trace[blockIdx.x * 4 + 2] = globaltimer_ns();

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
  const int ws = a.pv.world_size;
  if (a.M <= 0 || a.N % 8 != 0 || a.K % 8 != 0 || a.M % (ws * kBM) != 0) return cudaErrorInvalidValue;
  RsParams p{};
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.rank = a.pv.rank; p.world_size = ws;
  p.blocks_per_rank = a.M / ws / kBM;
  p.n_tiles_n = (a.N + kBN - 1) / kBN;
  // column panels only for a B beyond the L2: timed in turns on four GPUs (down-projection, B = 117 MB), one
  // panel took 2785 µs and panels of 16 / 11 / 8 tiles 2935 / 2999 / 3002 µs
  p.panel_w = a.panel_w > 0 ? (a.panel_w < p.n_tiles_n ? a.panel_w : p.n_tiles_n)
                            : pick_panel_w(p.n_tiles_n, (size_t)kBN * a.K * 2, kPanelBudgetL2);
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
    if (a.ar_peers == nullptr || a.ar_offset % 16 != 0) return cudaErrorInvalidValue;
    p.ar_peers = a.ar_peers;
    p.ar_mc = a.ar_mc;
    p.ar_offset = a.ar_offset;
  } else if (a.out == nullptr) {
    return cudaErrorInvalidValue;
  }
  CUtensorMap ta, tb;
  if (make_tmap(&ta, a.a, (uint64_t)a.M, (uint64_t)a.K, kBM)) return cudaErrorInvalidValue;
  if (make_tmap(&tb, a.b, (uint64_t)a.N, (uint64_t)a.K, kBN / 2)) return cudaErrorInvalidValue;
  const int n_rb = ws * p.blocks_per_rank;
  const int total_tiles = ((n_rb + 1) / 2) * p.n_tiles_n;
  int pairs = a.num_sms / 2;
  if (pairs > total_tiles) pairs = total_tiles;
  if (pairs < 1) return cudaErrorInvalidValue;
  const int grid = 2 * pairs;
  if ((uint32_t)(1024 + grid) * (uint32_t)ws > kBlockSlots) return cudaErrorInvalidValue;
  if (a.all_reduce) {
    auto kern = matmul_rs_kernel<true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairRsSmem::kTotal);
    if (e != cudaSuccess) return (int)e;
    // the CTAs of a rank wait for the same CTAs of the peers (entry barrier, arrival counters)
    if (int rc = check_co_resident(kern, grid, kThreads, PairRsSmem::kTotal, 2)) return rc;
    kern<<<grid, kThreads, PairRsSmem::kTotal, stream>>>(ta, tb, p);
    return (int)cudaGetLastError();
  }
  auto kern = matmul_rs_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairRsSmem::kTotal);
  if (e != cudaSuccess) return (int)e;
  if (int rc = check_co_resident(kern, grid, kThreads, PairRsSmem::kTotal, 2)) return rc;
  kern<<<grid, kThreads, PairRsSmem::kTotal, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

}  // namespace smr
