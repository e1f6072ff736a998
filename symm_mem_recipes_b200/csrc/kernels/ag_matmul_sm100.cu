// all_gather_matmul for sm_100a:  C[M,N] = all_gather(A_shard)[M,K] * B[N,K]^T
// (bf16 in, fp32 accumulate in TMEM, bf16 out), the all-gather running inside
// the same kernel as the GEMM.
//
// What it does follows symm_mem_recipes/triton_all_gather_matmul.py:20-56 and
// :98-193 (all-gather with progress flags; persistent GEMM that visits M in the
// order shards arrive, own shard first, :157-174).  How it does it is specific
// to Blackwell:
//
//  * grid = one GEMM CTA per SM (in pull mode n_copy of them are "copier" CTAs instead).
//  * PUSH mode (a_out in symmetric memory; the default): no SM is set aside
//    for communication.  Every rank broadcasts its OWN shard into the a_out
//    of all ranks with `multimem.st` on the NVLink multicast address, so a
//    shard leaves its GPU once and the NVSwitch fans it out (plain peer stores
//    when there is no multicast mapping).  The shard is cut into pieces of
//    1/16 of a 128-row block, dealt round-robin to ALL GEMM CTAs, whose four
//    epilogue warps push them in the time they would otherwise idle waiting
//    for an accumulator: before the epilogue of its j-th tile a CTA pushes its
//    pieces of every block that some tile of round j+1 reads, so the data is
//    on the wire one tile-time ahead of need and no CTA can block while it
//    holds a piece a peer waits for.  One SM sustains only ~30 GB/s of NVLink
//    stores (measured); spread over 148 SMs the gather costs no SM at all.
//    After a piece, the block's arrival counter on every rank gets +1
//    (red.release.sys); the counter of call number e reads pieces * e, so
//    nothing is reset between calls.  An entry barrier over the signal pad,
//    run by the epilogue warps, proves that every rank has finished reading
//    the a_out of the previous call.
//  * PULL mode (a_out is an ordinary tensor, as upstream): n_copy copier CTAs
//    are set aside; in each, one thread pulls the peers' shards with untiled
//    TMA bulk copies peer-HBM -> shared memory -> local a_out and publishes
//    one flag per block once its writes are done; entry barrier = the peers'
//    shards are ready, exit barrier = they may be overwritten (upstream :56,
//    :250).  One SM moves only ~14 GB/s this way (measured), so this mode
//    needs many copier CTAs and is slower than the push mode.
//  * M schedule: a few blocks of the own shard first (they never wait and
//    cover the start-up of the gather), then, for k = 0, 1, ...: block k of
//    rank+1, rank+2, ... and one more own block (upstream pivots by rank,
//    :157-163).  All senders deliver their k-th blocks at about the same
//    time, so this order keeps the GEMM behind the arrivals.
//  * GEMM CTA, warp-specialised:
//      warp 0   TMA producer: waits for the block's flag (remote blocks
//               only), then loads A [128 x 64] and B [BN x 64] tiles with the
//               128-byte swizzle into a ring of STAGES stages.
//      warp 1   MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16)
//               into one of two TMEM accumulators; tcgen05.commit frees the
//               stage / hands the accumulator to the epilogue.
//      warps 2-5 epilogue: tcgen05.ld the accumulator, convert to bf16, store C;
//               overlaps the next tile's main loop (double-buffered TMEM).
//  * every wait (flag, mbarrier, barrier) is bounded; on expiry the kernel
//    records a Status, lets copies in flight land, frees TMEM and returns.
//
// With n_copy = 0 the kernel is a plain persistent GEMM (upstream's `mm_only`).
#include "ag_matmul_common.cuh"

namespace smr {

using namespace agmm;

namespace {

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = BN * kBK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kRingBytes = kStageBytes * STAGES;
  static constexpr uint32_t kBarOffset = kRingBytes;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], copier full[32]
  static constexpr uint32_t kNumBars = 2 * STAGES + 4;
  static constexpr uint32_t kCopyBufs = kRingBytes / kCopyChunk;
  static constexpr uint32_t kMiscOffset = kBarOffset + 8 * (kNumBars + 32);
  static constexpr uint32_t kTotal = kMiscOffset + 16 + 1024;  // + alignment slack
};

// ---------------------------------------------------------------------------
// Copier: thread 0 of a copier CTA.
// Work items in the order the GEMM consumes them (block k of every shard,
// then block k+1); copier i takes items i, i + n_copy, ...
// ---------------------------------------------------------------------------
template <int BN, int STAGES>
__device__ void copier_thread(const AgMatmulParams& p, int copier, uint8_t* ring, uint64_t* cbar) {
  using L = SmemLayout<BN, STAGES>;
  constexpr uint32_t NBUF = L::kCopyBufs < 32 ? L::kCopyBufs : 32;
  const size_t block_bytes = (size_t)kBM * p.K * 2;
  const int bpr = p.blocks_per_rank;
  const int total_items = p.world_size * bpr;   // includes the own shard (last)
  const uint32_t chunks_per_block = (uint32_t)((block_bytes + kCopyChunk - 1) / kCopyChunk);

  // number of items of this copier and chunk stream length
  int my_items = 0;
  for (int w = copier; w < total_items; w += p.n_copy) ++my_items;
  const uint64_t total_chunks = (uint64_t)my_items * chunks_per_block;

  auto chunk_src_dst = [&](uint64_t c, const char*& src, char*& dst, uint32_t& bytes, int& gblock) {
    int item = copier + (int)(c / chunks_per_block) * p.n_copy;
    uint32_t ch = (uint32_t)(c % chunks_per_block);
    int blk = item / p.world_size;             // block k of every shard before block k+1
    int step = item % p.world_size;            // 0 = own shard (side output only)
    int peer = (p.rank + step) % p.world_size;
    size_t off = (size_t)ch * kCopyChunk;
    size_t left = block_bytes - off;
    bytes = (uint32_t)(left < kCopyChunk ? left : kCopyChunk);
    src = static_cast<const char*>(p.buffers[peer]) + p.shard_offset + (size_t)blk * block_bytes + off;
    gblock = peer * bpr + blk;
    dst = p.a_out + (size_t)gblock * block_bytes + off;
  };

  bool ok = true;
  uint64_t issued = 0;
  // prologue: fill the ring
  for (; issued < total_chunks && issued < NBUF; ++issued) {
    const char* src; char* dst; uint32_t bytes; int gb;
    chunk_src_dst(issued, src, dst, bytes, gb);
    uint32_t b = (uint32_t)(issued % NBUF);
    mbar_arrive_expect_tx(&cbar[b], bytes);
    bulk_load(ring + (size_t)b * kCopyChunk, src, bytes, &cbar[b]);
  }
  int pending_block = -1;        // block whose last store is issued, flag not yet published
  uint64_t pending_at = 0;
  for (uint64_t c = 0; c < total_chunks; ++c) {
    const char* src; char* dst; uint32_t bytes; int gb;
    chunk_src_dst(c, src, dst, bytes, gb);
    uint32_t b = (uint32_t)(c % NBUF);
    if (!mbar_wait(&cbar[b], (uint32_t)((c / NBUF) & 1), p.timeout_ns)) {
      report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, 0, kWhereCopierEntry, (uint32_t)c);
      ok = false;
      break;
    }
    fence_proxy_async();
    bulk_store(dst, ring + (size_t)b * kCopyChunk, bytes);
    bulk_commit_group();
    // refill the buffer used kStoreLag chunks ago, once its store has read it
    if (c >= (uint64_t)kStoreLag) {
      bulk_wait_group_read<kStoreLag>();
      uint64_t nc = c - kStoreLag + NBUF;
      if (nc < total_chunks && nc >= issued) {
        const char* s2; char* d2; uint32_t by2; int gb2;
        chunk_src_dst(nc, s2, d2, by2, gb2);
        uint32_t b2 = (uint32_t)(nc % NBUF);
        mbar_arrive_expect_tx(&cbar[b2], by2);
        bulk_load(ring + (size_t)b2 * kCopyChunk, s2, by2, &cbar[b2]);
        issued = nc + 1;
      }
    }
    // publish the previous block once its stores are kFlagLag groups old
    if (pending_block >= 0 && c - pending_at >= (uint64_t)kFlagLag) {
      bulk_wait_group<kFlagLag>();
      fence_proxy_async();
      st_release_gpu(&p.flags[pending_block], 1u);
      pending_block = -1;
    }
    if ((c % chunks_per_block) == chunks_per_block - 1) {
      if (pending_block >= 0) {   // short blocks: drain now
        bulk_wait_group<1>();
        fence_proxy_async();
        st_release_gpu(&p.flags[pending_block], 1u);
      }
      pending_block = gb;
      pending_at = c;
    }
  }
  bulk_wait_group<0>();
  if (ok && pending_block >= 0) {
    fence_proxy_async();
    st_release_gpu(&p.flags[pending_block], 1u);
  }
  // remaining refills that the loop above did not reach cannot exist: every
  // chunk index < total_chunks is issued either by the prologue or by the
  // refill of chunk (index - NBUF + kStoreLag).
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
ag_matmul_kernel(const __grid_constant__ CUtensorMap tmap_a_shard,
                 const __grid_constant__ CUtensorMap tmap_a_out,
                 const __grid_constant__ CUtensorMap tmap_b, const AgMatmulParams p) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint64_t* copy_bar = bars + L::kNumBars;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOffset);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // push mode: this call's number, the value every arrival counter will reach
  uint32_t epoch = 0, flag_target = p.flag_target;
  if (p.mode == 2) {
    epoch = ld_relaxed_gpu(&p.header[0]) + 1u;
    flag_target = epoch * kArrivalUnits;
  }

  // ======================= copier CTAs (pull mode only) =======================
  if ((int)blockIdx.x < p.n_copy) {
    if (threadIdx.x == 0) {
      for (int i = 0; i < 32; ++i) mbar_init(&copy_bar[i], 1);
      mbar_fence_init();
    }
    // entry: every peer's shard is written (its earlier kernels are done)
    bool ok = blockwise_barrier(p.pads, p.barrier_block_base + blockIdx.x, p.rank, p.world_size,
                                p.timeout_ns, p.status, kWhereCopierEntry);
    if (ok) {
      if (threadIdx.x == 0) copier_thread<BN, STAGES>(p, (int)blockIdx.x, smem, copy_bar);
      // exit: every peer has finished reading this rank's shard
      blockwise_barrier(p.pads, p.barrier_block_base + blockIdx.x, p.rank, p.world_size,
                        p.timeout_ns, p.status, kWhereCopierExit);
    }
    return;
  }

  // ======================= GEMM CTAs =======================
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);   // one arrival per epilogue warp
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a_shard);
    tma_prefetch_desc(&tmap_a_out);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_thread_sync();
  __syncthreads();
  tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int gemm_cta = (int)blockIdx.x - p.n_copy;
  const int n_gemm = (int)gridDim.x - p.n_copy;
  const int total_tiles = p.n_blocks_m * p.n_tiles_n;
  const int k_blocks = (p.K + kBK - 1) / kBK;
  const int rows_per_rank = p.blocks_per_rank * kBM;
  bool failed = false;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int t = gemm_cta; t < total_tiles && !failed; t += n_gemm) {
        int mi = t / p.n_tiles_n, ni = t % p.n_tiles_n;
        bool local;
        const int mblk = scheduled_block(p, mi, local);
        const CUtensorMap* amap = &tmap_a_out;
        int row0 = mblk * kBM;
        if (p.mode != 0 && local) {
          amap = &tmap_a_shard;
          row0 -= p.rank * rows_per_rank;
        }
        if (!local) {
          if (!wait_reached_acquire_sys(&p.flags[mblk], flag_target, p.timeout_ns)) {
            report_status(p.status, kTimeoutFlag, p.rank, blockIdx.x, mblk, kWhereGemmProgress);
            failed = true;
            break;
          }
          fence_proxy_async();   // flag seen by the generic proxy; data read by TMA
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.timeout_ns)) {
            report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, stage, kWhereGemmEmpty);
            failed = true;
            break;
          }
          uint8_t* sa = smem + (size_t)stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(sa, amap, &full_bar[stage], kb * kBK, row0);
          tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBK, ni * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(kBM, BN);
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      for (int t = gemm_cta; t < total_tiles && !failed; t += n_gemm) {
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
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // +32 bytes per K step inside the swizzled row = +2 descriptor units
            umma_bf16_ss(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                         (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);   // stage reusable when these MMAs finish
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(&tmem_full[acc]);       // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;           // TMEM lanes [32*quarter, +32)
    uint32_t acc = 0, acc_phase = 0;
    // push mode: this CTA's pieces of the own shard go out just ahead of need,
    // one round of tiles in advance, so the epilogue warps never sit on data a
    // peer is waiting for
    const int etid = (int)threadIdx.x - 64;
    int next_piece = gemm_cta, round = 0;
    const int all_pieces = p.blocks_per_rank * p.pieces;
    if (p.mode == 2 && !push_entry_barrier(p, gemm_cta, etid)) failed = true;
    for (int t = gemm_cta; t < total_tiles && !failed; t += n_gemm) {
      int mi = t / p.n_tiles_n, ni = t % p.n_tiles_n;
      bool local_unused;
      const int mblk = scheduled_block(p, mi, local_unused);
      if (p.mode == 2) {
        next_piece = push_pieces(p, next_piece, n_gemm, pieces_needed_through_round(p, round + 1, n_gemm), etid);
        ++round;
      }
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.timeout_ns)) {
        if (lane == 0)
          report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, acc, kWhereGemmTmemFull);
        failed = true;
        break;
      }
      tcgen05_fence_after_thread_sync();
      const int row = mblk * kBM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * 256u + ((uint32_t)(quarter * 32) << 16);
      __nv_bfloat16* crow = p.c + (size_t)row * p.N + (size_t)ni * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
        tmem_ld_wait();
        const int col0 = ni * BN + c * 32;
        if (row < p.M) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 < p.N) {   // N % 8 == 0: a group of 8 is in or out as a whole
              Vec16 o;
              o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              st_16(crow + c * 32 + v * 8, o);
            }
          }
        }
      }
      tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (p.mode == 2 && !failed) push_pieces(p, next_piece, n_gemm, all_pieces, etid);
  }

  // ---------------- teardown ----------------
  if (__any_sync(0xffffffffu, failed)) {
    // let TMA copies that are still in flight land before the CTA goes away
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  tcgen05_fence_before_thread_sync();
  __syncthreads();
  tcgen05_fence_after_thread_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (p.mode == 2 && threadIdx.x == 0) {
    // the last CTA of the grid to finish publishes this call's number
    uint32_t done = atomicAdd(&p.header[1], 1u);
    if (done == gridDim.x - 1) {
      p.header[1] = 0u;
      __threadfence();
      st_release_gpu(&p.header[0], epoch);
    }
  }
}

template <int BN, int STAGES>
int launch_variant(const CUtensorMap& ta_shard, const CUtensorMap& ta_out, const CUtensorMap& tb,
                   const AgMatmulParams& p, int grid, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  static_assert(L::kTotal <= 232448, "shared memory limit exceeded");
  auto kern = ag_matmul_kernel<BN, STAGES>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::kTotal);
  if (e != cudaSuccess) return (int)e;
  kern<<<grid, kGemmThreads, L::kTotal, stream>>>(ta_shard, ta_out, tb, p);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_ag_matmul(const AgMatmulArgs& a, cudaStream_t stream) {
  if (a.N % 8 != 0 || a.K % 8 != 0 || a.M <= 0 || a.N <= 0 || a.K <= 0) return cudaErrorInvalidValue;
  const bool comm = a.mode != 0;
  if (comm) {
    if ((a.mode == 1 && a.n_copy < 1) || a.world_size < 2 || a.rows_per_rank % kBM != 0 ||
        a.rows_per_rank * a.world_size != a.M || a.a_out == nullptr || a.pads == nullptr)
      return cudaErrorInvalidValue;
    if (a.mode == 1 && (a.buffers == nullptr || a.flags == nullptr)) return cudaErrorInvalidValue;
    if (a.mode == 2 && (a.aout_buffers == nullptr || a.local_pad == nullptr)) return cudaErrorInvalidValue;
    if (a.mode == 2 && (uint32_t)(a.M / kBM) + 2u > kFusedFlagSlots) return cudaErrorInvalidValue;
  }
  int bn = a.block_n;
  if (bn != 128 && bn != 192 && bn != 224 && bn != 256) return cudaErrorInvalidValue;
  if (a.elem_bytes != 0 && a.elem_bytes != 2) return cudaErrorInvalidValue;   // fp8: 2-CTA kernel

  AgMatmulParams p{};
  p.c = static_cast<__nv_bfloat16*>(a.c);
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.elem_bytes = 2;
  p.n_tiles_n = (a.N + bn - 1) / bn;
  p.n_blocks_m = (a.M + kBM - 1) / kBM;
  p.rank = comm ? a.rank : 0;
  p.world_size = comm ? a.world_size : 1;
  p.blocks_per_rank = comm ? a.rows_per_rank / kBM : p.n_blocks_m;
  p.n_copy = a.mode == 1 ? a.n_copy : 0;
  p.mode = comm ? a.mode : 0;
  p.lead = 0;
  p.pieces = 1;
  if (a.mode == 2) {
    p.lead = p.blocks_per_rank < 4 ? p.blocks_per_rank : 4;
    size_t block_vecs = (size_t)kBM * a.K * 2 / 16;
    p.pieces = block_vecs >= 8192 ? 16 : (block_vecs >= 1024 ? 4 : 1);
  }
  p.flags = a.mode == 2 ? a.local_pad + kFlagSlotsBase + 2 : a.flags;
  p.flag_target = 1u;
  p.header = a.mode == 2 ? a.local_pad + kFlagSlotsBase : nullptr;
  p.a_local = static_cast<const char*>(a.a_local);
  p.aout_buffers = a.aout_buffers;
  p.aout_mc = a.aout_mc;
  p.aout_offset = a.aout_offset;
  p.buffers = a.buffers;
  p.shard_offset = a.shard_offset;
  p.a_out = static_cast<char*>(a.a_out);
  p.pads = a.pads;
  p.barrier_block_base = a.barrier_block_base;
  p.timeout_ns = a.timeout_ns;
  p.status = a.status;

  CUtensorMap ta_shard, ta_out, tb;
  // a_local: the matrix GEMM CTAs read without waiting (own shard, or all of A
  // when there is no communication)
  int rows_local = comm ? a.rows_per_rank : a.M;
  if (make_tmap(&ta_shard, a.a_local, (uint64_t)rows_local, (uint64_t)a.K, kBM)) return cudaErrorInvalidValue;
  if (make_tmap(&ta_out, comm ? a.a_out : a.a_local, (uint64_t)a.M, (uint64_t)a.K, kBM)) return cudaErrorInvalidValue;
  if (make_tmap(&tb, a.b, (uint64_t)a.N, (uint64_t)a.K, (uint32_t)bn)) return cudaErrorInvalidValue;

  int total_tiles = p.n_blocks_m * p.n_tiles_n;
  int gemm_ctas = a.num_sms - p.n_copy;
  if (gemm_ctas < 1) return cudaErrorInvalidValue;
  if (gemm_ctas > total_tiles) gemm_ctas = total_tiles;
  int grid = gemm_ctas + p.n_copy;
  // the entry barriers use block slots (barrier_block_base + CTA index): stay inside the block-slot region
  if (comm && ((size_t)a.barrier_block_base + grid) * a.world_size > kBlockSlots) return cudaErrorInvalidValue;

  switch (bn) {
    case 128: return launch_variant<128, 6>(ta_shard, ta_out, tb, p, grid, stream);
    case 192: return launch_variant<192, 5>(ta_shard, ta_out, tb, p, grid, stream);
    case 224: return launch_variant<224, 5>(ta_shard, ta_out, tb, p, grid, stream);
    default:  return launch_variant<256, 4>(ta_shard, ta_out, tb, p, grid, stream);
  }
}

}  // namespace smr
