// The consumer GEMM of all_gather_matmul (upstream: `matmul_kernel_tma_persistent`,
// symm_mem_recipes/triton_all_gather_matmul.py:98-193, launched from :295-315)
// with tcgen05 `cta_group::2`: two CTAs on neighbouring SMs
// (a cluster of 2) share one 256 x BN tile.  Each CTA stages ITS OWN 128 rows
// of A and ITS OWN half of the B tile (BN/2 rows) with ordinary TMA loads — no
// cluster-multicast qualifier anywhere — and the leader CTA's single MMA thread
// issues `tcgen05.mma.cta_group::2`, which reads A and B from both CTAs'
// shared memory and writes each CTA's 128 accumulator rows into that CTA's own
// TMEM.  Per flop every SM pulls half as many B bytes out of L2 as a kernel with
// one CTA per 128 x BN tile would (ncu: tensor pipe 92 % active against 80 %).
//
// Hand-offs inside the pair:
//   full[s]        leader only.  The leader's producer arrives with the byte
//                  count of BOTH CTAs' loads; both CTAs' TMA loads complete on
//                  the leader's barrier (`.cta_group::2` form of the load).
//   empty[s]       both CTAs; `tcgen05.commit ... multicast::cluster` from the
//                  leader's MMA thread frees the stage in both.
//   tmem_full[b]   both CTAs; same multicast commit.
//   tmem_empty[b]  leader only, 8 arrivals: the four epilogue warps of each CTA
//                  (the peer's arrive through a shared::cluster address).
// Tail of the static schedule: when the last wave would fill only a few pairs
// (896 tiles on 74 pairs leave 8), each of its tiles is cut along K into 2, 4
// or 8 parts that run on as many pairs at once.  Every part stores its fp32
// partial accumulator to scratch memory, bumps the tile's arrival counter,
// waits (bounded) for the other parts and then reduces ITS share of the tile's
// columns in part order, so the result does not depend on timing.
// The two 128-row blocks of a pair are two consecutive positions of the M
// schedule, not necessarily neighbours in memory: each CTA loads, waits for and
// stores its own block.
//
// Gather (mode 2, "push"): every rank broadcasts its own shard into the a_out of all
// ranks, with multimem.st through the NVSwitch from four ranks on, with plain peer
// stores below.  The shard is cut into pieces dealt to ALL GEMM CTAs, whose four
// epilogue warps push them in the time they would idle waiting for an accumulator,
// one round of tiles ahead of the first need; a block's arrival counter on every
// rank grows with each piece, and the TMA producer of a tile that reads a remote
// block waits (bounded) on the local counter.  Measured against the alternative of
// pulling the peers' shards with dedicated copier CTAs (a one-CTA-per-tile kernel
// this library used to carry): 1940 µs against 705-724 µs on 4 GPUs at the
// Llama-3-70B shape; an ordinary (non-symmetric) a_out is therefore served by this
// kernel through the internal symmetric buffer plus one local copy.
#include "../device/tcgen05_pair.cuh"
#include "ag_matmul_common.cuh"
#include "residency.h"

namespace smr {

using namespace agmm;

namespace {

// Whether an instantiation's epilogue leaves through shared memory and TMA stores: plain bf16
// output in whole boxes of 64 columns (a 224-wide tile would spill into its neighbour's columns).
template <int BN, bool kFp8, bool kSwiGlu>
constexpr bool pair_tma_store() { return !kFp8 && !kSwiGlu && BN % 64 == 0; }

// kOut: the plain bf16 epilogue leaves through shared memory: each epilogue warp owns two
// 4 KB boxes (32 rows x 64 columns, 128-byte swizzle) that it fills from its accumulator rows
// and hands to a TMA store while it converts the next 64 columns into the other box.
template <int BN, int STAGES, bool kOut = false>
struct PairSmem {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = (BN / 2) * kBK * 2;     // this CTA's half of the B tile
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kRingBytes = kStageBytes * STAGES;
  static constexpr uint32_t kOutBoxBytes = 32 * 128;          // 32 rows x 64 bf16
  static constexpr uint32_t kOutOffset = kRingBytes;
  static constexpr uint32_t kOutBytes = kOut ? 4 * 2 * kOutBoxBytes : 0;
  static constexpr uint32_t kBarOffset = kRingBytes + kOutBytes;
  static constexpr uint32_t kNumBars = 2 * STAGES + 4;
  static constexpr uint32_t kMiscOffset = kBarOffset + 8 * kNumBars;
  static constexpr uint32_t kTotal = kMiscOffset + 16 + 1024;
  static_assert(kStageBytes % 1024 == 0, "stage bases must stay 1024-byte aligned");
};

// kFp8: A, B, C (and the gathered A) hold e4m3 bytes.  All byte geometry stays
// (128-byte rows, 16 KB A stage, 32 bytes of K per MMA); a K block is then 128
// elements instead of 64 and the epilogue packs four outputs per 32-bit word.
// kSwiGlu (bf16, BN = 256): the rows of B are interleaved in groups of 128 so that every
// 256-column tile holds 128 gate columns followed by the 128 matching up columns;
// the epilogue writes SiLU(gate) * up, i.e. C is [M, N / 2] and tile ni covers its
// columns [128 ni, 128 ni + 128).  The activation never makes a round trip through
// memory and C is half as wide.  The split-K tail is not used with it.
template <int BN, int STAGES, bool kFp8, bool kSwiGlu = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
ag_matmul_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a_shard,
                      const __grid_constant__ CUtensorMap tmap_a_out,
                      const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const AgMatmulParams p) {
  constexpr bool kTmaStore = pair_tma_store<BN, kFp8, kSwiGlu>();
  using L = PairSmem<BN, STAGES, kTmaStore>;
  extern __shared__ uint8_t smem_raw[];
  // same offset in both CTAs: the dynamic window starts at the same shared address
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOffset);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  static_assert(!kSwiGlu || (BN == 256 && !kFp8), "the SwiGLU epilogue is built for bf16 tiles of 256 columns");

  uint32_t epoch = 0, flag_target = p.flag_target;
  if (p.mode == 2) {
    epoch = ld_relaxed_gpu(&p.header[0]) + 1u;
    flag_target = epoch * kArrivalUnits;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 8);   // 4 epilogue warps x 2 CTAs (used in the leader)
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a_shard);
    tma_prefetch_desc(&tmap_a_out);
    tma_prefetch_desc(&tmap_b);
    if constexpr (kTmaStore) tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before_thread_sync();
  __syncthreads();
  cluster_sync_all();                 // barriers of both CTAs initialised, TMEM allocated
  tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool tr = p.trace != nullptr;
  uint64_t* trc = tr ? p.trace + (size_t)blockIdx.x * ag_trace::kTraceSlots : nullptr;
  if (tr && threadIdx.x == 0) trc[ag_trace::kStart] = globaltimer_ns();

  const int pair = (int)blockIdx.x >> 1;
  const int n_pairs = (int)gridDim.x >> 1;
  const int n_pair_rows = (p.n_blocks_m + 1) >> 1;         // 256-row tiles along M
  const int total_tiles = n_pair_rows * p.n_tiles_n;
  constexpr int kBKE = kFp8 ? 2 * kBK : kBK;                // elements of K per 128-byte row
  const int k_blocks = (p.K + kBKE - 1) / kBKE;
  const int rows_per_rank = p.blocks_per_rank * kBM;
  bool failed = false;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      PairWork w;
      uint64_t t_flag = 0, t_stage = 0, t_first = 0;
      bool first_remote = true;
      for (int wi = 0; !failed && pair_work(p, pair, n_pairs, total_tiles, k_blocks, wi, w); ++wi) {
        const int t = w.tile;
        int prow, ni;
        tile_coords(p, n_pair_rows, t, prow, ni);
        const int mi = prow * 2 + (int)cta_rank;
        bool local = true;
        const CUtensorMap* amap = &tmap_a_out;
        int row0;
        if (mi < p.n_blocks_m) {
          const int mblk = scheduled_block(p, mi, local);
          row0 = mblk * kBM;
          if (p.mode != 0 && local) {
            amap = &tmap_a_shard;
            row0 -= p.rank * rows_per_rank;
          }
          if (!local) {
            const uint64_t t0 = tr ? globaltimer_ns() : 0;
            if (!wait_reached_acquire_sys(&p.flags[mblk], flag_target, p.timeout_ns)) {
              report_status(p.status, kTimeoutFlag, p.rank, blockIdx.x, mblk, kWhereGemmProgress);
              failed = true;
              break;
            }
            fence_proxy_async();
            if (tr) {
              const uint64_t dt = globaltimer_ns() - t0;
              t_flag += dt;
              if (first_remote) { t_first = dt; first_remote = false; }
            }
          }
        } else {
          row0 = p.n_blocks_m * kBM;   // odd tail: rows past M read as zero
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_try_wait(&empty_bar[stage], phase ^ 1)) {
            const uint64_t t0 = tr ? globaltimer_ns() : 0;
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.timeout_ns)) {
              report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, stage, kWhereGemmEmpty);
              failed = true;
              break;
            }
            if (tr) t_stage += globaltimer_ns() - t0;
          }
          uint8_t* sa = smem + (size_t)stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2u * L::kStageBytes);
          const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, amap, full_leader, kb * kBKE, row0);
          tma_load_2d_pair(sb, &tmap_b, full_leader, kb * kBKE, ni * BN + (int)cta_rank * (BN / 2));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (tr) {
        trc[ag_trace::kFlagWait] = t_flag;
        trc[ag_trace::kStageWait] = t_stage;
        trc[ag_trace::kFirstFlagWait] = t_first;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = kFp8 ? umma_idesc_e4m3_f32(2 * kBM, BN) : umma_idesc_bf16_f32(2 * kBM, BN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      PairWork w;
      uint64_t t_tmem = 0, t_opnd = 0;
      for (int wi = 0; !failed && pair_work(p, pair, n_pairs, total_tiles, k_blocks, wi, w); ++wi) {
        if (!mbar_try_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          const uint64_t t0 = tr ? globaltimer_ns() : 0;
          if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.timeout_ns)) {
            report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, acc, kWhereGemmTmemEmpty);
            failed = true;
            break;
          }
          if (tr) t_tmem += globaltimer_ns() - t0;
        }
        tcgen05_fence_after_thread_sync();
        const uint32_t d_tmem = tmem_base + acc * 256u;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_try_wait(&full_bar[stage], phase)) {
            const uint64_t t0 = tr ? globaltimer_ns() : 0;
            if (!mbar_wait(&full_bar[stage], phase, p.timeout_ns)) {
              report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, stage, kWhereGemmFull);
              failed = true;
              break;
            }
            if (tr) t_opnd += globaltimer_ns() - t0;
          }
          tcgen05_fence_after_thread_sync();
          const uint32_t sa = smem_u32(smem + (size_t)stage * L::kStageBytes);
          const uint64_t da = umma_smem_desc_sw128(sa);
          const uint64_t db = umma_smem_desc_sw128(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            if constexpr (kFp8)
              umma_e4m3_ss_pair(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                (kb != w.kb0 || k != 0) ? 1u : 0u);
            else
              umma_bf16_ss_pair(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                                (kb != w.kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit_pair(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      if (tr) {
        trc[ag_trace::kTmemWait] = t_tmem;
        trc[ag_trace::kOperandWait] = t_opnd;
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
    const int quarter = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    const int etid = (int)threadIdx.x - 64;
    int next_piece = (int)blockIdx.x, round = 0;
    const int all_pieces = p.blocks_per_rank * p.pieces;
    [[maybe_unused]] int out_box = 0;                  // which of this warp's two output boxes is filled next
    if (p.mode == 2 && !push_entry_barrier(p, (int)blockIdx.x, etid)) failed = true;
    const bool trt = tr && etid == 0;
    uint64_t t_push = 0, t_acc = 0, n_units = 0;
    if (trt) trc[ag_trace::kEntered] = globaltimer_ns();
    __shared__ int tail_ok;
    PairWork w;
    for (int wi = 0; !failed && pair_work(p, pair, n_pairs, total_tiles, k_blocks, wi, w); ++wi) {
      const int t = w.tile;
      int prow, ni;
      tile_coords(p, n_pair_rows, t, prow, ni);
      const int mi = prow * 2 + (int)cta_rank;
      bool local_unused;
      const bool valid = mi < p.n_blocks_m;
      const int mblk = valid ? scheduled_block(p, mi, local_unused) : 0;
      if (p.mode == 2) {
        const uint64_t t0 = trt ? globaltimer_ns() : 0;
        next_piece = push_pieces(p, next_piece, (int)gridDim.x,
                                 pieces_due(p, round, n_pairs, 2, all_pieces), etid);
        ++round;
        if (trt) t_push += globaltimer_ns() - t0;
      }
      {
        const uint64_t t0 = trt ? globaltimer_ns() : 0;
        if (!mbar_wait(&tmem_full[acc], acc_phase, p.timeout_ns)) {
          if (lane == 0)
            report_status(p.status, kTimeoutMbarrier, p.rank, blockIdx.x, acc, kWhereGemmTmemFull);
          failed = true;
          break;
        }
        if (trt) { t_acc += globaltimer_ns() - t0; ++n_units; }
      }
      tcgen05_fence_after_thread_sync();
      const int row = mblk * kBM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * 256u + ((uint32_t)(quarter * 32) << 16);
      __nv_bfloat16* crow = p.c + (size_t)row * p.N + (size_t)ni * BN;
      uint8_t* crow8 = reinterpret_cast<uint8_t*>(p.c) + (size_t)row * p.N + (size_t)ni * BN;   // kFp8
      if (w.part >= 0) {
        // ---- split-K tail: park the fp32 partial, meet the other parts, reduce my columns ----
        const int r = quarter * 32 + lane;
        const size_t blk = (size_t)kBM * BN;                       // floats per CTA block
        float* mine = p.tail_scratch + (((size_t)w.tail_idx * p.tail_splits + w.part) * 2 + cta_rank) * blk +
                      (size_t)r * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          if (w.kb1 > w.kb0) {
            tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = 0u;
          }
#pragma unroll
          for (int q = 0; q < 8; ++q)
            st_16(mine + c * 32 + q * 4, Vec16{v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]});
        }
        tcgen05_fence_before_thread_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
        __threadfence();
        if (etid == 0) tail_ok = 1;
        epilogue_group_sync();
        uint32_t* counter = p.tail_counters + w.tail_idx * 2 + cta_rank;
        if (etid == 0) {
          red_add_release_gpu(counter, 1u);
          if (!wait_ge_acquire_gpu(counter, (uint32_t)p.tail_splits, p.timeout_ns)) {
            report_status(p.status, kTimeoutFlag, p.rank, blockIdx.x, w.tail_idx, kWhereGemmTmemFull, w.part);
            tail_ok = 0;
          }
        }
        epilogue_group_sync();
        if (!tail_ok) { failed = true; break; }
        const int cw = BN / p.tail_splits;                         // my share of the tile's columns
        const float* base = p.tail_scratch + ((size_t)w.tail_idx * p.tail_splits * 2 + cta_rank) * blk +
                            (size_t)r * BN + (size_t)w.part * cw;
        for (int c8 = 0; c8 < cw; c8 += 8) {
          float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int sp = 0; sp < p.tail_splits; ++sp) {             // part order: deterministic
            const float* src = base + (size_t)sp * 2 * blk + c8;
            Vec16 lo = ld_16_stream(src), hi = ld_16_stream(src + 4);
            s[0] += __uint_as_float(lo.x); s[1] += __uint_as_float(lo.y);
            s[2] += __uint_as_float(lo.z); s[3] += __uint_as_float(lo.w);
            s[4] += __uint_as_float(hi.x); s[5] += __uint_as_float(hi.y);
            s[6] += __uint_as_float(hi.z); s[7] += __uint_as_float(hi.w);
          }
          const int col = ni * BN + w.part * cw + c8;
          if (valid && row < p.M && col < p.N) {
            if constexpr (kFp8) {
              st_8(crow8 + w.part * cw + c8, pack_e4m3x4(s[0], s[1], s[2], s[3]),
                   pack_e4m3x4(s[4], s[5], s[6], s[7]));
            } else {
              Vec16 o;
              o.x = pack_bf16x2(s[0], s[1]); o.y = pack_bf16x2(s[2], s[3]);
              o.z = pack_bf16x2(s[4], s[5]); o.w = pack_bf16x2(s[6], s[7]);
              st_16(crow + w.part * cw + c8, o);
            }
          }
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        continue;
      }
      if constexpr (kSwiGlu) {
        const int F = p.N >> 1;                            // output columns
        __nv_bfloat16* orow = p.c + (size_t)row * F + (size_t)ni * (BN / 2);
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), g);                 // gate columns
          tmem_ld_32x32b_x32(taddr + (uint32_t)(BN / 2 + c * 32), u);        // the matching up columns
          tmem_ld_wait();
          const int col0 = ni * (BN / 2) + c * 32;
          if (valid && row < p.M) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 < F) {
                float y[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  const float gv = __uint_as_float(g[v * 8 + q]);
                  y[q] = gv / (1.0f + __expf(-gv)) * __uint_as_float(u[v * 8 + q]);
                }
                Vec16 o;
                o.x = pack_bf16x2(y[0], y[1]); o.y = pack_bf16x2(y[2], y[3]);
                o.z = pack_bf16x2(y[4], y[5]); o.w = pack_bf16x2(y[6], y[7]);
                st_16(orow + c * 32 + v * 8, o);
              }
            }
          }
        }
      } else if constexpr (kTmaStore) {
        // 64 columns at a time: two TMEM loads in flight, bf16 into this warp's free box
        // (16-byte chunk j of row r sits at chunk j ^ (r & 7): the 128-byte swizzle of the
        // tensor map, and conflict-free for the warp's stores), then one TMA store.
        const uint32_t box0 = smem_u32(smem + L::kOutOffset) + (uint32_t)quarter * 2u * L::kOutBoxBytes;
        const bool store_ok = valid && mblk * kBM + quarter * 32 < p.M;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 64), r0);
          tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 64 + 32), r1);
          if (lane == 0) bulk_wait_group_read<1>();      // the store that last read this box is done with it
          __syncwarp();
          tmem_ld_wait();
          if (c == BN / 64 - 1) {
            // the accumulator is in registers: hand it back before the stores
            tcgen05_fence_before_thread_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
          }
          const uint32_t box = box0 + (uint32_t)out_box * L::kOutBoxBytes;
          const uint32_t rowaddr = box + (uint32_t)lane * 128u;
          const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            st_shared_16(rowaddr + ((((uint32_t)j) ^ sw) << 4),
                         pack_bf16x2(__uint_as_float(r0[j * 8 + 0]), __uint_as_float(r0[j * 8 + 1])),
                         pack_bf16x2(__uint_as_float(r0[j * 8 + 2]), __uint_as_float(r0[j * 8 + 3])),
                         pack_bf16x2(__uint_as_float(r0[j * 8 + 4]), __uint_as_float(r0[j * 8 + 5])),
                         pack_bf16x2(__uint_as_float(r0[j * 8 + 6]), __uint_as_float(r0[j * 8 + 7])));
            st_shared_16(rowaddr + ((((uint32_t)(j + 4)) ^ sw) << 4),
                         pack_bf16x2(__uint_as_float(r1[j * 8 + 0]), __uint_as_float(r1[j * 8 + 1])),
                         pack_bf16x2(__uint_as_float(r1[j * 8 + 2]), __uint_as_float(r1[j * 8 + 3])),
                         pack_bf16x2(__uint_as_float(r1[j * 8 + 4]), __uint_as_float(r1[j * 8 + 5])),
                         pack_bf16x2(__uint_as_float(r1[j * 8 + 6]), __uint_as_float(r1[j * 8 + 7])));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (store_ok && ni * BN + c * 64 < p.N) {
              uint8_t* src = smem + L::kOutOffset + ((size_t)quarter * 2 + out_box) * L::kOutBoxBytes;
              tma_store_2d(&tmap_c, src, ni * BN + c * 64, mblk * kBM + quarter * 32);
            }
            bulk_commit_group();
          }
          out_box ^= 1;
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        continue;
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
        tmem_ld_wait();
        const int col0 = ni * BN + c * 32;
        if constexpr (kFp8) {
          if (valid && row < p.M) {
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              if (col0 + v * 16 < p.N) {
                Vec16 o;
                const uint32_t* q = r + v * 16;
                o.x = pack_e4m3x4(__uint_as_float(q[0]), __uint_as_float(q[1]),
                                  __uint_as_float(q[2]), __uint_as_float(q[3]));
                o.y = pack_e4m3x4(__uint_as_float(q[4]), __uint_as_float(q[5]),
                                  __uint_as_float(q[6]), __uint_as_float(q[7]));
                o.z = pack_e4m3x4(__uint_as_float(q[8]), __uint_as_float(q[9]),
                                  __uint_as_float(q[10]), __uint_as_float(q[11]));
                o.w = pack_e4m3x4(__uint_as_float(q[12]), __uint_as_float(q[13]),
                                  __uint_as_float(q[14]), __uint_as_float(q[15]));
                st_16(crow8 + c * 32 + v * 16, o);
              }
            }
          }
        } else if (valid && row < p.M) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 < p.N) {
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
      }   // plain epilogue
      tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if constexpr (kTmaStore) {
      if (lane == 0) bulk_wait_group<0>();             // C is written before the kernel ends
    }
    if (trt) trc[ag_trace::kTilesDone] = globaltimer_ns();
    if (p.mode == 2 && !failed) {
      const uint64_t t0 = trt ? globaltimer_ns() : 0;
      push_pieces(p, next_piece, (int)gridDim.x, all_pieces, etid);
      if (trt) t_push += globaltimer_ns() - t0;
    }
    if (trt) {
      trc[ag_trace::kPush] = t_push;
      trc[ag_trace::kAccWait] = t_acc;
      trc[ag_trace::kTiles] = n_units;
      trc[ag_trace::kEnd] = globaltimer_ns();
    }
  }

  // ---------------- teardown ----------------
  if (__any_sync(0xffffffffu, failed)) {
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  tcgen05_fence_before_thread_sync();
  __syncthreads();
  cluster_sync_all();   // the peer may still read this CTA's smem / signal its barriers until here
  tcgen05_fence_after_thread_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
  if (p.mode == 2 && threadIdx.x == 0) {
    uint32_t done = atomicAdd(&p.header[1], 1u);
    if (done == gridDim.x - 1) {
      p.header[1] = 0u;
      __threadfence();
      st_release_gpu(&p.header[0], epoch);
    }
  }
}

template <int BN, int STAGES, bool kFp8, bool kSwiGlu = false>
int launch_pair_variant(const CUtensorMap& ta_shard, const CUtensorMap& ta_out, const CUtensorMap& tb,
                        const CUtensorMap& tc, const AgMatmulParams& p, int grid, cudaStream_t stream) {
  using L = PairSmem<BN, STAGES, pair_tma_store<BN, kFp8, kSwiGlu>()>;
  static_assert(L::kTotal <= 232448, "shared memory limit exceeded");
  auto kern = ag_matmul_2cta_kernel<BN, STAGES, kFp8, kSwiGlu>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::kTotal);
  if (e != cudaSuccess) return (int)e;
  // The pairs wait for one another (pieces of the gather, parts of the split-K tail): all of them must be resident.
  if (int rc = check_co_resident(kern, grid, kGemmThreads, L::kTotal, 2)) return rc;
  kern<<<grid, kGemmThreads, L::kTotal, stream>>>(ta_shard, ta_out, tb, tc, p);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_ag_matmul_2cta(const AgMatmulArgs& a, cudaStream_t stream) {
  if (a.elem_bytes != 0 && a.elem_bytes != 1 && a.elem_bytes != 2) return cudaErrorInvalidValue;
  const bool fp8 = a.elem_bytes == 1;
  const int es = fp8 ? 1 : 2;
  const int align = 16 / es;                                       // elements per 16 bytes
  if (a.N % align != 0 || a.K % align != 0 || a.M <= 0 || a.N <= 0 || a.K <= 0) return cudaErrorInvalidValue;
  if (a.mode != 0 && a.mode != 2) return cudaErrorInvalidValue;
  const bool comm = a.mode == 2;
  if (comm) {
    if (a.world_size < 2 || a.rows_per_rank % kBM != 0 || a.rows_per_rank * a.world_size != a.M ||
        a.a_out == nullptr || a.pads == nullptr || a.aout_buffers == nullptr || a.local_pad == nullptr)
      return cudaErrorInvalidValue;
    if ((uint32_t)(a.M / kBM) + 2u > kFusedFlagSlots) return cudaErrorInvalidValue;
  }
  const int bn = a.block_n;
  if (bn != 128 && bn != 192 && bn != 224 && bn != 256) return cudaErrorInvalidValue;
  const bool swiglu = a.epilogue == 1;
  if (a.epilogue != 0 && a.epilogue != 1) return cudaErrorInvalidValue;
  // gate / up interleaved in groups of 128 rows of B: whole groups only, bf16, 256-column tiles
  if (swiglu && (fp8 || bn != 256 || a.N % 256 != 0)) return cudaErrorInvalidValue;

  AgMatmulParams p{};
  p.c = static_cast<__nv_bfloat16*>(a.c);
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.elem_bytes = es;
  p.n_tiles_n = (a.N + bn - 1) / bn;
  p.panel_w = a.panel_w > 0 ? (a.panel_w < p.n_tiles_n ? a.panel_w : p.n_tiles_n)
                            : pick_panel_w(p.n_tiles_n, (size_t)bn * a.K * es);
  p.n_blocks_m = (a.M + kBM - 1) / kBM;
  p.rank = comm ? a.rank : 0;
  p.world_size = comm ? a.world_size : 1;
  p.blocks_per_rank = comm ? a.rows_per_rank / kBM : p.n_blocks_m;
  p.mode = a.mode;
  p.lead = 0;
  p.pieces = 1;
  if (comm) {
    p.lead = p.blocks_per_rank < 4 ? p.blocks_per_rank : 4;
    if (a.lead >= 0) p.lead = a.lead < p.blocks_per_rank ? a.lead : p.blocks_per_rank;
    p.push_ahead = a.push_ahead > 0 ? a.push_ahead : 1;
    size_t block_vecs = (size_t)kBM * a.K * es / 16;
    p.pieces = block_vecs >= 8192 ? 16 : (block_vecs >= 1024 ? 4 : 1);
    // A CTA's epilogue warps take 40-60 µs to broadcast 128 KB, about one round of tiles, which is all the
    // lead the schedule gives a piece once the own blocks are used up: with eight ranks (16 blocks per rank,
    // 1.7 pieces of 128 KB per CTA) the CTAs waited 165 µs per call for remote blocks.  So the smaller the
    // shard, the finer the pieces: about six per CTA over the whole shard (64 per block at eight ranks of
    // the headline shape, 32 at four, 16 at two; on four ranks 64 measured 10-29 µs faster than 16).
    while (p.pieces < 256 && (size_t)p.blocks_per_rank * p.pieces < (size_t)6 * a.num_sms &&
           (size_t)(2 * p.pieces) * 128 <= block_vecs)
      p.pieces *= 2;
    if (a.push_pieces > 0) {
      if ((a.push_pieces & (a.push_pieces - 1)) != 0 || (uint32_t)a.push_pieces > kArrivalUnits) return cudaErrorInvalidValue;
      p.pieces = a.push_pieces;
      while (p.pieces > 1 && (size_t)p.pieces * 128 > block_vecs) p.pieces >>= 1;   // a piece feeds 128 threads at least once
    }
  }
  p.flags = comm ? a.local_pad + kFlagSlotsBase + 2 : nullptr;
  p.flag_target = 1u;
  p.header = comm ? a.local_pad + kFlagSlotsBase : nullptr;
  p.a_local = static_cast<const char*>(a.a_local);
  p.aout_buffers = a.aout_buffers;
  p.aout_mc = a.push_plain_stores ? nullptr : a.aout_mc;
  p.aout_offset = a.aout_offset;
  p.a_out = static_cast<char*>(a.a_out);
  p.pads = a.pads;
  p.barrier_block_base = a.barrier_block_base;
  p.timeout_ns = a.timeout_ns;
  p.status = a.status;
  p.trace = a.trace;

  CUtensorMap ta_shard, ta_out, tb, tc;
  int rows_local = comm ? a.rows_per_rank : a.M;
  if (make_tmap(&ta_shard, a.a_local, (uint64_t)rows_local, (uint64_t)a.K, kBM, es)) return cudaErrorInvalidValue;
  if (make_tmap(&ta_out, comm ? a.a_out : a.a_local, (uint64_t)a.M, (uint64_t)a.K, kBM, es))
    return cudaErrorInvalidValue;
  if (make_tmap(&tb, a.b, (uint64_t)a.N, (uint64_t)a.K, (uint32_t)(bn / 2), es)) return cudaErrorInvalidValue;
  // C as the TMA stores of the plain bf16 epilogue see it: boxes of 32 rows x 64 columns
  const int c_cols = swiglu ? a.N / 2 : a.N;
  if (make_tmap(&tc, a.c, (uint64_t)a.M, (uint64_t)c_cols, 32, es)) return cudaErrorInvalidValue;

  const int total_tiles = ((p.n_blocks_m + 1) / 2) * p.n_tiles_n;
  int pairs = a.num_sms / 2;
  if (pairs > total_tiles) pairs = total_tiles;
  if (pairs < 1) return cudaErrorInvalidValue;
  const int grid = 2 * pairs;
  if (comm) {
    if (a.lead < 0) {
      // own blocks first for as long as the first round of tiles lasts: no CTA then starts the kernel
      // waiting for a peer (measured on two ranks: 693 µs with 12 own blocks first, 734 µs with 4)
      const int first_round = 2 * ((pairs + p.panel_w - 1) / p.panel_w);
      p.lead = first_round < p.blocks_per_rank ? first_round : p.blocks_per_rank;
    }
  }
  // the entry barrier of CTA i uses block slot (barrier_block_base + i): it must stay inside the block-slot region
  if (comm && ((size_t)a.barrier_block_base + grid) * a.world_size > kBlockSlots) return cudaErrorInvalidValue;
  // split-K tail: only when the last wave fills less than half of the pairs
  p.tail_tiles = 0;
  p.tail_splits = 1;
  const int rem = total_tiles % pairs;
  const int k_blocks = (a.K * es + 127) / 128;                    // one K block = 128 bytes of a row
  if (a.tail_scratch != nullptr && !swiglu && rem > 0 && rem * 2 <= pairs) {
    int splits = pairs / rem;
    splits = splits >= 8 ? 8 : (splits >= 4 ? 4 : 2);
    // every part reduces BN / splits columns in vectors of 8
    while (splits > 1 && bn % (8 * splits) != 0) splits >>= 1;
    const size_t need = (size_t)rem * splits * 2 * kBM * bn * sizeof(float);
    if (splits >= 2 && k_blocks >= 2 * splits && need <= a.tail_scratch_bytes && (size_t)rem * 2 <= a.tail_counter_slots) {
      p.tail_tiles = rem;
      p.tail_splits = splits;
      p.tail_scratch = static_cast<float*>(a.tail_scratch);
      p.tail_counters = a.tail_counters;
      cudaError_t me = cudaMemsetAsync(a.tail_counters, 0, sizeof(uint32_t) * rem * 2, stream);
      if (me != cudaSuccess) return (int)me;
    }
  }
  if (swiglu) return launch_pair_variant<256, 6, false, true>(ta_shard, ta_out, tb, tc, p, grid, stream);
  if (fp8) {
    switch (bn) {
      case 128: return launch_pair_variant<128, 8, true>(ta_shard, ta_out, tb, tc, p, grid, stream);
      case 192: return launch_pair_variant<192, 7, true>(ta_shard, ta_out, tb, tc, p, grid, stream);
      case 224: return launch_pair_variant<224, 7, true>(ta_shard, ta_out, tb, tc, p, grid, stream);
      default:  return launch_pair_variant<256, 6, true>(ta_shard, ta_out, tb, tc, p, grid, stream);
    }
  }
  switch (bn) {
    case 128: return launch_pair_variant<128, 8, false>(ta_shard, ta_out, tb, tc, p, grid, stream);
    case 192: return launch_pair_variant<192, 6, false>(ta_shard, ta_out, tb, tc, p, grid, stream);
    case 224: return launch_pair_variant<224, 7, false>(ta_shard, ta_out, tb, tc, p, grid, stream);
    default:  return launch_pair_variant<256, 6, false>(ta_shard, ta_out, tb, tc, p, grid, stream);
  }
}

}  // namespace smr
