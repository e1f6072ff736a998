// Fused GEMM + reduce-scatter for sm_100a (row-parallel linear layer, prefill):
//     out_r[M/WS, N] = sum over ranks s of ( A_s[M, K_s] * B_s[N, K_s]^T )[rows of rank r]
// No upstream counterpart (the upstream package has the all-gather half only).
//
//  * The GEMM is the tcgen05 / TMEM pipeline of ag_matmul_sm100.cu (TMA
//    producer warp, MMA warp, four epilogue warps, two TMEM accumulators).
//  * Tiles are visited by destination rank: rank+1 first, ..., own rows last,
//    so the links are busy from the first tile and nothing waits on the wire
//    at the end.
//  * Epilogue: accumulator -> bf16 -> a swizzled shared-memory strip of
//    [128 rows x 64 columns] -> ONE TMA tensor store (cp.async.bulk.tensor,
//    shared -> global) into the DESTINATION rank's inbox [src][row][N], through
//    a tensor map built over that peer's memory.  Two strips alternate, so the
//    next strip is converted while the previous one is on the wire, and whole
//    128-byte lines cross NVLink.  A tile's arrival counter on the destination
//    gets +1 (red.release.sys) once the tile's stores have completed, which is
//    checked one tile later so the epilogue never waits for the wire.
//  * Reduce: after its GEMM tiles every CTA takes output tiles of its own rank,
//    waits (bounded) until WS partials have arrived, sums them in rank order in
//    fp32 and writes bf16.  All ranks thus produce identical bits.
//  * An entry barrier over the signal pad proves that every rank has finished
//    reducing the previous call before its inbox is overwritten.  Counters
//    count calls (epoch word in the pad), so nothing is reset between calls.
#include <cuda.h>
#include <cuda_runtime.h>

#include "../device/barrier.cuh"
#include "../device/mbarrier.cuh"
#include "../device/tcgen05.cuh"
#include "../device/tma.cuh"
#include "../device/vec.cuh"
#include "../symm/driver_api.h"
#include "launch.h"

namespace smr {

namespace {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr int kStripCols = 64;                         // columns staged at a time (128 bytes: one swizzle row)
constexpr uint32_t kStripBytesOne = kBM * kStripCols * 2;   // 16 KB
constexpr int kMaxWorld = 8;

struct InboxMaps {
  CUtensorMap m[kMaxWorld];   // m[d]: this rank's slice [M/WS, N] of rank d's inbox
};

struct RsParams {
  int M, N, K;
  int rank, world_size;
  int blocks_per_rank;       // 128-row blocks per destination
  int n_tiles_n;
  void* const* buffers;      // workspace payload base of every rank
  size_t inbox_offset;       // inbox [WS src][M/WS][N] bf16 inside the payload
  uint32_t* const* pads;
  uint32_t* local_pad;
  __nv_bfloat16* out;        // [M/WS, N]
  uint64_t timeout_ns;
  Status* status;
  uint64_t* trace;           // optional [grid][4] %globaltimer stamps: start, entered, GEMM done, reduced
};

struct Smem {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = kBN * kBK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kRingBytes = kStageBytes * kStages;
  static constexpr uint32_t kStripOffset = kRingBytes;
  static constexpr uint32_t kStripBytes = 2 * kStripBytesOne;   // two strips alternate
  static constexpr uint32_t kBarOffset = kStripOffset + kStripBytes;
  static constexpr uint32_t kNumBars = 2 * kStages + 4;
  static constexpr uint32_t kMiscOffset = kBarOffset + 8 * kNumBars;
  static constexpr uint32_t kTotal = kMiscOffset + 16 + 1024;
};
static_assert(Smem::kTotal <= 232448, "shared memory budget exceeded");

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// 2-D tile shared -> global through a tensor map (which may describe a peer GPU's memory)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}

// tile index -> destination rank, 128-row block inside the destination, N tile
__device__ __forceinline__ void tile_coords(const RsParams& p, int t, int& dest, int& mb, int& ni) {
  const int per_dest = p.blocks_per_rank * p.n_tiles_n;
  int step = t / per_dest, rem = t - step * per_dest;
  dest = p.rank + 1 + step;
  if (dest >= p.world_size) dest -= p.world_size;
  mb = rem / p.n_tiles_n;
  ni = rem - mb * p.n_tiles_n;
}

// Ordered fp32 sum of the WS partials of one [128 x 256] output tile.  16
// independent 16-byte loads are in flight per thread (the phase is bound by
// memory latency otherwise): 16 / WS output vectors at a time.  WS = 0 selects
// the generic loop for other world sizes.
template <int WS>
__device__ __forceinline__ void reduce_tile(const RsParams& p, const __nv_bfloat16* inbox, int mb, int ni,
                                            int rows_per_rank) {
  const int n0 = ni * kBN;
  const int vec_per_row = (min(kBN, p.N - n0)) / 8;
  const int total = kBM * vec_per_row;
  const size_t src_stride = (size_t)rows_per_rank * p.N;
  if constexpr (WS == 0) {
    for (int idx = threadIdx.x; idx < total; idx += kThreads) {
      const int row = mb * kBM + idx / vec_per_row, cv = idx % vec_per_row;
      const size_t off = (size_t)row * p.N + n0 + cv * 8;
      float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int src = 0; src < p.world_size; ++src) {
        Vec16 v = ld_16_stream(inbox + (size_t)src * src_stride + off);
        s[0] += bf16lo_to_f32(v.x); s[1] += bf16hi_to_f32(v.x);
        s[2] += bf16lo_to_f32(v.y); s[3] += bf16hi_to_f32(v.y);
        s[4] += bf16lo_to_f32(v.z); s[5] += bf16hi_to_f32(v.z);
        s[6] += bf16lo_to_f32(v.w); s[7] += bf16hi_to_f32(v.w);
      }
      Vec16 o;
      o.x = pack_bf16x2(s[0], s[1]); o.y = pack_bf16x2(s[2], s[3]);
      o.z = pack_bf16x2(s[4], s[5]); o.w = pack_bf16x2(s[6], s[7]);
      st_16(p.out + off, o);
    }
  } else {
    constexpr int U = 16 / WS;
    for (int idx0 = threadIdx.x; idx0 < total; idx0 += kThreads * U) {
      Vec16 v[U][WS];
      size_t off[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = idx0 + u * kThreads;
        const int row = mb * kBM + idx / vec_per_row, cv = idx % vec_per_row;
        off[u] = (size_t)row * p.N + n0 + cv * 8;
        if (idx < total) {
#pragma unroll
          for (int src = 0; src < WS; ++src) v[u][src] = ld_16_stream(inbox + (size_t)src * src_stride + off[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (idx0 + u * kThreads >= total) break;
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int src = 0; src < WS; ++src) {
          const Vec16& w = v[u][src];
          s[0] += bf16lo_to_f32(w.x); s[1] += bf16hi_to_f32(w.x);
          s[2] += bf16lo_to_f32(w.y); s[3] += bf16hi_to_f32(w.y);
          s[4] += bf16lo_to_f32(w.z); s[5] += bf16hi_to_f32(w.z);
          s[6] += bf16lo_to_f32(w.w); s[7] += bf16hi_to_f32(w.w);
        }
        Vec16 o;
        o.x = pack_bf16x2(s[0], s[1]); o.y = pack_bf16x2(s[2], s[3]);
        o.z = pack_bf16x2(s[4], s[5]); o.w = pack_bf16x2(s[6], s[7]);
        st_16(p.out + off[u], o);
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
matmul_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ InboxMaps inbox_maps, const RsParams p) {
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
        if (etid == 0) bulk_wait_group_read<1>();
        epilogue_sync();
        uint8_t* buf = strip + (size_t)(strip_ctr & 1u) * kStripBytesOne;
        uint8_t* row = buf + (size_t)r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {                    // 16-byte chunk c of the row, 128-byte swizzle
          const uint32_t* v = c < 4 ? &v0[c * 8] : &v1[(c - 4) * 8];
          Vec16 o;
          o.x = pack_bf16x2(__uint_as_float(v[0]), __uint_as_float(v[1]));
          o.y = pack_bf16x2(__uint_as_float(v[2]), __uint_as_float(v[3]));
          o.z = pack_bf16x2(__uint_as_float(v[4]), __uint_as_float(v[5]));
          o.w = pack_bf16x2(__uint_as_float(v[6]), __uint_as_float(v[7]));
          *reinterpret_cast<Vec16*>(row + ((c ^ (r & 7)) << 4)) = o;
        }
        fence_proxy_async();                             // generic writes to smem, async-proxy read
        epilogue_sync();
        if (etid == 0) {
          tma_store_2d(&inbox_maps.m[dest], buf, col0, mb * kBM);
          bulk_commit_group();
        }
        ++strip_ctr;
        ++strips;
      }
      // the accumulator has been read: hand it back
      tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (etid == 0) {
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
    const __nv_bfloat16* inbox = reinterpret_cast<const __nv_bfloat16*>(
        static_cast<const char*>(p.buffers[p.rank]) + p.inbox_offset);
    for (int t = blockIdx.x; t < my_tiles; t += gridDim.x) {
      const int mb = t / p.n_tiles_n, ni = t - mb * p.n_tiles_n;
      bool ok = true;
      if (threadIdx.x == 0 && !wait_ge_acquire_sys(&my_counters[t], target, p.timeout_ns)) {
        report_status(p.status, kTimeoutFlag, p.rank, blockIdx.x, t, kWhereRsArrive, target);
        ok = false;
      }
      if (!__syncthreads_and(ok)) break;
      switch (p.world_size) {
        case 2: reduce_tile<2>(p, inbox, mb, ni, rows_per_rank); break;
        case 4: reduce_tile<4>(p, inbox, mb, ni, rows_per_rank); break;
        case 8: reduce_tile<8>(p, inbox, mb, ni, rows_per_rank); break;
        default: reduce_tile<0>(p, inbox, mb, ni, rows_per_rank); break;
      }
    }
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

int make_tmap(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  const DriverApi& d = DriverApi::get();
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = d.cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                                        dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// [rows, cols] bf16 destination with a [128 rows x 64 cols] swizzled box
int make_store_tmap(CUtensorMap* map, void* base, uint64_t rows, uint64_t cols) {
  const DriverApi& d = DriverApi::get();
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)kStripCols, (cuuint32_t)kBM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = d.cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1;
}

}  // namespace

size_t matmul_rs_workspace_bytes(int M, int N) { return (size_t)M * N * 2; }

int launch_matmul_reduce_scatter(const MatmulRsArgs& a, cudaStream_t stream) {
  const int ws = a.pv.world_size;
  if (a.M <= 0 || a.N % 8 != 0 || a.K % 8 != 0 || a.M % (ws * kBM) != 0) return cudaErrorInvalidValue;
  RsParams p{};
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.rank = a.pv.rank; p.world_size = ws;
  p.blocks_per_rank = a.M / ws / kBM;
  p.n_tiles_n = (a.N + kBN - 1) / kBN;
  if ((uint32_t)(p.blocks_per_rank * p.n_tiles_n) + 2u > kFlagSlots) return cudaErrorInvalidValue;
  p.buffers = a.pv.buffers;
  p.inbox_offset = a.inbox_offset;
  p.pads = a.pv.pads;
  p.local_pad = a.local_pad;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.timeout_ns = a.timeout_ns;
  p.status = a.status;
  p.trace = a.trace;
  CUtensorMap ta, tb;
  if (make_tmap(&ta, a.a, (uint64_t)a.M, (uint64_t)a.K, kBM)) return cudaErrorInvalidValue;
  if (make_tmap(&tb, a.b, (uint64_t)a.N, (uint64_t)a.K, kBN)) return cudaErrorInvalidValue;
  if (ws > kMaxWorld) return cudaErrorInvalidValue;
  InboxMaps maps{};
  const size_t slice_bytes = (size_t)(a.M / ws) * a.N * 2;
  for (int d = 0; d < ws; ++d) {
    // this rank's slice of rank d's inbox, as mapped into this process
    char* base = static_cast<char*>(a.peer_base[d]) + a.inbox_offset + (size_t)p.rank * slice_bytes;
    if (make_store_tmap(&maps.m[d], base, (uint64_t)(a.M / ws), (uint64_t)a.N)) return cudaErrorInvalidValue;
  }
  int total_tiles = ws * p.blocks_per_rank * p.n_tiles_n;
  int grid = a.num_sms < total_tiles ? a.num_sms : total_tiles;
  if (grid < 1 || (uint32_t)(1024 + grid) * (uint32_t)ws > kBlockSlots) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(matmul_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)Smem::kTotal);
  if (e != cudaSuccess) return (int)e;
  matmul_rs_kernel<<<grid, kThreads, Smem::kTotal, stream>>>(ta, tb, maps, p);
  return (int)cudaGetLastError();
}

}  // namespace smr
