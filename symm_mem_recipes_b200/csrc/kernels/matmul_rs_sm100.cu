// Fused GEMM + reduce-scatter for sm_100a (row-parallel linear layer, prefill):
//     out_r[M/WS, N] = sum over ranks s of ( A_s[M, K_s] * B_s[N, K_s]^T )[rows of rank r]
// No upstream counterpart (the upstream package has the all-gather half only).
//
//  * The GEMM is the tcgen05 / TMEM pipeline of ag_matmul_sm100.cu (TMA
//    producer warp, MMA warp, four epilogue warps, two TMEM accumulators).
//  * Tiles are visited by destination rank: rank+1 first, ..., own rows last,
//    so the links are busy from the first tile and nothing waits on the wire
//    at the end.
//  * Epilogue: accumulator -> bf16 -> a shared-memory staging strip of 64
//    columns -> one 128-byte bulk store (cp.async.bulk, shared -> global) per
//    row into the DESTINATION rank's inbox [src][row][N].  Full-row packets
//    cross NVLink, not 16-byte fragments.  When a tile's stores have completed
//    the destination's arrival counter for that tile gets +1 (red.release.sys).
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
constexpr int kStripCols = 64;                         // columns staged at a time
constexpr uint32_t kStripPitch = kStripCols * 2 + 16;  // bytes; +16 spreads rows over banks

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
};

struct Smem {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = kBN * kBK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kRingBytes = kStageBytes * kStages;
  static constexpr uint32_t kStripOffset = kRingBytes;
  static constexpr uint32_t kStripBytes = kBM * kStripPitch;
  static constexpr uint32_t kBarOffset = kStripOffset + kStripBytes;
  static constexpr uint32_t kNumBars = 2 * kStages + 4;
  static constexpr uint32_t kMiscOffset = kBarOffset + 8 * kNumBars;
  static constexpr uint32_t kTotal = kMiscOffset + 16 + 1024;
};
static_assert(Smem::kTotal <= 232448, "shared memory budget exceeded");

// tile index -> destination rank, 128-row block inside the destination, N tile
__device__ __forceinline__ void tile_coords(const RsParams& p, int t, int& dest, int& mb, int& ni) {
  const int per_dest = p.blocks_per_rank * p.n_tiles_n;
  int step = t / per_dest, rem = t - step * per_dest;
  dest = p.rank + 1 + step;
  if (dest >= p.world_size) dest -= p.world_size;
  mb = rem / p.n_tiles_n;
  ni = rem - mb * p.n_tiles_n;
}

__global__ void __launch_bounds__(kThreads, 1)
matmul_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const RsParams p) {
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
  // every rank has entered this call: its reduce of the previous call is done
  bool entered = blockwise_barrier(p.pads, 1024u + blockIdx.x, p.rank, p.world_size, p.timeout_ns,
                                   p.status, kWhereRsEntry);
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
    // ---------------- epilogue: TMEM -> bf16 strip -> bulk stores to the destination ----------------
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                  // row of the tile owned by this thread
    uint8_t* my_strip = strip + (size_t)r * kStripPitch;
    uint32_t acc = 0, acc_phase = 0;
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
      // inbox of the destination: [src = this rank][row in destination][N]
      __nv_bfloat16* inbox = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(p.buffers[dest]) + p.inbox_offset);
      __nv_bfloat16* drow = inbox + ((size_t)p.rank * rows_per_rank + (size_t)mb * kBM + r) * p.N;
#pragma unroll 1
      for (int sidx = 0; sidx < kBN / kStripCols; ++sidx) {
        const int col0 = ni * kBN + sidx * kStripCols;
        if (col0 >= p.N) break;                          // uniform over the CTA
        bulk_wait_group_read<0>();                       // my previous row store has left the strip
#pragma unroll
        for (int h = 0; h < kStripCols / 32; ++h) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + (uint32_t)(sidx * kStripCols + h * 32), v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            Vec16 o;
            o.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
            *reinterpret_cast<Vec16*>(my_strip + h * 64 + q * 16) = o;
          }
        }
        fence_proxy_async();                             // strip written by this thread, read by the bulk store
        int cols = p.N - col0;
        if (cols > kStripCols) cols = kStripCols;
        bulk_store(drow + col0, my_strip, (uint32_t)cols * 2u);
        bulk_commit_group();
      }
      // the accumulator has been read: hand it back before waiting on the wire
      tcgen05_fence_before_thread_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      bulk_wait_group<0>();                              // my rows have been written at the destination
      asm volatile("bar.sync 1, 128;" ::: "memory");     // the four epilogue warps
      if (warp == 2 && lane == 0) {
        uint32_t* counters = p.pads[dest] + kFlagSlotsBase + 2;
        fence_proxy_async();
        red_add_release_sys(&counters[mb * p.n_tiles_n + ni], 1u);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    bulk_wait_group<0>();
  }

  // ---------------- GEMM teardown ----------------
  if (__any_sync(0xffffffffu, failed)) {
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  tcgen05_fence_before_thread_sync();
  failed = __syncthreads_or(failed) != 0;
  tcgen05_fence_after_thread_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);

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
      const int n0 = ni * kBN;
      const int vec_per_row = (min(kBN, p.N - n0)) / 8;
      for (int idx = threadIdx.x; idx < kBM * vec_per_row; idx += kThreads) {
        const int row = mb * kBM + idx / vec_per_row, cv = idx % vec_per_row;
        const size_t off = (size_t)row * p.N + n0 + cv * 8;
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int src = 0; src < p.world_size; ++src) {
          Vec16 v = ld_16_stream(inbox + (size_t)src * rows_per_rank * p.N + off);
          s[0] += bf16lo_to_f32(v.x); s[1] += bf16hi_to_f32(v.x);
          s[2] += bf16lo_to_f32(v.y); s[3] += bf16hi_to_f32(v.y);
          s[4] += bf16lo_to_f32(v.z); s[5] += bf16hi_to_f32(v.z);
          s[6] += bf16lo_to_f32(v.w); s[7] += bf16hi_to_f32(v.w);
        }
        Vec16 o;
        o.x = pack_bf16x2(s[0], s[1]);
        o.y = pack_bf16x2(s[2], s[3]);
        o.z = pack_bf16x2(s[4], s[5]);
        o.w = pack_bf16x2(s[6], s[7]);
        st_16(p.out + off, o);
      }
    }
  }

  // ---------------- the last CTA to finish publishes this call's number ----------------
  __syncthreads();
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
  CUtensorMap ta, tb;
  if (make_tmap(&ta, a.a, (uint64_t)a.M, (uint64_t)a.K, kBM)) return cudaErrorInvalidValue;
  if (make_tmap(&tb, a.b, (uint64_t)a.N, (uint64_t)a.K, kBN)) return cudaErrorInvalidValue;
  int total_tiles = ws * p.blocks_per_rank * p.n_tiles_n;
  int grid = a.num_sms < total_tiles ? a.num_sms : total_tiles;
  if (grid < 1 || (uint32_t)(1024 + grid) * (uint32_t)ws > kBlockSlots) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(matmul_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)Smem::kTotal);
  if (e != cudaSuccess) return (int)e;
  matmul_rs_kernel<<<grid, kThreads, Smem::kTotal, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

}  // namespace smr
