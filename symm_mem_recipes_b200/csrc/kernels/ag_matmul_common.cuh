// Pieces of the all_gather_matmul kernel (ag_matmul_2cta_sm100.cu) that its launcher and the
// host-side schedule checks share: parameters, the M schedule, the epilogue-warp push of the
// own shard and the tensor-map builder.
//
// Upstream counterparts (symm_mem_recipes/triton_all_gather_matmul.py):
//   push_pieces + arrival counters   <->  all_gather_with_progress, :20-56 (copy
//                                         engine + cuStreamWriteValue32 per shard)
//   flag wait in the producer warp   <->  wait_signal, :72-95
//   scheduled_block                  <->  the rank pivot of pid_m, :157-163
//   make_tmap                        <->  create_2d_tma_descriptor + cache, :196-213, 255-286
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../device/barrier.cuh"
#include "../device/mbarrier.cuh"
#include "../device/multimem.cuh"
#include "../device/tcgen05.cuh"
#include "../device/tma.cuh"
#include "../device/vec.cuh"
#include "../symm/driver_api.h"
#include "launch.h"
#include "tile_order.h"

namespace smr {
namespace agmm {

constexpr int kBM = 128;
constexpr int kBK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192; // 6 warps
constexpr int kEpiWarp0 = 2;
constexpr uint32_t kTmemCols = 512;
// Push mode: a block's arrival counter grows by kArrivalUnits per call whatever the number of pieces
// (each piece adds kArrivalUnits / pieces), so calls with different piece counts can share an allocation.
constexpr uint32_t kArrivalUnits = 256;  // pieces: a power of two up to this

struct AgMatmulParams {
  __nv_bfloat16* c;      // [M, N]; one byte per element when elem_bytes == 1
  int M, N, K;
  int elem_bytes;        // 2 = bf16 in and out; 1 = fp8 e4m3 in and out
  int n_tiles_n;         // ceil(N / BN)
  int panel_w;           // N tiles per column panel of the tile order (n_tiles_n: one panel)
  int n_blocks_m;        // ceil(M / 128)
  // gather
  int rank, world_size;
  int blocks_per_rank;   // 128-row blocks per shard
  int mode;              // 0 none, 2 push
  int lead;              // own blocks scheduled before the first remote one
  int pieces;            // push: pieces per 128-row block (arrivals per block and call)
  int push_ahead;        // push: rounds of tiles by which the broadcast runs ahead of the first need (>= 1)
  uint32_t* flags;       // [n_blocks_m] arrival flags read by the GEMM CTAs (local memory)
  uint32_t flag_target;  // filled from the call number in the kernel
  uint32_t* header;      // push: [0] epoch, [1] CTAs done (local, in the a_out signal pad)
  const char* a_local;   // own shard
  void* const* aout_buffers;   // push: payload base of the a_out allocation on every rank
  void* aout_mc;         // push: multicast payload base of the a_out allocation, or nullptr
  size_t aout_offset;    // push: offset of a_out inside that payload
  char* a_out;           // local gathered A [M, K]
  uint32_t* const* pads; // signal pads (entry barrier of the push)
  uint32_t barrier_block_base;     // first blockwise-barrier slot id used by it
  uint64_t timeout_ns;
  Status* status;
  // split-K tail (2-CTA kernel): the tiles of the last, partly filled wave are cut along K
  int tail_tiles;        // tiles handled that way (0 = none); they are the last ones of the schedule
  int tail_splits;       // K parts per such tile (2, 4 or 8)
  float* tail_scratch;   // [tail_tiles][tail_splits][2 CTAs][128 x BN] fp32 partial accumulators
  uint32_t* tail_counters;   // [tail_tiles][2] arrivals, zeroed before the launch
  // optional per-CTA %globaltimer record (2-CTA kernel), kTraceSlots words per CTA; see ag_trace::
  uint64_t* trace;
};

// Per-CTA timing record of the CTA-pair kernel (nanoseconds of %globaltimer).  Absolute stamps
// and accumulated waiting times of each warp role, enough to tell where a fused call loses time
// against the GEMM alone.  Upstream has no counterpart (it reads kernel times from the profiler,
// symm_mem_recipes/utils.py:74-82).
namespace ag_trace {
constexpr int kStart = 0;          // stamp: kernel entry
constexpr int kEntered = 1;        // stamp: entry barrier of the push mode passed
constexpr int kFlagWait = 2;       // producer: total wait for arrival flags of remote blocks
constexpr int kPush = 3;           // epilogue warps: total time inside push_pieces
constexpr int kAccWait = 4;        // epilogue warps: total wait for a complete accumulator
constexpr int kTilesDone = 5;      // stamp: last tile stored
constexpr int kTmemWait = 6;       // MMA thread: total wait for a free accumulator
constexpr int kOperandWait = 7;    // MMA thread: total wait for operand stages
constexpr int kStageWait = 8;      // producer: total wait for free stages
constexpr int kEnd = 9;            // stamp: epilogue warps done (trailing pushes included)
constexpr int kFirstFlagWait = 10; // producer: wait for the first remote block
constexpr int kTiles = 11;         // units of work of this CTA
constexpr int kTraceSlots = 12;
}  // namespace ag_trace

// ---------------------------------------------------------------------------
// Push, run by the 128 epilogue threads of every GEMM CTA before their first
// tile: entry barrier, then pieces `cta, cta + n_ctas, ...` of the OWN shard
// are broadcast into every rank's a_out and the arrival counters bumped.
// `etid` is the thread's index among the 128; named barrier 1 joins them.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void epilogue_group_sync() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// Entry barrier of the push mode, among the CTAs with this index on every rank.
__device__ inline bool push_entry_barrier(const AgMatmulParams& p, int cta, int etid) {
  __shared__ int entry_ok;
  if (etid == 0) entry_ok = 1;
  epilogue_group_sync();
  if (etid < p.world_size) {
    if (!barrier_signal_wait(p.pads, (p.barrier_block_base + (uint32_t)cta) * (uint32_t)p.world_size,
                             p.rank, p.world_size, etid, p.timeout_ns, p.status,
                             p.barrier_block_base + (uint32_t)cta, kWhereCopierEntry))
      entry_ok = 0;
  }
  epilogue_group_sync();
  return entry_ok != 0;
}

// Broadcast this CTA's pieces `next, next + n_ctas, ...` while they are below
// `limit` (an index into the piece sequence of the shard).  Returns the first
// piece not pushed.
__device__ inline int push_pieces(const AgMatmulParams& p, int next, int n_ctas, int limit, int etid) {
  constexpr int U = 8;
  const size_t block_vecs = (size_t)kBM * p.K * p.elem_bytes / 16;
  const size_t piece_vecs = (block_vecs + p.pieces - 1) / p.pieces;
  int piece = next;
  for (; piece < limit; piece += n_ctas) {
    const int blk = piece / p.pieces, sub = piece - blk * p.pieces;
    const int gblk = p.rank * p.blocks_per_rank + blk;
    const size_t v0 = (size_t)sub * piece_vecs;
    const size_t v1 = v0 + piece_vecs < block_vecs ? v0 + piece_vecs : block_vecs;
    const Vec16* src = reinterpret_cast<const Vec16*>(p.a_local) + (size_t)blk * block_vecs;
    const size_t dst_off = p.aout_offset + (size_t)gblk * block_vecs * 16;
    if (p.aout_mc != nullptr) {
      Vec16* dst = reinterpret_cast<Vec16*>(static_cast<char*>(p.aout_mc) + dst_off);
      for (size_t i = v0 + etid; i < v1; i += (size_t)128 * U) {
        Vec16 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i + (size_t)u * 128 < v1) v[u] = ld_16_nc(src + i + (size_t)u * 128);
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i + (size_t)u * 128 < v1) multimem_st_16(dst + i + (size_t)u * 128, v[u]);
      }
    } else {
      for (size_t i = v0 + etid; i < v1; i += (size_t)128 * U) {
        Vec16 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i + (size_t)u * 128 < v1) v[u] = ld_16_nc(src + i + (size_t)u * 128);
        for (int s2 = 1; s2 <= p.world_size; ++s2) {      // own a_out last
          int peer = (p.rank + s2) % p.world_size;
          Vec16* dst = reinterpret_cast<Vec16*>(static_cast<char*>(p.aout_buffers[peer]) + dst_off);
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i + (size_t)u * 128 < v1) st_16(dst + i + (size_t)u * 128, v[u]);
        }
      }
    }
    epilogue_group_sync();   // the group's stores precede the releases below
    if (etid < p.world_size)
      red_add_release_sys(p.pads[etid] + kFlagSlotsBase + 2 + gblk, kArrivalUnits / (uint32_t)p.pieces);
  }
  return piece;
}

// Position `mi` of the M schedule -> 128-row block of the gathered A.
//   mi < lead                      own block mi
//   then groups k = 0 .. : block k of rank+1 .. rank+WS-1, then own block
//   lead + k while own blocks remain.
__host__ __device__ __forceinline__ int scheduled_block(const AgMatmulParams& p, int mi, bool& local) {
  if (p.mode == 0) {
    local = true;
    return mi;
  }
  const int ws = p.world_size, bpr = p.blocks_per_rank;
  int step, k;
  if (mi < p.lead) {
    step = 0; k = mi;
  } else {
    int q = mi - p.lead;
    const int full = bpr - p.lead;             // groups that still carry an own block
    if (q < full * ws) {
      int g = q / ws, s2 = q - g * ws;
      if (s2 < ws - 1) { step = s2 + 1; k = g; }
      else { step = 0; k = g + p.lead; }
    } else {
      q -= full * ws;
      int g = q / (ws - 1), s2 = q - g * (ws - 1);
      step = s2 + 1; k = full + g;
    }
  }
  int src = p.rank + step;
  if (src >= ws) src -= ws;
  local = (step == 0);
  return src * bpr + k;
}

// Pieces of the own shard that every rank must have pushed before any CTA may
// block on the tiles of rounds <= `round` (round j = tiles j*G .. (j+1)*G-1 of
// the static schedule): all pieces of the remote blocks those tiles read.
// `n_units` tiles run concurrently (CTAs, or CTA pairs); a tile covers
// `pos_per_tile` consecutive schedule positions (1, or 2 for a CTA pair).
__host__ __device__ __forceinline__ int pieces_needed_through_round(const AgMatmulParams& p, int round,
                                                           int n_units, int pos_per_tile = 1) {
  const int ws = p.world_size, bpr = p.blocks_per_rank;
  long long tiles = (long long)(round + 1) * n_units;
  // the first column panel walks every row block; later panels find them all arrived
  int mi_end = (int)((tiles + p.panel_w - 1) / p.panel_w) * pos_per_tile;       // positions touched: [0, mi_end)
  if (mi_end > p.n_blocks_m) mi_end = p.n_blocks_m;
  if (mi_end <= p.lead) return 0;
  int q = mi_end - 1 - p.lead;
  const int full = bpr - p.lead;
  int k_max = q < full * ws ? q / ws : full + (q - full * ws) / (ws - 1);
  if (k_max >= bpr) k_max = bpr - 1;
  return (k_max + 1) * p.pieces;
}

// Pieces of the own shard that should be on the wire once round `round` begins.  Never less
// than the schedule needs (`pieces_needed_through_round(round + 1)`: nobody can then block on a
// piece that a blocked CTA still holds); `push_ahead` > 1 asks for that many rounds of lookahead
// instead of one.  (Spreading the whole shard evenly over the first rounds of the kernel was
// measured too: 40-190 µs slower, eager stores compete with the GEMM's own loads.)
__host__ __device__ __forceinline__ int pieces_due(const AgMatmulParams& p, int round, int n_units,
                                                   int pos_per_tile, int all_pieces) {
  int due = pieces_needed_through_round(p, round + (p.push_ahead > 1 ? p.push_ahead : 1), n_units, pos_per_tile);
  return due < all_pieces ? due : all_pieces;
}

__host__ __device__ __forceinline__ void tile_coords(const AgMatmulParams& p, int n_rows, int t, int& row, int& ni) {
  panel_tile_coords(p.n_tiles_n, p.panel_w, n_rows, t, row, ni);
}

// The i-th piece of work of a CTA pair in the 2-CTA kernel: a whole tile, or
// one K part of a tile of the split-K tail.
struct PairWork {
  int tile;        // index into the tile schedule
  int kb0, kb1;    // K blocks [kb0, kb1)
  int part;        // -1 = whole tile, else the part's index
  int tail_idx;    // index of the tile among the tail tiles
};
__host__ __device__ __forceinline__ bool pair_work(const AgMatmulParams& p, int pair, int n_pairs,
                                                   int total_tiles, int k_blocks, int i, PairWork& w) {
  const int full_tiles = total_tiles - p.tail_tiles;
  const int t = pair + i * n_pairs;
  if (t < full_tiles) {
    w.tile = t; w.kb0 = 0; w.kb1 = k_blocks; w.part = -1; w.tail_idx = 0;
    return true;
  }
  // at most one unit of tail work per pair, right after its whole tiles
  const int first_tail_i = (full_tiles - pair + n_pairs - 1) / n_pairs;   // first i with t >= full_tiles
  if (p.tail_tiles == 0 || i != first_tail_i || pair >= p.tail_tiles * p.tail_splits) return false;
  const int per = (k_blocks + p.tail_splits - 1) / p.tail_splits;
  w.tail_idx = pair / p.tail_splits;
  w.part = pair - w.tail_idx * p.tail_splits;
  w.tile = full_tiles + w.tail_idx;
  w.kb0 = w.part * per;
  w.kb1 = w.kb0 + per < k_blocks ? w.kb0 + per : k_blocks;
  if (w.kb1 < w.kb0) w.kb1 = w.kb0;
  return true;
}

// row-major [rows, cols] of bf16 (or of 1-byte elements) with a box of
// `box_rows` rows x 128 bytes and the 128-byte swizzle
inline int make_tmap(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                     int elem_bytes = 2) {
  const DriverApi& d = DriverApi::get();
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (cuuint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = d.cuTensorMapEncodeTiled(map, dt, 2, const_cast<void*>(base),
                                        dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}


}  // namespace agmm
}  // namespace smr
