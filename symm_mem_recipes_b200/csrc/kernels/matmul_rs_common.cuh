// Pieces of the fused GEMM + reduce-scatter kernel that its launcher and the host-side
// schedule checks share: tile geometry, the strip-major inbox layout, the
// kernel parameters, the ordered reduction of arrived partials and the
// tensor-map builder.
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
namespace rs {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr int kStripCols = 64;                         // columns staged at a time (128 bytes: one swizzle row)
constexpr uint32_t kStripBytesOne = kBM * kStripCols * 2;   // 16 KB
constexpr int kStripsPerTile = kBN / kStripCols;       // 4

// Byte offset of a strip inside an inbox: [src][row block][N tile][strip] x 16 KB
__host__ __device__ __forceinline__ size_t strip_offset(int src, int mb, int ni, int sidx, int blocks_per_rank,
                                                        int n_tiles_n) {
  return ((((size_t)src * blocks_per_rank + mb) * n_tiles_n + ni) * kStripsPerTile + sidx) * kStripBytesOne;
}

struct RsParams {
  int M, N, K;
  int rank, world_size;
  int blocks_per_rank;       // 128-row blocks per destination
  int n_tiles_n;
  int panel_w;               // N tiles per column panel of the tile order (n_tiles_n: one panel)
  void* const* buffers;      // workspace payload base of every rank
  size_t inbox_offset;       // inbox [WS src][M/WS][N] bf16 inside the payload
  uint32_t* const* pads;
  uint32_t* local_pad;
  __nv_bfloat16* out;        // [M/WS, N]
  uint64_t timeout_ns;
  Status* status;
  uint64_t* trace;           // optional [grid][4] %globaltimer stamps: start, entered, GEMM done, reduced
  // all-reduce form only: the reduced rows are broadcast into a symmetric [M, N] output on every rank
  void* const* ar_peers;     // payload base of the output allocation on every rank
  void* ar_mc;               // its multicast base, or nullptr (then plain stores to every peer)
  size_t ar_offset;          // offset of the output tensor inside that payload
};

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Epilogue, one thread per row of the tile: the row's 64 accumulator columns of a strip (v0: columns
// 0..31, v1: 32..63) become bf16 and go to row `r` of the strip buffer, whose 16-byte chunks are
// XOR-swizzled by row so that the 32 lanes of a warp do not collide on shared-memory banks.
__device__ __forceinline__ void strip_row_to_smem(uint8_t* buf, int r, const uint32_t (&v0)[32],
                                                  const uint32_t (&v1)[32]) {
  uint8_t* row = buf + (size_t)r * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {                    // 16-byte chunk c of the row
    const uint32_t* v = c < 4 ? &v0[c * 8] : &v1[(c - 4) * 8];
    Vec16 o;
    o.x = pack_bf16x2(__uint_as_float(v[0]), __uint_as_float(v[1]));
    o.y = pack_bf16x2(__uint_as_float(v[2]), __uint_as_float(v[3]));
    o.z = pack_bf16x2(__uint_as_float(v[4]), __uint_as_float(v[5]));
    o.w = pack_bf16x2(__uint_as_float(v[6]), __uint_as_float(v[7]));
    *reinterpret_cast<Vec16*>(row + ((c ^ (r & 7)) << 4)) = o;
  }
}

// Thread-store epilogue: the 128 epilogue threads copy a finished 16 KB strip from shared memory to
// `dst` (a peer's inbox) with 16-byte loads and stores, 512 contiguous bytes per warp instruction.
__device__ __forceinline__ void strip_copy_out(char* dst, const uint8_t* buf, int etid) {
#pragma unroll
  for (int j = 0; j < (int)(kStripBytesOne / 16 / 128); ++j) {
    const int idx = etid + j * 128;                // 16-byte vector of the strip
    st_16(dst + (size_t)idx * 16, *reinterpret_cast<const Vec16*>(buf + (size_t)idx * 16));
  }
}

// CTA-pair kernel: entry `rb` of the list of 128-row blocks in visiting order (destination rank+1
// first, own rows last) -> destination rank and row block inside it.  CTA c of the pair working on
// tile t handles entry 2 * (t / n_tiles_n) + c.
__host__ __device__ __forceinline__ void row_block_coords(const RsParams& p, int rb, int& dest, int& mb) {
  const int step = rb / p.blocks_per_rank;
  mb = rb - step * p.blocks_per_rank;
  dest = p.rank + 1 + step;
  if (dest >= p.world_size) dest -= p.world_size;
}

// Epilogue of a tile of the rank's own rows.  Each 64-column strip of the accumulator is staged in
// shared memory as bf16 exactly as if it were to be shipped (so the own partial is rounded like the
// peers' partials that crossed the wire); then the 128 epilogue threads walk the strip in the order it
// has in memory, 16 bytes per thread and 512 contiguous bytes per warp instruction: the strips of the
// peers in the inbox have the same layout, so their loads are fully coalesced, and a warp's stores
// fill four whole 128-byte rows of the output.  The sum is fp32, in rank order from +0, rounded once.
// The peers' vectors of the next batch (JB vectors per peer) are loaded before the current batch is
// added, also across the TMEM read and staging of the next strip: 2 x (WS - 1) x JB 16-byte loads in
// flight per thread.  WS = 0: generic loop for other world sizes.
// kAllReduce: instead of the local [M/WS, N] output, the row goes to rows [rank * M/WS + ...] of
// the symmetric [M, N] output of EVERY rank (one multimem.st per 16 bytes, or WS stores).
template <int WS, bool kAllReduce = false>
__device__ __forceinline__ void reduce_own_tile(const RsParams& p, uint32_t taddr, int mb, int ni, int r, int etid,
                                                uint8_t* strip, int n_strip_bufs, uint32_t& strip_ctr) {
  constexpr int NP = WS > 0 ? WS - 1 : 1;                   // peers
  constexpr int JB = WS == 0 ? 4 : (WS <= 2 ? 8 : (WS <= 4 ? 4 : 2));   // 16-byte vectors per thread and batch
  constexpr int NB = 8 / JB;                                // batches per strip (a strip is 8 vectors per thread)
  constexpr size_t kVecStep = 128 * 16;                     // distance between a thread's vectors j and j + 1
  const int n0 = ni * kBN;
  const size_t src_stride = (size_t)p.blocks_per_rank * p.n_tiles_n * kStripsPerTile * kStripBytesOne;
  const char* tile_base = static_cast<const char*>(p.buffers[p.rank]) + p.inbox_offset +
                          strip_offset(0, mb, ni, 0, p.blocks_per_rank, p.n_tiles_n) + (size_t)etid * 16;
  auto add_vec = [](float (&s)[8], const Vec16& w) {
    s[0] += bf16lo_to_f32(w.x); s[1] += bf16hi_to_f32(w.x);
    s[2] += bf16lo_to_f32(w.y); s[3] += bf16hi_to_f32(w.y);
    s[4] += bf16lo_to_f32(w.z); s[5] += bf16hi_to_f32(w.z);
    s[6] += bf16lo_to_f32(w.w); s[7] += bf16hi_to_f32(w.w);
  };
  auto write_out = [&](int idx, int col0, const float (&s)[8]) {
    const int row = idx >> 3;
    const int col = col0 + (((idx & 7) ^ (row & 7)) << 3);  // undo the strip's swizzle
    if (col >= p.N) return;                                 // N % 8 == 0
    Vec16 o;
    o.x = pack_bf16x2(s[0], s[1]); o.y = pack_bf16x2(s[2], s[3]);
    o.z = pack_bf16x2(s[4], s[5]); o.w = pack_bf16x2(s[6], s[7]);
    const size_t out_row = (size_t)(mb * kBM + row);
    if constexpr (kAllReduce) {
      const size_t off = p.ar_offset +
                         (((size_t)p.rank * p.blocks_per_rank * kBM + out_row) * p.N + col) * sizeof(__nv_bfloat16);
      if (p.ar_mc != nullptr) {
        multimem_st_16(static_cast<char*>(p.ar_mc) + off, o);
      } else {
        for (int s2 = 1; s2 <= p.world_size; ++s2) {        // own copy last
          int peer = p.rank + s2;
          if (peer >= p.world_size) peer -= p.world_size;
          st_16(static_cast<char*>(p.ar_peers[peer]) + off, o);
        }
      }
    } else {
      st_16(p.out + out_row * p.N + col, o);
    }
  };
  auto load_batch = [&](Vec16 (&v)[NP][JB], int sidx, int b) {
#pragma unroll
    for (int q = 0; q < NP; ++q) {
      const int src = q < p.rank ? q : q + 1;
      const char* base = tile_base + (size_t)src * src_stride + (size_t)sidx * kStripBytesOne + (size_t)(b * JB) * kVecStep;
#pragma unroll
      for (int j = 0; j < JB; ++j) v[q][j] = ld_16_stream(base + (size_t)j * kVecStep);
    }
  };

  Vec16 nxt[NP][JB];
  if constexpr (WS > 0) load_batch(nxt, 0, 0);
#pragma unroll 1
  for (int sidx = 0; sidx < kStripsPerTile; ++sidx) {
    const int col0 = n0 + sidx * kStripCols;
    if (col0 >= p.N) break;                                 // uniform over the CTA
    uint8_t* buf = strip + (size_t)(strip_ctr % (uint32_t)n_strip_bufs) * kStripBytesOne;
    {
      uint32_t v0[32], v1[32];
      tmem_ld_32x32b_x32(taddr + (uint32_t)(sidx * kStripCols), v0);
      tmem_ld_32x32b_x32(taddr + (uint32_t)(sidx * kStripCols + 32), v1);
      tmem_ld_wait();
      epilogue_sync();                                      // nobody reads the buffer we are about to fill any more
      strip_row_to_smem(buf, r, v0, v1);
    }
    epilogue_sync();                                        // the own strip is complete in shared memory
    ++strip_ctr;
    const bool more = sidx + 1 < kStripsPerTile && col0 + kStripCols < p.N;
    if constexpr (WS == 0) {
#pragma unroll 1
      for (int b = 0; b < NB; ++b) {
        float s[JB][8];
#pragma unroll
        for (int j = 0; j < JB; ++j)
#pragma unroll
          for (int e = 0; e < 8; ++e) s[j][e] = 0.f;
        for (int src = 0; src < p.world_size; ++src) {
#pragma unroll
          for (int j = 0; j < JB; ++j) {
            const size_t voff = (size_t)(b * JB + j) * kVecStep;
            const Vec16 w = src == p.rank
                                ? *reinterpret_cast<const Vec16*>(buf + (size_t)etid * 16 + voff)
                                : ld_16_stream(tile_base + (size_t)src * src_stride + (size_t)sidx * kStripBytesOne + voff);
            add_vec(s[j], w);
          }
        }
#pragma unroll
        for (int j = 0; j < JB; ++j) write_out(etid + (b * JB + j) * 128, col0, s[j]);
      }
    } else {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        Vec16 cur[NP][JB];
#pragma unroll
        for (int q = 0; q < NP; ++q)
#pragma unroll
          for (int j = 0; j < JB; ++j) cur[q][j] = nxt[q][j];
        if (b + 1 < NB) load_batch(nxt, sidx, b + 1);
        else if (more) load_batch(nxt, sidx + 1, 0);
#pragma unroll
        for (int j = 0; j < JB; ++j) {
          const int idx = etid + (b * JB + j) * 128;
          const Vec16 own = *reinterpret_cast<const Vec16*>(buf + (size_t)idx * 16);
          float s[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) s[e] = 0.f;
#pragma unroll
          for (int q = 0; q < NP; ++q) {
            if (q == p.rank) add_vec(s, own);
            add_vec(s, cur[q][j]);
          }
          if (p.rank == NP) add_vec(s, own);
          write_out(idx, col0, s);
        }
      }
    }
  }
}

inline int make_tmap(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
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

}  // namespace rs
}  // namespace smr
