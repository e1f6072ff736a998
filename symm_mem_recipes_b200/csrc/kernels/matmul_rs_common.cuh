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

// Ordered fp32 sum of the WS partials of one [128 x 256] output tile, read from the
// strip-major inbox (un-doing the row XOR of the 16-byte chunks) and written row-major.
// 16 independent 16-byte loads are in flight per thread (the phase is bound by memory
// latency otherwise): 16 / WS output vectors at a time.  WS = 0: generic loop.
// kAllReduce: instead of the local [M/WS, N] output, the tile goes to rows
// [rank * M/WS + ...] of the symmetric [M, N] output of EVERY rank (one multimem.st, or WS stores).
template <int WS, bool kAllReduce = false>
__device__ __forceinline__ void reduce_tile(const RsParams& p, const char* inbox, int mb, int ni) {
  const int n0 = ni * kBN;
  const int strips = min(kStripsPerTile, (p.N - n0 + kStripCols - 1) / kStripCols);
  const int total = strips * kBM * 8;                       // 16-byte vectors of the tile
  const size_t src_stride = (size_t)p.blocks_per_rank * p.n_tiles_n * kStripsPerTile * kStripBytesOne;
  const char* tile_base = inbox + strip_offset(0, mb, ni, 0, p.blocks_per_rank, p.n_tiles_n);
  // vector idx -> (strip, row, chunk): consecutive idx walk a strip's bytes in order (coalesced)
  auto locate = [&](int idx, size_t& in_off, size_t& out_off, bool& in_range) {
    const int sidx = idx / (kBM * 8), rem = idx - sidx * (kBM * 8);
    const int row = rem >> 3, pos = rem & 7;                // pos: position inside the swizzled row
    const int c = pos ^ (row & 7);                          // logical 16-byte chunk
    in_off = (size_t)sidx * kStripBytesOne + (size_t)rem * 16;
    const int col = n0 + sidx * kStripCols + c * 8;
    in_range = col < p.N;
    out_off = (size_t)(mb * kBM + row) * p.N + col;
  };
  constexpr int U = WS == 0 ? 1 : 16 / WS;
  for (int idx0 = threadIdx.x; idx0 < total; idx0 += kThreads * U) {
    Vec16 v[U][WS == 0 ? 1 : WS];
    size_t out_off[U];
    bool live[U];
    float s[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int idx = idx0 + u * kThreads;
      size_t in_off = 0;
      live[u] = false;
      if (idx < total) locate(idx, in_off, out_off[u], live[u]);
#pragma unroll
      for (int q = 0; q < 8; ++q) s[u][q] = 0.f;
      if (live[u]) {
        if constexpr (WS == 0) {
          for (int src = 0; src < p.world_size; ++src) {
            const Vec16 w = ld_16_stream(tile_base + (size_t)src * src_stride + in_off);
            s[u][0] += bf16lo_to_f32(w.x); s[u][1] += bf16hi_to_f32(w.x);
            s[u][2] += bf16lo_to_f32(w.y); s[u][3] += bf16hi_to_f32(w.y);
            s[u][4] += bf16lo_to_f32(w.z); s[u][5] += bf16hi_to_f32(w.z);
            s[u][6] += bf16lo_to_f32(w.w); s[u][7] += bf16hi_to_f32(w.w);
          }
        } else {
#pragma unroll
          for (int src = 0; src < WS; ++src) v[u][src] = ld_16_stream(tile_base + (size_t)src * src_stride + in_off);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      if constexpr (WS != 0) {
#pragma unroll
        for (int src = 0; src < WS; ++src) {
          const Vec16& w = v[u][src];
          s[u][0] += bf16lo_to_f32(w.x); s[u][1] += bf16hi_to_f32(w.x);
          s[u][2] += bf16lo_to_f32(w.y); s[u][3] += bf16hi_to_f32(w.y);
          s[u][4] += bf16lo_to_f32(w.z); s[u][5] += bf16hi_to_f32(w.z);
          s[u][6] += bf16lo_to_f32(w.w); s[u][7] += bf16hi_to_f32(w.w);
        }
      }
      Vec16 o;
      o.x = pack_bf16x2(s[u][0], s[u][1]); o.y = pack_bf16x2(s[u][2], s[u][3]);
      o.z = pack_bf16x2(s[u][4], s[u][5]); o.w = pack_bf16x2(s[u][6], s[u][7]);
      if constexpr (kAllReduce) {
        const size_t off = p.ar_offset +
                           ((size_t)p.rank * p.blocks_per_rank * kBM * p.N + out_off[u]) * sizeof(__nv_bfloat16);
        if (p.ar_mc != nullptr) {
          multimem_st_16(static_cast<char*>(p.ar_mc) + off, o);
        } else {
          for (int s2 = 1; s2 <= p.world_size; ++s2) {            // own copy last
            int peer = p.rank + s2;
            if (peer >= p.world_size) peer -= p.world_size;
            st_16(static_cast<char*>(p.ar_peers[peer]) + off, o);
          }
        }
      } else {
        st_16(p.out + out_off[u], o);
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
