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

// Epilogue of a tile of the rank's own rows, one thread per row `r` of the CTA's 128-row block:
// the row's accumulator (TMEM) and the peers' bf16 partials of the same row (strip-major inbox,
// 16-byte chunks XOR-swizzled by row) are added in rank order in fp32, the own value rounded to
// bf16 first as if it had crossed the wire, and the bf16 result is written row-major.  CH x 8
// columns at a time (32 up to four ranks, 16 at eight: the loaded vectors live in registers):
// (WS - 1) x CH independent 16-byte loads in flight per thread.  WS = 0: generic loop.
// kAllReduce: instead of the local [M/WS, N] output, the row goes to rows [rank * M/WS + ...] of
// the symmetric [M, N] output of EVERY rank (one multimem.st per 16 bytes, or WS stores).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

template <int WS, bool kAllReduce = false>
__device__ __forceinline__ void reduce_own_tile(const RsParams& p, uint32_t taddr, int mb, int ni, int r) {
  constexpr int CH = (WS == 0 || WS > 4) ? 2 : 4;           // 16-byte chunks (8 columns each) per step
  constexpr int COLS = CH * 8;
  const int n0 = ni * kBN;
  const char* inbox = static_cast<const char*>(p.buffers[p.rank]) + p.inbox_offset;
  const size_t src_stride = (size_t)p.blocks_per_rank * p.n_tiles_n * kStripsPerTile * kStripBytesOne;
  const int ws = WS == 0 ? p.world_size : WS;
  const size_t out_row = (size_t)(mb * kBM + r);
#pragma unroll 1
  for (int h = 0; h < kBN / COLS; ++h) {
    const int col0 = n0 + h * COLS;
    if (col0 >= p.N) break;                                 // uniform over the CTA
    const int sidx = (h * COLS) / kStripCols, c0 = ((h * COLS) % kStripCols) / 8;   // strip, first logical chunk in it
    uint32_t own[COLS];
    if constexpr (CH == 4) tmem_ld_32x32b_x32(taddr + (uint32_t)(h * COLS), own);
    else tmem_ld_32x32b_x16(taddr + (uint32_t)(h * COLS), own);
    const char* row_base = inbox + strip_offset(0, mb, ni, sidx, p.blocks_per_rank, p.n_tiles_n) + (size_t)r * 128;
    float s[COLS];
#pragma unroll
    for (int q = 0; q < COLS; ++q) s[q] = 0.f;
    auto add_vec = [&](int c, const Vec16& w) {
      s[c * 8 + 0] += bf16lo_to_f32(w.x); s[c * 8 + 1] += bf16hi_to_f32(w.x);
      s[c * 8 + 2] += bf16lo_to_f32(w.y); s[c * 8 + 3] += bf16hi_to_f32(w.y);
      s[c * 8 + 4] += bf16lo_to_f32(w.z); s[c * 8 + 5] += bf16hi_to_f32(w.z);
      s[c * 8 + 6] += bf16lo_to_f32(w.w); s[c * 8 + 7] += bf16hi_to_f32(w.w);
    };
    auto own_vec = [&](int c) {
      Vec16 w;
      w.x = pack_bf16x2(__uint_as_float(own[c * 8 + 0]), __uint_as_float(own[c * 8 + 1]));
      w.y = pack_bf16x2(__uint_as_float(own[c * 8 + 2]), __uint_as_float(own[c * 8 + 3]));
      w.z = pack_bf16x2(__uint_as_float(own[c * 8 + 4]), __uint_as_float(own[c * 8 + 5]));
      w.w = pack_bf16x2(__uint_as_float(own[c * 8 + 6]), __uint_as_float(own[c * 8 + 7]));
      return w;
    };
    if constexpr (WS == 0) {
      tmem_ld_wait();
      for (int src = 0; src < ws; ++src) {
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const Vec16 w = src == p.rank ? own_vec(c)
                                        : ld_16_stream(row_base + (size_t)src * src_stride + (((c0 + c) ^ (r & 7)) << 4));
          add_vec(c, w);
        }
      }
    } else {
      Vec16 v[WS][CH];
#pragma unroll
      for (int src = 0; src < WS; ++src) {
        if (src != p.rank) {
#pragma unroll
          for (int c = 0; c < CH; ++c)
            v[src][c] = ld_16_stream(row_base + (size_t)src * src_stride + (((c0 + c) ^ (r & 7)) << 4));
        }
      }
      tmem_ld_wait();
#pragma unroll
      for (int src = 0; src < WS; ++src) {
#pragma unroll
        for (int c = 0; c < CH; ++c) add_vec(c, src == p.rank ? own_vec(c) : v[src][c]);
      }
    }
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int col = col0 + c * 8;
      if (col >= p.N) break;                                // N % 8 == 0
      Vec16 o;
      o.x = pack_bf16x2(s[c * 8 + 0], s[c * 8 + 1]); o.y = pack_bf16x2(s[c * 8 + 2], s[c * 8 + 3]);
      o.z = pack_bf16x2(s[c * 8 + 4], s[c * 8 + 5]); o.w = pack_bf16x2(s[c * 8 + 6], s[c * 8 + 7]);
      if constexpr (kAllReduce) {
        const size_t off = p.ar_offset +
                           (((size_t)p.rank * p.blocks_per_rank * kBM + out_row) * p.N + col) * sizeof(__nv_bfloat16);
        if (p.ar_mc != nullptr) {
          multimem_st_16(static_cast<char*>(p.ar_mc) + off, o);
        } else {
          for (int s2 = 1; s2 <= p.world_size; ++s2) {      // own copy last
            int peer = p.rank + s2;
            if (peer >= p.world_size) peer -= p.world_size;
            st_16(static_cast<char*>(p.ar_peers[peer]) + off, o);
          }
        }
      } else {
        st_16(p.out + out_row * p.N + col, o);
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
