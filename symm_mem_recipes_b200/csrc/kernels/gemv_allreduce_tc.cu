// Fused GEMV + all-reduce on the tensor cores (tcgen05), for decode batches
// 1..16.  No upstream counterpart (upstream's only reduction is the one-shot
// all-reduce, symm_mem_recipes/triton_one_shot_all_reduce.py:59-93, whose
// rank-ordered sum this kernel keeps).  Same contract as gemv_allreduce.cu:
//     out[b, n] = sum over ranks r of  x_r[b, :] . W_r[:, n]
//
// The product is computed transposed ("swap A/B") so that the skinny batch
// becomes the MMA's N dimension (16) and 128 output columns fill its M:
//     D[128 n, 16 b] (TMEM, fp32) += W^T[128 n, 16 k] * x^T[16 k, 16 b]
// W is stored [K, N] with N contiguous, i.e. the A operand is "MN-major": TMA
// loads [64 k x 64 n] boxes with the 128-byte swizzle and the shared-memory
// descriptor says MN-major (8-row k groups 1024 B apart, 64-column n groups
// 8192 B apart).  x is the K-major B operand, one [16 x 64] box per k step.
// One thread streams the weights through an 8-stage TMA ring (144 KB in
// flight per SM) — the op is bound by HBM, the MMA work is negligible.  (A
// 12-stage ring was measured: 5-9 % faster where a CTA streams 2 MB (N 14336:
// 44.3 -> 41.9 µs) and about 1 µs slower on the short K ranges of the fused
// all-reduce shapes; it was not kept.)  The
// first ring of loads is issued before the CTA's set-up barrier, so the weight
// stream starts while tensor memory is still being allocated.
//
// Grid = (N / 128 column tiles) x (K splits), chosen to fill the SMs; the K
// splits of a tile form a thread-block CLUSTER.  Each CTA parks its fp32
// partial [16 b x 128 n] in its own shared memory, the cluster meets, and CTA
// kh sums the partials of its share of the tile's columns (128 / splits) over
// the cluster's shared memories (distributed shared memory, split order): the
// K reduction never touches global memory.  With one rank that sum is the
// result.  With several, the CTA pushes it into slot `rank` of every rank's
// inbox for those columns, raises the slot's flag (st.release.sys), waits
// (bounded) for the WS flags of its columns and adds the slots in rank order,
// so every rank produces the same bits.
//
// Nothing is reset between calls and the kernel can be replayed from a CUDA
// graph: inbox and flags are double-buffered by the parity of a call number,
// and every CTA keeps its own call counter in the workspace (read when it
// starts, written when it ends; all CTAs of all ranks make the same calls, so
// the counters agree without an atomic or a fence at the kernel's end).
//
// Tagged variant (kTagged, meant for batch <= 4): the sums travel as 8-byte
// words {fp32 value, call number}, the protocol of the low-latency all-reduce
// in all_reduce.cu.  No flag and no release fence (which has to wait for the
// acknowledgements of all pushes): the reducer polls the words themselves
// until they carry this call's number.  Twice the bytes on the wire, one
// NVLink crossing on the critical path instead of a crossing, a fence and a
// flag.
#include <cuda.h>
#include <cuda_runtime.h>

#include "../device/barrier.cuh"
#include "../device/mbarrier.cuh"
#include "../device/tcgen05.cuh"
#include "../device/tma.cuh"
#include "../device/vec.cuh"
#include "../symm/driver_api.h"
#include "launch.h"
#include "residency.h"

namespace smr {

namespace {

constexpr int kTileN = 128;      // output columns per CTA = MMA M
constexpr int kBatchN = 16;      // MMA N: the batch, zero-padded by TMA
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kStages = 8;
constexpr int kThreads = 192;
constexpr uint32_t kWBytes = 2 * 64 * kBK * 2;        // two [64 k x 64 n] boxes
constexpr uint32_t kXBytes = kBatchN * kBK * 2;
constexpr uint32_t kStageBytes = kWBytes + kXBytes;   // 18432 = 18 * 1024
constexpr uint32_t kRingBytes = kStageBytes * kStages;
constexpr uint32_t kBarOffset = kRingBytes;
constexpr uint32_t kNumBars = 2 * kStages + 1;
constexpr uint32_t kMiscOffset = kBarOffset + 8 * kNumBars;
constexpr uint32_t kSmemTotal = kMiscOffset + 16 + 1024;
constexpr int kFlagStride = 32;   // flag slots per tile (>= WS * splits)
constexpr uint32_t kTmemCols = 32;

struct GemvTcParams {
  __nv_bfloat16* out;     // [batch, N]
  int batch, K, N;
  int rank, world_size;
  int ksplit;             // K splits of a column tile = CTAs of a cluster
  void* const* buffers;   // workspace payload base of every rank
  size_t counters_offset; // [tiles * ksplit] u32: calls made so far, one counter per CTA
  size_t flags_offset;    // [2 parity][tiles][kFlagStride] u32, flag of (tile, kh, source rank) at kh * WS + rank
  size_t inbox_offset;    // [2 parity][WS][16][N] fp32 (tagged: 8-byte words {fp32, call number})
  int tiles;
  uint64_t timeout_ns;
  Status* status;
};

// MN-major, 128-byte swizzle: 8-row k groups 1024 B apart (SBO), 64-element
// n groups 8192 B apart (LBO).
__device__ __forceinline__ uint64_t umma_smem_desc_mn_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(8192u >> 4) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1u << 46;
  d |= (uint64_t)2u << 61;
  return d;
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void group_sync_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Cluster-wide barrier (every thread of every CTA of the cluster) and a 16-byte load from the
// shared memory of CTA `cta` of the cluster at the same offset as `local_smem_addr`.
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t local_smem_addr, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

// kWeightsNK: W is stored [N, K] (K contiguous), the layout the prefill GEMMs use, so that one
// copy of a row-parallel weight serves prefill and decode.  The A operand is then K-major: one
// [128 n x 64 k] TMA box per stage and the K-major descriptor of the GEMM kernels.
template <bool kTagged, bool kWeightsNK = false>
__global__ void __launch_bounds__(kThreads, 1)
gemv_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const GemvTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  // the same offset in every CTA of the cluster: the dynamic window starts at the same shared address
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kMiscOffset);
  __shared__ int flags_ok;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = (int)blockIdx.x / p.ksplit, kh = (int)blockIdx.x % p.ksplit;   // kh = rank in the cluster
  const int n0 = tile * kTileN;
  const int rank = p.rank, ws = p.world_size;

  char* my_ws = static_cast<char*>(p.buffers[rank]);
  uint32_t* my_counter = reinterpret_cast<uint32_t*>(my_ws + p.counters_offset) + blockIdx.x;
  uint32_t epoch = 0, parity = 0;
  if (ws > 1) {                          // a world of one exchanges nothing: no call number needed
    epoch = ld_relaxed_gpu(my_counter) + 1u;
    parity = epoch & 1u;
  }

  const int kb_total = (p.K + kBK - 1) / kBK;
  const int kb_per = (kb_total + p.ksplit - 1) / p.ksplit;
  const int kb0 = kh * kb_per;
  const int kb1 = kb0 + kb_per < kb_total ? kb0 + kb_per : kb_total;
  const int n_kb = kb1 > kb0 ? kb1 - kb0 : 0;

  auto load_stage = [&](int i, uint32_t stage) {
    const int kb = kb0 + i;
    uint8_t* sw = smem + (size_t)stage * kStageBytes;
    mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
    if constexpr (kWeightsNK) {
      tma_load_2d(sw, &tmap_w, &full_bar[stage], kb * kBK, n0);             // [128 n x 64 k], 16 KB
    } else {
      tma_load_2d(sw, &tmap_w, &full_bar[stage], n0, kb * kBK);               // n 0..63
      tma_load_2d(sw + 8192, &tmap_w, &full_bar[stage], n0 + 64, kb * kBK);   // n 64..127
    }
    tma_load_2d(sw + kWBytes, &tmap_x, &full_bar[stage], kb * kBK, 0);
  };

  const int n_first = n_kb < kStages ? n_kb : kStages;     // loads that need no free-stage wait
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_fence_init();
    flags_ok = 1;
    // the weight stream starts now, under the rest of the set-up
    for (int i = 0; i < n_first; ++i) load_stage(i, (uint32_t)i);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_thread_sync();
  __syncthreads();
  tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_slot;
  bool failed = false;

  float* part = reinterpret_cast<float*>(smem);          // [16][128] fp32 partial of this CTA (ring idle by then)
  const int share = kTileN / p.ksplit;                   // columns of the tile this CTA finishes
  const int c_share0 = kh * share;                       // first of them, inside the tile
  const int quarter = warp & 3;
  const int etid = (int)threadIdx.x - 64;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = (uint32_t)(n_first % kStages), phase = n_first == kStages ? 1u : 0u;
      for (int i = n_first; i < n_kb; ++i) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.timeout_ns)) {
          report_status(p.status, kTimeoutMbarrier, rank, blockIdx.x, stage, kWhereGemmEmpty);
          failed = true;
          break;
        }
        load_stage(i, stage);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // kind::f16, bf16 x bf16 -> fp32, A MN-major (bit 15), B K-major, M = 128, N = 16
      constexpr uint32_t idesc = umma_idesc_bf16_f32(kTileN, kBatchN) | (kWeightsNK ? 0u : (1u << 15));
      uint32_t stage = 0, phase = 0;
      for (int i = 0; i < n_kb; ++i) {
        if (!mbar_wait(&full_bar[stage], phase, p.timeout_ns)) {
          report_status(p.status, kTimeoutMbarrier, rank, blockIdx.x, stage, kWhereGemmFull);
          failed = true;
          break;
        }
        tcgen05_fence_after_thread_sync();
        const uint32_t sw = smem_u32(smem + (size_t)stage * kStageBytes);
        const uint64_t da = kWeightsNK ? umma_smem_desc_sw128(sw) : umma_smem_desc_mn_sw128(sw);
        const uint64_t db = umma_smem_desc_sw128(sw + kWBytes);
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          // A, MN-major: +16 k rows = +2048 B; A, K-major and B: +16 k elements inside the 128-byte row = +32 B
          const uint64_t a_step = kWeightsNK ? (uint64_t)(2 * k) : (uint64_t)(k * (2048 >> 4));
          umma_bf16_ss(tmem_base, da + a_step, db + (uint64_t)(2 * k), idesc, (i | k) != 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (!failed) umma_commit(tmem_full);
    }
  } else {
    // ---------------- epilogue, part 1 (warps 2..5): accumulator -> this CTA's shared memory ----------------
    const int col = quarter * 32 + lane;                 // column of the tile owned by this thread
    uint32_t acc[16];
    if (n_kb > 0) {
      if (!mbar_wait(tmem_full, 0, p.timeout_ns)) {
        if (lane == 0) report_status(p.status, kTimeoutMbarrier, rank, blockIdx.x, 0, kWhereGemmTmemFull);
        failed = true;
      } else {
        tcgen05_fence_after_thread_sync();
        tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(quarter * 32) << 16), acc);
        tmem_ld_wait();
      }
    } else {
#pragma unroll
      for (int b = 0; b < 16; ++b) acc[b] = 0u;
    }
    if (failed) {
#pragma unroll
      for (int b = 0; b < 16; ++b) acc[b] = 0u;
    }
#pragma unroll
    for (int b = 0; b < 16; ++b) part[b * kTileN + col] = __uint_as_float(acc[b]);
  }

  // ---- every partial of the tile is in its CTA's shared memory ----
  __syncwarp();
  cluster_barrier();

  if (warp >= 2) {
    // ---------------- epilogue, part 2: K reduction over the cluster, then the ranks ----------------
    // item = (batch row b, four consecutive columns of this CTA's share); at most 16 * 32 items
    const int n_items = p.batch * (share / 4);
    const uint32_t part_addr = smem_u32(part);
    if (ws == 1) {
      for (int item = etid; item < n_items; item += 128) {
        const int b = item / (share / 4), c = c_share0 + (item % (share / 4)) * 4;
        if (n0 + c >= p.N) continue;                                      // N % 8 == 0
        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < p.ksplit; ++j) {                              // split order: deterministic
          const float4 v = ld_dsmem_f4(part_addr + (uint32_t)(b * kTileN + c) * 4u, (uint32_t)j);
          s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
        }
        uint2 o;
        o.x = pack_bf16x2(s4.x, s4.y);
        o.y = pack_bf16x2(s4.z, s4.w);
        *reinterpret_cast<uint2*>(p.out + (size_t)b * p.N + n0 + c) = o;
      }
    } else {
      const size_t slot_stride = (size_t)kBatchN * p.N;                   // floats (or words) per slot
      const size_t parity_off = (size_t)parity * ws * slot_stride;
      // ---- push this rank's sum of the share into slot `rank` of every rank's inbox ----
      for (int item = etid; item < n_items && !failed; item += 128) {
        const int b = item / (share / 4), c = c_share0 + (item % (share / 4)) * 4;
        if (n0 + c >= p.N) continue;
        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < p.ksplit; ++j) {
          const float4 v = ld_dsmem_f4(part_addr + (uint32_t)(b * kTileN + c) * 4u, (uint32_t)j);
          s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
        }
        const size_t off = parity_off + (size_t)rank * slot_stride + (size_t)b * p.N + n0 + c;
        if constexpr (kTagged) {
          const Vec16 w0{__float_as_uint(s4.x), epoch, __float_as_uint(s4.y), epoch};
          const Vec16 w1{__float_as_uint(s4.z), epoch, __float_as_uint(s4.w), epoch};
          for (int j = 1; j <= ws; ++j) {                                 // own inbox last
            int peer = rank + j;
            if (peer >= ws) peer -= ws;
            char* dst = static_cast<char*>(p.buffers[peer]) + p.inbox_offset + off * 8;
            st_16(dst, w0);
            st_16(dst + 16, w1);
          }
        } else {
          const Vec16 v{__float_as_uint(s4.x), __float_as_uint(s4.y), __float_as_uint(s4.z), __float_as_uint(s4.w)};
          for (int j = 1; j <= ws; ++j) {
            int peer = rank + j;
            if (peer >= ws) peer -= ws;
            float* inbox = reinterpret_cast<float*>(static_cast<char*>(p.buffers[peer]) + p.inbox_offset);
            st_16(inbox + off, v);
          }
        }
      }
      if constexpr (kTagged) {
        // ---- poll the own inbox until every rank's words for an item carry this call's number ----
        const char* inbox = my_ws + p.inbox_offset;
        for (int item = etid; item < n_items && !failed && flags_ok; item += 128) {
          const int b = item / (share / 4), c = c_share0 + (item % (share / 4)) * 4;
          if (n0 + c >= p.N) continue;
          float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
          Deadline d(p.timeout_ns);
          for (int sl = 0; sl < ws; ++sl) {                               // rank order: same bits on every rank
            const char* src = inbox + (parity_off + (size_t)sl * slot_stride + (size_t)b * p.N + n0 + c) * 8;
            Vec16 a, g;
            bool got = false;
            while (!got) {
              asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src) : "memory");
              asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(g.x), "=r"(g.y), "=r"(g.z), "=r"(g.w) : "l"(src + 16) : "memory");
              got = a.y == epoch && a.w == epoch && g.y == epoch && g.w == epoch;
              if (!got && !d.alive()) {
                report_status(p.status, kTimeoutFlag, rank, tile, sl, kWhereGemvArrive, epoch);
                flags_ok = 0;
                break;
              }
            }
            if (!got) break;
            s4.x += __uint_as_float(a.x); s4.y += __uint_as_float(a.z);
            s4.z += __uint_as_float(g.x); s4.w += __uint_as_float(g.z);
          }
          if (!flags_ok) break;
          uint2 o;
          o.x = pack_bf16x2(s4.x, s4.y);
          o.y = pack_bf16x2(s4.z, s4.w);
          *reinterpret_cast<uint2*>(p.out + (size_t)b * p.N + n0 + c) = o;
        }
      } else {
        group_sync_128();   // the group's pushes precede the releases below
        const size_t flag_idx = ((size_t)parity * p.tiles + tile) * kFlagStride + (size_t)kh * ws;
        if (etid < ws && !failed) {
          uint32_t* peer_flags = reinterpret_cast<uint32_t*>(static_cast<char*>(p.buffers[etid]) + p.flags_offset);
          st_release_sys(peer_flags + flag_idx + rank, epoch);
        }
        if (etid < ws) {
          const uint32_t* mine = reinterpret_cast<const uint32_t*>(my_ws + p.flags_offset) + flag_idx + etid;
          Deadline d(p.timeout_ns);
          while (ld_acquire_sys(mine) != epoch) {
            if (!d.alive()) {
              report_status(p.status, kTimeoutFlag, rank, tile, etid, kWhereGemvArrive, epoch);
              flags_ok = 0;
              break;
            }
          }
        }
        group_sync_128();
        if (flags_ok && !failed) {
          const float* inbox = reinterpret_cast<const float*>(my_ws + p.inbox_offset) + parity_off;
          for (int item = etid; item < n_items; item += 128) {
            const int b = item / (share / 4), c = c_share0 + (item % (share / 4)) * 4;
            if (n0 + c >= p.N) continue;
            const float* src = inbox + (size_t)b * p.N + n0 + c;
            float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sl0 = 0; sl0 < ws; sl0 += 8) {                       // 8 independent loads in flight
              Vec16 v[8];
#pragma unroll
              for (int u = 0; u < 8; ++u)
                if (sl0 + u < ws) v[u] = ld_16_stream(src + (size_t)(sl0 + u) * slot_stride);
#pragma unroll
              for (int u = 0; u < 8; ++u)
                if (sl0 + u < ws) {
                  s4.x += __uint_as_float(v[u].x); s4.y += __uint_as_float(v[u].y);
                  s4.z += __uint_as_float(v[u].z); s4.w += __uint_as_float(v[u].w);
                }
            }
            uint2 o;
            o.x = pack_bf16x2(s4.x, s4.y);
            o.y = pack_bf16x2(s4.z, s4.w);
            *reinterpret_cast<uint2*>(p.out + (size_t)b * p.N + n0 + c) = o;
          }
        }
      }
    }
  }

  if (__any_sync(0xffffffffu, failed)) {
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  tcgen05_fence_before_thread_sync();
  __syncthreads();
  tcgen05_fence_after_thread_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (ws > 1 && threadIdx.x == 0) *my_counter = epoch;   // this CTA has made its call; read by its next launch
  // no CTA of the cluster leaves while another may still read its shared memory
  __syncwarp();
  cluster_barrier();
}

int encode(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
           uint32_t box_outer) {
  const DriverApi& d = DriverApi::get();
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = d.cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                                        dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1;
}

// K splits per column tile = cluster size: 1, 2, 4 or 8 (a share of 128 / ksplit columns per CTA).
int pick_ksplit(int N, int K, int num_sms, int world_size) {
  int tiles = (N + kTileN - 1) / kTileN;
  int ks = num_sms / tiles;
  ks = ks >= 8 ? 8 : (ks >= 4 ? 4 : (ks >= 2 ? 2 : 1));           // 8 = the portable cluster size
  while (ks > 1 && ((K + kBK - 1) / kBK < ks || world_size * ks > kFlagStride)) ks >>= 1;
  return ks;
}

// One launch: the K splits of a tile are the CTAs of a cluster (the attribute is set per launch because the
// split count depends on the shape).
template <class Kernel>
int launch_gemv_tc(Kernel kernel, const CUtensorMap& tw, const CUtensorMap& tx, GemvTcParams p,
                   cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
  if (e != cudaSuccess) return (int)e;
  // The largest split (cluster size) not above the planned one whose clusters are all resident at
  // once: one wave streams the weights fastest, and with several ranks it is required, because the
  // CTAs of a tile wait for the same tile's CTAs on the peers (every rank arrives at the same split:
  // same shape, same GPU).  A world of one whose tiles alone exceed the GPU runs in waves.
  int ks = p.ksplit;
  while (ks > 1 && check_co_resident(kernel, p.tiles * ks, kThreads, kSmemTotal, ks) != 0) ks >>= 1;
  if (p.world_size > 1) {
    if (int rc = check_co_resident(kernel, p.tiles * ks, kThreads, kSmemTotal, ks)) return rc;
  }
  p.ksplit = ks;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(p.tiles * p.ksplit), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)p.ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, tw, tx, p);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

}  // namespace

size_t gemv_tc_workspace_bytes(int N, int K, int world_size, int num_sms, size_t* flags_offset,
                               size_t* inbox_offset, int* tiles, int* ksplit, bool tagged,
                               size_t* counters_offset) {
  int t = (N + kTileN - 1) / kTileN;
  int ks = pick_ksplit(N, K, num_sms, world_size);
  size_t counters_off = 256;
  size_t counters_bytes = (size_t)t * ks * 4;
  size_t flags_off = (counters_off + counters_bytes + 255) & ~(size_t)255;
  size_t flags_bytes = (size_t)2 * t * kFlagStride * 4;
  size_t inbox_off = (flags_off + flags_bytes + 255) & ~(size_t)255;
  size_t inbox_bytes = (size_t)2 * world_size * kBatchN * N * (tagged ? 8 : 4);
  if (counters_offset) *counters_offset = counters_off;
  if (flags_offset) *flags_offset = flags_off;
  if (inbox_offset) *inbox_offset = inbox_off;
  if (tiles) *tiles = t;
  if (ksplit) *ksplit = ks;
  return inbox_off + inbox_bytes;
}

int launch_gemv_all_reduce_tc(const GemvArgs& a, int num_sms, cudaStream_t stream, bool tagged, bool weights_nk) {
  if (a.batch < 1 || a.batch > kBatchN || a.N % 8 != 0 || a.K % 8 != 0 || a.ws_offset != 0)
    return cudaErrorInvalidValue;
  GemvTcParams p{};
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.batch = a.batch; p.K = a.K; p.N = a.N;
  p.rank = a.pv.rank; p.world_size = a.pv.world_size;
  p.buffers = a.pv.buffers;
  p.timeout_ns = a.timeout_ns;
  p.status = a.status;
  gemv_tc_workspace_bytes(a.N, a.K, a.pv.world_size, num_sms, &p.flags_offset, &p.inbox_offset, &p.tiles,
                          &p.ksplit, tagged, &p.counters_offset);
  if (p.world_size * p.ksplit > kFlagStride) return cudaErrorInvalidValue;
  CUtensorMap tw, tx;
  if (weights_nk) {
    if (encode(&tw, a.w, (uint64_t)a.K, (uint64_t)a.N, kBK, kTileN)) return cudaErrorInvalidValue;   // [N, K]
  } else {
    if (encode(&tw, a.w, (uint64_t)a.N, (uint64_t)a.K, 64, kBK)) return cudaErrorInvalidValue;       // [K, N]
  }
  if (encode(&tx, a.x, (uint64_t)a.K, (uint64_t)a.batch, kBK, kBatchN)) return cudaErrorInvalidValue;
  if (weights_nk)
    return tagged ? launch_gemv_tc(gemv_tc_kernel<true, true>, tw, tx, p, stream)
                  : launch_gemv_tc(gemv_tc_kernel<false, true>, tw, tx, p, stream);
  return tagged ? launch_gemv_tc(gemv_tc_kernel<true>, tw, tx, p, stream)
                : launch_gemv_tc(gemv_tc_kernel<false>, tw, tx, p, stream);
}

}  // namespace smr

// ---------------------------------------------------------------------------
// Allocation-free C entry point (see gemv_noalloc.h).  The global memory that the
// kernel above needs besides its operands lives in this array: offset 0 holds the
// one-entry "workspace base of every rank" table the kernel reads, offset 64 the
// 32-byte Status record its bounded waits report into; a (here unused) workspace
// would start at offset 256.  In a world of one the K splits of a tile meet in
// shared memory, so nothing else is kept in global memory between or during calls.
// ---------------------------------------------------------------------------
#include <mutex>
#include <stdio.h>

#include "gemv_noalloc.h"

namespace {

static __device__ __align__(256) unsigned char g_gemv_noalloc_scratch[SMR_GEMV_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
unsigned char* g_noalloc_base[kMaxDevices] = {};   // device address of the array, per device
int g_noalloc_sms[kMaxDevices] = {};
constexpr size_t kNoallocStatusOffset = 64;

int noalloc_fail(int code, char* err, int err_len, const char* what, const char* detail = "") {
  if (err != nullptr && err_len > 0) snprintf(err, (size_t)err_len, "smr_gemv_bf16_noalloc: %s%s", what, detail);
  return code;
}

}  // namespace

extern "C" int smr_gemv_bf16_noalloc(const void* x, const void* w, void* out, int batch, int K, int N,
                                     void* stream_ptr, char* err, int err_len) {
  using namespace smr;
  if (batch < 1 || batch > SMR_GEMV_NOALLOC_MAX_BATCH)
    return noalloc_fail(1, err, err_len, "batch must be between 1 and 16");
  if (N < 8 || N > SMR_GEMV_NOALLOC_MAX_N || N % 8 != 0)
    return noalloc_fail(1, err, err_len, "N must be a multiple of 8 and at most 8192 (the limit of this entry point)");
  if (K < 8 || K % 8 != 0) return noalloc_fail(1, err, err_len, "K must be a positive multiple of 8");
  if (x == nullptr || w == nullptr || out == nullptr || ((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) % 16 != 0)
    return noalloc_fail(2, err, err_len, "x, w and out must be non-null and 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail(3, err, err_len, "cudaGetDevice: ", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return noalloc_fail(3, err, err_len, "device ordinal out of range");
  unsigned char* base;
  int sms;
  {
    // Once per device, with that device current: the array's name is only a
    // host-side handle; the kernel needs the address the symbol has on THIS GPU.
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_base[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_gemv_noalloc_scratch);
      if (e != cudaSuccess) return noalloc_fail(3, err, err_len, "cudaGetSymbolAddress: ", cudaGetErrorString(e));
      void* ws_base = static_cast<unsigned char*>(p) + 256;
      e = cudaMemcpy(p, &ws_base, sizeof(void*), cudaMemcpyHostToDevice);   // the one-entry base table
      if (e != cudaSuccess) return noalloc_fail(3, err, err_len, "cudaMemcpy(base table): ", cudaGetErrorString(e));
      int n = 0;
      e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return noalloc_fail(3, err, err_len, "cudaDeviceGetAttribute: ", cudaGetErrorString(e));
      g_noalloc_sms[dev] = n;
      g_noalloc_base[dev] = static_cast<unsigned char*>(p);
    }
    base = g_noalloc_base[dev];
    sms = g_noalloc_sms[dev];
  }

  GemvTcParams p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.batch = batch; p.K = K; p.N = N;
  p.rank = 0; p.world_size = 1;
  p.buffers = reinterpret_cast<void* const*>(base);
  p.timeout_ns = 2000000000ull;
  p.status = reinterpret_cast<Status*>(base + kNoallocStatusOffset);
  // tiles and K splits of this shape; the offsets describe a workspace that a world of one never touches
  gemv_tc_workspace_bytes(N, K, 1, sms, &p.flags_offset, &p.inbox_offset, &p.tiles, &p.ksplit, false,
                          &p.counters_offset);
  CUtensorMap tw, tx;
  try {
    if (encode(&tw, w, (uint64_t)N, (uint64_t)K, 64, kBK) || encode(&tx, x, (uint64_t)K, (uint64_t)batch, kBK, kBatchN))
      return noalloc_fail(3, err, err_len, "cuTensorMapEncodeTiled rejected the operands");
  } catch (const std::exception& ex) {
    return noalloc_fail(3, err, err_len, "CUDA driver: ", ex.what());
  }
  int rc = launch_gemv_tc(gemv_tc_kernel<false>, tw, tx, p, stream);
  if (rc != 0) return noalloc_fail(3, err, err_len, "kernel launch: ", cudaGetErrorString((cudaError_t)rc));
  return 0;
}

extern "C" int smr_gemv_bf16_noalloc_status(void* stream_ptr, unsigned int record[6], char* err, int err_len) {
  using namespace smr;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail(3, err, err_len, "cudaGetDevice: ", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return noalloc_fail(3, err, err_len, "device ordinal out of range");
  unsigned char* base;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    base = g_noalloc_base[dev];
  }
  if (record != nullptr)
    for (int i = 0; i < 6; ++i) record[i] = 0u;
  if (base == nullptr) return 0;                 // no call on this device yet: nothing can have failed
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return noalloc_fail(3, err, err_len, "cudaStreamSynchronize: ", cudaGetErrorString(e));
  Status st{};
  e = cudaMemcpy(&st, base + kNoallocStatusOffset, sizeof(Status), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return noalloc_fail(3, err, err_len, "cudaMemcpy(status): ", cudaGetErrorString(e));
  if (record != nullptr) {
    record[0] = st.code; record[1] = st.rank; record[2] = st.block;
    record[3] = st.peer; record[4] = st.where; record[5] = st.aux;
  }
  if (st.code == kOk) return 0;
  e = cudaMemset(base + kNoallocStatusOffset, 0, sizeof(Status));    // reported once
  if (e != cudaSuccess) return noalloc_fail(3, err, err_len, "cudaMemset(status): ", cudaGetErrorString(e));
  return noalloc_fail(4, err, err_len, "a wait inside an earlier call ran out after 2 s (the CTAs of the kernel were "
                                       "not all resident at once?); that call left `out` unwritten");
}
