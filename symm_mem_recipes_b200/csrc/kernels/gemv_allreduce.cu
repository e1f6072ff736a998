// Fused GEMV + all-reduce for tensor-parallel decode (no upstream counterpart):
//     out[b, n] = sum over ranks r of  x_r[b, :] . W_r[:, n]          b <= 16
// Each rank streams its weight shard W_r[K, N] from HBM exactly once.  A CTA
// owns 64 output columns: it computes the rank's fp32 partial for them, pushes
// it into the inbox of every peer with 16-byte peer stores, raises a per-tile
// flag on every peer (st.release.sys), waits (bounded) for the WS flags of its
// own tile and sums the WS partials in rank order.  The reduction of early
// tiles therefore overlaps the weight stream of later ones, and every rank
// produces the same bits.
//
// Re-launch safety without host-side state (graph replay): the kernel reads an
// epoch counter from its workspace, uses epoch+1 as the flag value and
// (epoch+1) & 1 as the inbox parity, and the last CTA to finish stores the new
// epoch.  A peer can be at most one call ahead (it needs this rank's partials
// to finish a call), so two inbox parities suffice.
#include <cuda_runtime.h>

#include "../device/barrier.cuh"
#include "../device/vec.cuh"
#include "launch.h"
#include "residency.h"

namespace smr {

namespace {

constexpr int kTN = 64;            // columns per CTA
constexpr int kCG = kTN / 8;       // 16-byte column groups per CTA
constexpr int kFlagStride = 16;    // u32 slots per tile (>= max world size)

struct GemvParams {
  const __nv_bfloat16* x;   // [batch, K]
  const __nv_bfloat16* w;   // [K, N]
  __nv_bfloat16* out;       // [batch, N]
  int batch, K, N;
  int rank, world_size;
  void* const* buffers;     // workspace base of every rank (peer-mapped)
  size_t ws_offset;         // offset of the workspace inside the payload
  size_t flags_offset;      // from workspace base
  size_t inbox_offset;      // from workspace base
  int max_tiles;
  uint64_t timeout_ns;
  Status* status;
};

// workspace header: [0] epoch, [1] CTAs done
template <int BT, int THREADS, int U>
__global__ void __launch_bounds__(THREADS, 1)
gemv_all_reduce_kernel(const GemvParams p) {
  constexpr int KL = THREADS / kCG;       // k-lanes
  constexpr int NW = THREADS / 32;
  extern __shared__ __align__(16) uint8_t smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);                 // [K][BT]
  float* red = reinterpret_cast<float*>(smem + (((size_t)p.K * BT * 2 + 15) & ~(size_t)15));  // [NW][BT][kTN]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cg = tid % kCG, kl = tid / kCG;
  const int tile = blockIdx.x, n0 = tile * kTN;
  const int rank = p.rank, ws = p.world_size;

  char* my_ws = static_cast<char*>(p.buffers[rank]) + p.ws_offset;
  uint32_t* header = reinterpret_cast<uint32_t*>(my_ws);
  const uint32_t epoch = ld_relaxed_gpu(&header[0]) + 1u;
  const uint32_t parity = epoch & 1u;

  // ---- stage x transposed: xs[k][b], zero rows for b >= batch ----
  for (int idx = tid; idx < p.K * BT; idx += THREADS) {
    int b = idx / p.K, k = idx - b * p.K;
    xs[k * BT + b] = b < p.batch ? p.x[(size_t)b * p.K + k] : __float2bfloat16(0.f);
  }
  __syncthreads();

  float acc[BT][8];
#pragma unroll
  for (int b = 0; b < BT; ++b)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[b][j] = 0.f;

  const bool col_ok = n0 + cg * 8 < p.N;   // N % 8 == 0
  const __nv_bfloat16* wcol = p.w + n0 + cg * 8;
  for (int k0 = kl; k0 < p.K; k0 += KL * U) {
    Vec16 wv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int k = k0 + u * KL;
      if (k < p.K && col_ok) wv[u] = ld_16_nc(wcol + (size_t)k * p.N);
      else wv[u] = Vec16{0u, 0u, 0u, 0u};
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int k = k0 + u * KL;
      if (k >= p.K) break;
      float wf[8] = {bf16lo_to_f32(wv[u].x), bf16hi_to_f32(wv[u].x), bf16lo_to_f32(wv[u].y),
                     bf16hi_to_f32(wv[u].y), bf16lo_to_f32(wv[u].z), bf16hi_to_f32(wv[u].z),
                     bf16lo_to_f32(wv[u].w), bf16hi_to_f32(wv[u].w)};
      const __nv_bfloat16* xk = xs + (size_t)k * BT;
#pragma unroll
      for (int b = 0; b < BT; ++b) {
        float xv = __bfloat162float(xk[b]);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[b][j] = fmaf(xv, wf[j], acc[b][j]);
      }
    }
  }

  // ---- reduce over k-lanes: inside the warp (4 k-lanes), then across warps ----
#pragma unroll
  for (int b = 0; b < BT; ++b)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = acc[b][j];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      acc[b][j] = v;
    }
  if (lane < kCG) {
#pragma unroll
    for (int b = 0; b < BT; ++b)
#pragma unroll
      for (int j = 0; j < 8; ++j) red[((size_t)warp * BT + b) * kTN + lane * 8 + j] = acc[b][j];
  }
  __syncthreads();

  // ---- push the partial of this tile to every rank's inbox ----
  // item = (b, 4 columns): BT * 16 items
  const size_t inbox_stride_src = (size_t)BT * p.N;            // floats per source rank
  const size_t inbox_parity = (size_t)parity * ws * inbox_stride_src;
  for (int item = tid; item < BT * (kTN / 4); item += THREADS) {
    int b = item / (kTN / 4), c4 = (item % (kTN / 4)) * 4;
    if (n0 + c4 >= p.N) continue;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float4 v = *reinterpret_cast<const float4*>(&red[((size_t)w * BT + b) * kTN + c4]);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    size_t off = inbox_parity + (size_t)rank * inbox_stride_src + (size_t)b * p.N + n0 + c4;
    Vec16 o{__float_as_uint(s.x), __float_as_uint(s.y), __float_as_uint(s.z), __float_as_uint(s.w)};
    for (int j = 0; j < ws; ++j) {
      int peer = (rank + 1 + j) % ws;     // own inbox last
      float* inbox = reinterpret_cast<float*>(static_cast<char*>(p.buffers[peer]) + p.ws_offset + p.inbox_offset);
      st_16(inbox + off, o);
    }
  }
  __syncthreads();   // all pushes of the CTA precede the release below

  // ---- signal every peer, wait for every peer ----
  bool ok = true;
  const size_t flag_idx = ((size_t)parity * p.max_tiles + tile) * kFlagStride;
  if (tid < ws) {
    uint32_t* peer_flags = reinterpret_cast<uint32_t*>(static_cast<char*>(p.buffers[tid]) + p.ws_offset + p.flags_offset);
    st_release_sys(peer_flags + flag_idx + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(my_ws + p.flags_offset) + flag_idx + tid;
    Deadline d(p.timeout_ns);
    while (ld_acquire_sys(mine) != epoch) {
      if (!d.alive()) {
        report_status(p.status, kTimeoutFlag, rank, tile, tid, kWhereGemvArrive, epoch);
        ok = false;
        break;
      }
    }
  }
  ok = __syncthreads_and(ok) != 0;

  // ---- ordered sum of the WS partials, bf16 out ----
  if (ok) {
    const float* inbox = reinterpret_cast<const float*>(my_ws + p.inbox_offset) + inbox_parity;
    for (int item = tid; item < BT * (kTN / 4); item += THREADS) {
      int b = item / (kTN / 4), c4 = (item % (kTN / 4)) * 4;
      if (b >= p.batch || n0 + c4 >= p.N) continue;
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < ws; ++r) {
        Vec16 v = ld_16(inbox + (size_t)r * inbox_stride_src + (size_t)b * p.N + n0 + c4);
        s.x += __uint_as_float(v.x); s.y += __uint_as_float(v.y);
        s.z += __uint_as_float(v.z); s.w += __uint_as_float(v.w);
      }
      uint2 o;
      o.x = pack_bf16x2(s.x, s.y);
      o.y = pack_bf16x2(s.z, s.w);
      *reinterpret_cast<uint2*>(p.out + (size_t)b * p.N + n0 + c4) = o;
    }
  }

  // ---- the last CTA to finish publishes the new epoch ----
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    uint32_t done = atomicAdd(&header[1], 1u);
    if (done == gridDim.x - 1) {
      header[1] = 0u;
      __threadfence();
      st_release_gpu(&header[0], epoch);
    }
  }
}

template <int BT, int THREADS, int U>
int launch_variant(const GemvParams& p, int tiles, cudaStream_t stream) {
  auto kern = gemv_all_reduce_kernel<BT, THREADS, U>;
  size_t smem = (((size_t)p.K * BT * 2 + 15) & ~(size_t)15) + (size_t)(THREADS / 32) * BT * kTN * 4;
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  // A tile waits for the same tile of every peer: with peers, all tiles must be resident at once.
  if (p.world_size > 1) {
    if (int rc = check_co_resident(kern, tiles, THREADS, smem)) return rc;
  }
  kern<<<tiles, THREADS, smem, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace

size_t gemv_workspace_bytes(int batch_tile, int N, int world_size, size_t* flags_offset,
                            size_t* inbox_offset, int* max_tiles) {
  int tiles = (N + kTN - 1) / kTN;
  size_t flags_off = 256;
  size_t flags_bytes = (size_t)2 * tiles * kFlagStride * 4;
  size_t inbox_off = (flags_off + flags_bytes + 255) & ~(size_t)255;
  size_t inbox_bytes = (size_t)2 * world_size * batch_tile * N * 4;
  if (flags_offset) *flags_offset = flags_off;
  if (inbox_offset) *inbox_offset = inbox_off;
  if (max_tiles) *max_tiles = tiles;
  return inbox_off + inbox_bytes;
}

int gemv_batch_tile(int batch) {
  if (batch <= 1) return 1;
  if (batch <= 2) return 2;
  if (batch <= 4) return 4;
  if (batch <= 8) return 8;
  if (batch <= 16) return 16;
  return -1;
}

int launch_gemv_all_reduce(const GemvArgs& a, cudaStream_t stream) {
  int bt = gemv_batch_tile(a.batch);
  if (bt < 0 || a.batch < 1 || a.N % 8 != 0 || a.K < 1) return cudaErrorInvalidValue;
  GemvParams p{};
  p.x = static_cast<const __nv_bfloat16*>(a.x);
  p.w = static_cast<const __nv_bfloat16*>(a.w);
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.batch = a.batch; p.K = a.K; p.N = a.N;
  p.rank = a.pv.rank; p.world_size = a.pv.world_size;
  p.buffers = a.pv.buffers;
  p.ws_offset = a.ws_offset;
  p.timeout_ns = a.timeout_ns;
  p.status = a.status;
  gemv_workspace_bytes(bt, a.N, a.pv.world_size, &p.flags_offset, &p.inbox_offset, &p.max_tiles);
  int tiles = p.max_tiles;
  switch (bt) {
    case 1: return launch_variant<1, 512, 8>(p, tiles, stream);
    case 2: return launch_variant<2, 512, 8>(p, tiles, stream);
    case 4: return launch_variant<4, 512, 8>(p, tiles, stream);
    case 8: return launch_variant<8, 256, 4>(p, tiles, stream);
    default: return launch_variant<16, 256, 4>(p, tiles, stream);
  }
}

}  // namespace smr
