// Rank-local pieces of a Llama-style decoder layer that sit between the fused
// GEMM + collective kernels: RMSNorm (optionally fused with the residual add
// that precedes it), rotary embedding in place on the QKV buffer, and
// SiLU(gate) * up, and the attention of one decode step.  Each is one pass over its operand in bf16 with fp32 math;
// the PyTorch compositions they replace take five to ten passes with fp32
// temporaries.  No upstream counterpart (the upstream recipes stop at the
// single fused op).
//
// Arithmetic contracts (what the CPU oracles in oracle/cpu_reference.cpp and
// the tests pin down):
//   rms_norm:  s = x (+ r, rounded to bf16 when r is given; also stored as
//              `sum_out`);  n = bf16( s * rsqrt(mean(s^2) + eps) );
//              out = bf16( n * w ).
//   rope:      pairs (i, i + D/2) of every rotated head, Llama convention:
//              angle = pos * theta^(-2i/D), fp32; results rounded to bf16.
//   silu_mul:  out = bf16( g / (1 + exp(-g)) * u ) for gate g, up u.
//   decode_attention: softmax(q . K / sqrt(D)) V over the cached positions 0..pos, fp32; bf16 out.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../device/vec.cuh"
#include "launch.h"

namespace smr {

namespace {

constexpr int kNormThreads = 256;

__device__ __forceinline__ void unpack8(const Vec16& v, float (&f)[8]) {
  f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x);
  f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
  f[4] = bf16lo_to_f32(v.z); f[5] = bf16hi_to_f32(v.z);
  f[6] = bf16lo_to_f32(v.w); f[7] = bf16hi_to_f32(v.w);
}
__device__ __forceinline__ Vec16 pack8(const float (&f)[8]) {
  Vec16 o;
  o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
  return o;
}
__device__ __forceinline__ float round_bf16(float f) {
  return __bfloat162float(__float2bfloat16_rn(f));
}

// One CTA per row.  Pass 1: s = x (+ r), sum of squares (s stored when asked
// for).  Pass 2 re-reads s (from L1 / L2) and writes the normalised row.
// `sum_out` may be the buffer of `x` or of `residual` (running residual stream
// updated in place) and `out` may be the buffer of `x`; `out` must not be the
// buffer of `sum_out` or of `residual`.
__global__ void __launch_bounds__(kNormThreads)
rms_norm_kernel(const __nv_bfloat16* x, const __nv_bfloat16* residual, const __nv_bfloat16* __restrict__ w,
                __nv_bfloat16* sum_out, __nv_bfloat16* out, int H, float eps) {
  const size_t row = blockIdx.x;
  const Vec16* xr = reinterpret_cast<const Vec16*>(x + row * H);
  const Vec16* rr = residual ? reinterpret_cast<const Vec16*>(residual + row * H) : nullptr;
  Vec16* sr = sum_out ? reinterpret_cast<Vec16*>(sum_out + row * H) : nullptr;
  const int n_vec = H / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n_vec; i += kNormThreads) {
    float a[8];
    unpack8(ld_16(xr + i), a);
    if (rr != nullptr) {
      float b[8];
      unpack8(ld_16(rr + i), b);
#pragma unroll
      for (int q = 0; q < 8; ++q) a[q] = round_bf16(a[q] + b[q]);
      if (sr != nullptr) st_16(sr + i, pack8(a));
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) ss += a[q] * a[q];
  }
  // block sum
  __shared__ float warp_sums[kNormThreads / 32];
  __shared__ float scale_s;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < kNormThreads / 32 ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) scale_s = rsqrtf(t / (float)H + eps);
  }
  __syncthreads();
  const float scale = scale_s;
  const Vec16* wr = reinterpret_cast<const Vec16*>(w);
  Vec16* orow = reinterpret_cast<Vec16*>(out + row * H);
  for (int i = threadIdx.x; i < n_vec; i += kNormThreads) {
    float a[8], g[8];
    if (sr != nullptr) {
      // this thread stored s[i] itself in pass 1; reading it back (instead of x and r again) also
      // keeps the kernel correct when sum_out is the same buffer as x or as the residual
      unpack8(ld_16(sr + i), a);
    } else {
      unpack8(ld_16(xr + i), a);
      if (rr != nullptr) {
        float b[8];
        unpack8(ld_16(rr + i), b);
#pragma unroll
        for (int q = 0; q < 8; ++q) a[q] = round_bf16(a[q] + b[q]);
      }
    }
    unpack8(ld_16(wr + i), g);
#pragma unroll
    for (int q = 0; q < 8; ++q) a[q] = round_bf16(a[q] * scale) * g[q];
    st_16(orow + i, pack8(a));
  }
}

// In place on rows of `row_stride` elements: heads [0, n_heads) of D elements
// each are rotated.  Token t sits at position pos0 + (t % seq); with `pos_dev`
// the first position is read from device memory instead (a decode step
// captured in a CUDA graph takes its position from a tensor).  One thread per
// (token, head, 8 consecutive pair indices).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, long long n_items, int row_stride, int n_heads, int D,
                            int seq, int pos0, const int* __restrict__ pos_dev, float log2_theta) {
  if (pos_dev != nullptr) pos0 = *pos_dev;
  const int vec_per_head = D / 16;                      // vectors of 8 pairs
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x; item < n_items; item += stride) {
    const int v = (int)(item % vec_per_head);
    const long long th = item / vec_per_head;
    const int head = (int)(th % n_heads);
    const long long t = th / n_heads;
    const float pos = (float)(pos0 + (int)(t % seq));
    __nv_bfloat16* base = qkv + t * row_stride + (long long)head * D + v * 8;
    float x1[8], x2[8], y1[8], y2[8];
    unpack8(ld_16(base), x1);
    unpack8(ld_16(base + D / 2), x2);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int i = v * 8 + q;                          // pair index in [0, D/2)
      const float inv_freq = exp2f(-(2.0f * (float)i / (float)D) * log2_theta);
      float ang = pos * inv_freq;
      // bring the angle into [-pi, pi] before the fast sine / cosine
      ang -= 6.283185307179586f * rintf(ang * 0.15915494309189535f);
      float sn, cs;
      __sincosf(ang, &sn, &cs);
      y1[q] = x1[q] * cs - x2[q] * sn;
      y2[q] = x2[q] * cs + x1[q] * sn;
    }
    st_16(base, pack8(y1));
    st_16(base + D / 2, pack8(y2));
  }
}

// gu [T, 2F]: gate = columns [0, F), up = [F, 2F); out [T, F].
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                long long n_vec, int F) {
  const int vec_per_row = F / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n_vec; idx += stride) {
    const long long row = idx / vec_per_row;
    const int cv = (int)(idx - row * vec_per_row);
    const __nv_bfloat16* g = gu + row * 2 * F + cv * 8;
    float a[8], b[8];
    unpack8(ld_16_stream(g), a);
    unpack8(ld_16_stream(g + F), b);
#pragma unroll
    for (int q = 0; q < 8; ++q) a[q] = a[q] / (1.0f + __expf(-a[q])) * b[q];
    st_16(out + row * F + cv * 8, pack8(a));
  }
}

// One decode step of attention (one new token per sequence) for this rank's heads, split along the
// cached sequence ("flash decoding").  CTA (b x kv head, split) has eight warps; warp `unit` walks
// positions unit, unit + n_units, ... <= pos, four at a time (eight independent row loads in flight),
// with an online softmax for the G = hq / hkv query heads that share the KV head: a lane owns VEC of
// the D = 32 * VEC dimensions, so one K or V row is one coalesced warp load.  The warps of a CTA
// merge their (max, sum, weighted V) through shared memory into one partial per CTA in scratch; the
// last CTA of a (b, kv head) to arrive merges those (one warp per head weighs the splits, then all
// threads add them up) and writes bf16.  The new token's key and value
// come from the QKV row (split 0 also writes them into the caches), so no CTA depends on another's
// cache write.  The position may come from device memory and the grid does not depend on it: a
// captured graph serves every position.
constexpr int kAttnWarps = 8;
constexpr int kAttnMaxG = 8;
constexpr int kAttnBatch = 4;            // positions whose rows are loaded before any is used
constexpr int kAttnMaxSplit = 64;        // CTAs per (sequence, KV head) at most
// "No position seen yet" as a running maximum.  A finite stand-in for minus infinity: a warp or a CTA
// may see no position at all (pos + 1 < units), and exp(-inf - (-inf)) would be NaN in the merges,
// while exp(kNoScore - kNoScore) = 1 weights a sum and a vector that are both zero.
constexpr float kNoScore = -1.0e30f;

// VEC (2 or 4) consecutive bf16 as one 4- or 8-byte access
template <int VEC>
__device__ __forceinline__ void load_bf16_vec(const __nv_bfloat16* p, float (&f)[VEC]) {
  static_assert(VEC == 2 || VEC == 4, "a lane owns 2 or 4 of the head's dimensions");
  if constexpr (VEC == 4) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    f[0] = bf16lo_to_f32(w.x); f[1] = bf16hi_to_f32(w.x);
    f[2] = bf16lo_to_f32(w.y); f[3] = bf16hi_to_f32(w.y);
  } else {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
    f[0] = bf16lo_to_f32(w); f[1] = bf16hi_to_f32(w);
  }
}
template <int VEC>
__device__ __forceinline__ void store_bf16_vec(__nv_bfloat16* dst, const float (&f)[VEC]) {
  if constexpr (VEC == 4) {
    uint2 w;
    w.x = pack_bf16x2(f[0], f[1]);
    w.y = pack_bf16x2(f[2], f[3]);
    *reinterpret_cast<uint2*>(dst) = w;
  } else {
    *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(f[0], f[1]);
  }
}
template <int VEC>
__device__ __forceinline__ void copy_bf16_vec(__nv_bfloat16* dst, const __nv_bfloat16* src) {
  if constexpr (VEC == 4) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(src);
  else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
}

// Merges the `n` partials that the warps of a CTA left in shared memory for query head g, dimension d:
// partial i has its max at m[i * stride], its sum at l[i * stride] and its weighted V at a[i * stride].
// Returns the merged weighted V, max, sum.
__device__ __forceinline__ void merge_partials(const float* m, const float* l, const float* a, int n, int stride,
                                               float& out_a, float& out_m, float& out_l) {
  float big = kNoScore;
#pragma unroll 8
  for (int i = 0; i < n; ++i) big = fmaxf(big, m[(size_t)i * stride]);
  float sum = 0.f, acc = 0.f;
#pragma unroll 8
  for (int i = 0; i < n; ++i) {
    const float w = __expf(m[(size_t)i * stride] - big);   // 0 for a partial that saw no position while another did
    sum += w * l[(size_t)i * stride];
    acc += w * a[(size_t)i * stride];
  }
  out_a = acc; out_m = big; out_l = sum;
}

template <int VEC>
__global__ void __launch_bounds__(kAttnWarps * 32, 2)
decode_attention_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                        __nv_bfloat16* __restrict__ out, float* scratch, unsigned int* counters, int hq, int hkv,
                        int s_max, int pos0, const int* __restrict__ pos_dev, float scale, float log2_theta) {
  constexpr int D = 32 * VEC;
  constexpr int kRow = D + 2;                                  // D weighted-V sums, then max and sum
  __shared__ float sm[kAttnWarps][kAttnMaxG][kRow];
  __shared__ __align__(16) float wsm[kAttnWarps][kAttnBatch * kAttnMaxG];   // a batch's softmax weights, per warp
  __shared__ __align__(16) float csm[kAttnWarps][kAttnMaxG];                // and its rescaling of the running sums
  __shared__ float split_w[kAttnMaxG][kAttnMaxSplit];   // the last CTA's weights of the splits, per head
  __shared__ float head_sum[kAttnMaxG];
  __shared__ int is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, b = bh / hkv, kvh = bh - b * hkv;
  const int n_split = gridDim.y, split = blockIdx.y;
  const int n_units = n_split * kAttnWarps, unit = split * kAttnWarps + warp;
  const int G = hq / hkv;
  int pos = pos_dev != nullptr ? *pos_dev : pos0;
  pos = pos < 0 ? 0 : (pos >= s_max ? s_max - 1 : pos);
  const __nv_bfloat16* row = qkv + (size_t)b * (hq + 2 * hkv) * D;
  const __nv_bfloat16* k_new = row + (size_t)hq * D + (size_t)kvh * D + lane * VEC;
  const __nv_bfloat16* v_new = row + (size_t)(hq + hkv) * D + (size_t)kvh * D + lane * VEC;

  // Rotary embedding of the new token's queries and key inside this kernel (log2_theta != 0): the
  // pair (i, i + D/2) sits in lanes t and t ^ 16 at the same j; results are rounded to bf16 as the
  // stand-alone RoPE kernel rounds them, so both routes give the same bits.
  float cs[VEC], sn[VEC];
  const bool rotate = log2_theta != 0.f;
  if (rotate) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int i = (lane * VEC + j) & (D / 2 - 1);
      float ang = (float)pos * exp2f(-(2.0f * (float)i / (float)D) * log2_theta);
      ang -= 6.283185307179586f * rintf(ang * 0.15915494309189535f);
      __sincosf(ang, &sn[j], &cs[j]);
    }
  }
  auto rope = [&](float (&x)[VEC]) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, x[j], 16);
      x[j] = round_bf16(lane < 16 ? x[j] * cs[j] - other * sn[j] : x[j] * cs[j] + other * sn[j]);
    }
  };
  float k_tok[VEC], v_tok[VEC];                          // the new token's key (rotated) and value
  load_bf16_vec<VEC>(k_new, k_tok);
  load_bf16_vec<VEC>(v_new, v_tok);
  if (rotate) rope(k_tok);

  float q[kAttnMaxG][VEC], acc[kAttnMaxG][VEC];
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[g][j] = q[g][j] = 0.f;
    if (g < G) {
      load_bf16_vec<VEC>(row + (size_t)(kvh * G + g) * D + lane * VEC, q[g]);
      if (rotate) rope(q[g]);
#pragma unroll
      for (int j = 0; j < VEC; ++j) q[g][j] *= scale;
    }
  }
  // After the reduction below, lane L owns the score of position slot L >> 3 of the batch and query
  // head L & 7, and keeps the running maximum of that head (the same value in the four lanes of a
  // head) and its own slot's share of the running sum.
  const int my_slot = lane >> 3, my_g = lane & 7;
  float m_run = kNoScore, l_run = 0.f;
  for (int p0 = unit; p0 <= pos; p0 += kAttnBatch * n_units) {
    float k[kAttnBatch][VEC], v[kAttnBatch][VEC];
#pragma unroll
    for (int i = 0; i < kAttnBatch; ++i) {                      // all loads of the batch before any use
      const int p = p0 + i * n_units;
#pragma unroll
      for (int j = 0; j < VEC; ++j) k[i][j] = v[i][j] = 0.f;
      if (p < pos) {
        const size_t off = (((size_t)b * s_max + p) * hkv + kvh) * D + lane * VEC;
        load_bf16_vec<VEC>(k_cache + off, k[i]);
        load_bf16_vec<VEC>(v_cache + off, v[i]);
      } else if (p == pos) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          k[i][j] = k_tok[j];
          v[i][j] = v_tok[j];
        }
      }
    }
    // this lane's share of the 4 x 8 dot products, then a halving exchange: 31 shuffles leave the
    // complete sum of product (slot, head) in lane slot * 8 + head (a shuffle tree per product
    // would take 160)
    float val[kAttnBatch * kAttnMaxG];
#pragma unroll
    for (int i = 0; i < kAttnBatch; ++i)
#pragma unroll
      for (int g = 0; g < kAttnMaxG; ++g) {
        float d = 0.f;
#pragma unroll
        for (int j = 0; j < VEC; ++j) d += q[g][j] * k[i][j];
        val[i * kAttnMaxG + g] = d;
      }
#pragma unroll
    for (int sft = 16, n = 32; sft >= 1; sft >>= 1, n >>= 1) {
      const bool upper = (lane & sft) != 0;
#pragma unroll
      for (int t = 0; t < n / 2; ++t) {
        const float send = upper ? val[t] : val[t + n / 2];
        const float keep = upper ? val[t + n / 2] : val[t];
        val[t] = keep + __shfl_xor_sync(0xffffffffu, send, sft);
      }
    }
    const bool valid = my_g < G && p0 + my_slot * n_units <= pos;
    const float sc = valid ? val[0] : kNoScore;
    float mb = fmaxf(sc, __shfl_xor_sync(0xffffffffu, sc, 8));
    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 16));
    const float m_new = fmaxf(m_run, mb);
    const float corr = __expf(m_run - m_new);                  // 1 while the head has seen no position
    const float w = valid ? __expf(sc - m_new) : 0.f;
    l_run = l_run * corr + w;
    m_run = m_new;
    // every lane needs all 32 weights and the 8 corrections: through shared memory (broadcast reads)
    wsm[warp][lane] = w;
    if (lane < kAttnMaxG) csm[warp][lane] = corr;
    __syncwarp();
#pragma unroll
    for (int g = 0; g < kAttnMaxG; ++g) {
      const float c = csm[warp][g];
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[g][j] *= c;
    }
#pragma unroll
    for (int i = 0; i < kAttnBatch; ++i)
#pragma unroll
      for (int g = 0; g < kAttnMaxG; ++g) {
        const float wv = wsm[warp][i * kAttnMaxG + g];
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[g][j] += wv * v[i][j];
      }
    __syncwarp();                                               // all lanes have read before the next batch writes
  }
  // the head's sum: add the four slots' shares (its maximum is already the same in the four lanes)
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 8);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
  if (split == 0 && warp == 0) {                      // the new token's key and value enter the caches
    const size_t off = (((size_t)b * s_max + pos) * hkv + kvh) * D + lane * VEC;
    store_bf16_vec<VEC>(k_cache + off, k_tok);
    copy_bf16_vec<VEC>(v_cache + off, v_new);
  }
  // ---- the CTA's warps merge through shared memory into one partial per CTA ----
#pragma unroll
  for (int g = 0; g < kAttnMaxG; ++g) {
    if (g < G) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) sm[warp][g][lane * VEC + j] = acc[g][j];
    }
  }
  if (lane < kAttnMaxG) {                               // lane g holds head g's maximum and sum
    sm[warp][lane][D] = m_run;
    sm[warp][lane][D + 1] = l_run;
  }
  __syncthreads();
  float* mine = scratch + ((size_t)bh * n_split + split) * kAttnMaxG * kRow;
  for (int item = threadIdx.x; item < G * D; item += kAttnWarps * 32) {
    const int g = item / D, d = item - g * D;
    float a, mm, ll;
    merge_partials(&sm[0][g][D], &sm[0][g][D + 1], &sm[0][g][d], kAttnWarps, kAttnMaxG * kRow, a, mm, ll);
    mine[g * kRow + d] = a;
    if (d == 0) {
      mine[g * kRow + D] = mm;
      mine[g * kRow + D + 1] = ll;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&counters[bh], 1u) == (unsigned int)(n_split - 1);
  __syncthreads();
  if (!is_last) return;
  // ---- the last CTA of this (b, kv head) merges the CTAs' partials ----
  // Warp g first turns head g's maxima and sums of the splits into one weight per split (a lane
  // takes up to two splits) and the head's total; then every thread adds up its (head, dimension)
  // items over the splits with those weights, eight splits' loads in flight for each of its items.
  __threadfence();
  static_assert(kAttnWarps >= kAttnMaxG && kAttnMaxSplit <= 64, "a warp per head, two splits per lane");
  const float* all = scratch + (size_t)bh * n_split * kAttnMaxG * kRow;
  if (warp < G) {
    const int g = warp;
    float mv[2], lv[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = lane + 32 * u;
      const float* rec = all + ((size_t)i * kAttnMaxG + g) * kRow + D;
      mv[u] = i < n_split ? __ldcg(rec) : kNoScore;
      lv[u] = i < n_split ? __ldcg(rec + 1) : 0.f;
    }
    float big = fmaxf(mv[0], mv[1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, o));
    float total = 0.f;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = lane + 32 * u;
      const float w = i < n_split ? __expf(mv[u] - big) : 0.f;   // 0 for a split that saw no position while another did
      split_w[g][i] = w;
      total += w * lv[u];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if (lane == 0) head_sum[g] = total;
  }
  __syncthreads();
  constexpr int kItems = kAttnMaxG * D / (kAttnWarps * 32);   // (head, dimension) items per thread at most
  float tot[kItems];
#pragma unroll
  for (int t = 0; t < kItems; ++t) tot[t] = 0.f;
#pragma unroll 8
  for (int i = 0; i < n_split; ++i) {
#pragma unroll
    for (int t = 0; t < kItems; ++t) {
      const int item = threadIdx.x + t * kAttnWarps * 32;
      if (item < G * D) {
        const int g = item / D, d = item - g * D;
        tot[t] += split_w[g][i] * __ldcg(all + ((size_t)i * kAttnMaxG + g) * kRow + d);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kItems; ++t) {
    const int item = threadIdx.x + t * kAttnWarps * 32;
    if (item < G * D) {
      const int g = item / D, d = item - g * D;
      out[((size_t)b * hq + kvh * G + g) * D + d] = __float2bfloat16_rn(tot[t] / head_sum[g]);
    }
  }
  if (threadIdx.x == 0) counters[bh] = 0u;            // ready for the next launch
}

int grid_for(long long items, int threads, int num_sms) {
  long long blocks = (items + threads - 1) / threads;
  const long long cap = (long long)num_sms * 8;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int launch_rms_norm(const void* x, const void* residual, const void* w, void* sum_out, void* out, int rows, int H,
                    float eps, cudaStream_t stream) {
  if (rows < 0 || H <= 0 || H % 8 != 0) return cudaErrorInvalidValue;
  if (!aligned16(x) || !aligned16(w) || !aligned16(out) || (residual && !aligned16(residual)) ||
      (sum_out && !aligned16(sum_out)))
    return cudaErrorInvalidValue;
  if (sum_out != nullptr && residual == nullptr) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  rms_norm_kernel<<<rows, kNormThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(out),
      H, eps);
  return (int)cudaGetLastError();
}

int launch_rope_inplace(void* qkv, long long tokens, int row_stride, int n_heads, int head_dim, int seq, int pos0,
                        const int* pos_dev, float theta, int num_sms, cudaStream_t stream) {
  if (tokens < 0 || n_heads < 1 || head_dim < 16 || head_dim % 16 != 0 || seq < 1 || row_stride % 8 != 0 ||
      (long long)n_heads * head_dim > row_stride || theta <= 1.0f || !aligned16(qkv))
    return cudaErrorInvalidValue;
  if (tokens == 0) return cudaSuccess;
  const long long items = tokens * n_heads * (head_dim / 16);
  rope_kernel<<<grid_for(items, 256, num_sms), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(qkv), items, row_stride,
                                                                n_heads, head_dim, seq, pos0, pos_dev, log2f(theta));
  return (int)cudaGetLastError();
}

int launch_silu_mul(const void* gate_up, void* out, long long rows, int F, int num_sms, cudaStream_t stream) {
  if (rows < 0 || F <= 0 || F % 8 != 0 || !aligned16(gate_up) || !aligned16(out)) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  const long long n_vec = rows * (F / 8);
  silu_mul_kernel<<<grid_for(n_vec, 256, num_sms), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(gate_up),
                                                                    static_cast<__nv_bfloat16*>(out), n_vec, F);
  return (int)cudaGetLastError();
}

size_t decode_attention_scratch_bytes(int batch, int hkv, int head_dim, int s_max, int* n_split_out) {
  // about two CTAs per SM over all (b, kv head); a CTA's eight warps take four positions at a time, so
  // a split shorter than 64 positions is not worth a CTA; few enough splits for one CTA to combine them
  // (rounded down: 296 CTAs of 256 threads and 128 registers are what 148 SMs hold at once, and a few
  // CTAs left for a second wave would double the kernel's time)
  const int rows = batch * hkv > 0 ? batch * hkv : 1;
  int n_split = 296 / rows;
  const int by_length = (s_max + 63) / 64;
  if (n_split > by_length) n_split = by_length;
  n_split = n_split < 1 ? 1 : (n_split > kAttnMaxSplit ? kAttnMaxSplit : n_split);
  if (n_split_out) *n_split_out = n_split;
  const size_t partials = (size_t)batch * hkv * n_split * kAttnMaxG * (head_dim + 2) * sizeof(float);
  return 256 + ((size_t)batch * hkv * sizeof(unsigned int) + 255) / 256 * 256 + partials;
}

int launch_decode_attention(const void* qkv, void* k_cache, void* v_cache, void* out, void* scratch,
                            size_t scratch_bytes, int batch, int hq, int hkv, int head_dim, int s_max, int pos0,
                            const int* pos_dev, float rope_theta, cudaStream_t stream) {
  if (rope_theta != 0.f && rope_theta <= 1.0f) return cudaErrorInvalidValue;
  const float log2_theta = rope_theta != 0.f ? log2f(rope_theta) : 0.f;
  if (batch < 1 || hq < 1 || hkv < 1 || hq % hkv != 0 || hq / hkv > kAttnMaxG || (head_dim != 64 && head_dim != 128) ||
      s_max < 1 || (pos_dev == nullptr && (pos0 < 0 || pos0 >= s_max)))
    return cudaErrorInvalidValue;
  if (!aligned16(qkv) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out) || !aligned16(scratch))
    return cudaErrorInvalidValue;
  int n_split = 1;
  if (decode_attention_scratch_bytes(batch, hkv, head_dim, s_max, &n_split) > scratch_bytes) return cudaErrorInvalidValue;
  // layout of the scratch: [0, 256) unused, then one arrival counter per (b, kv head) (zero between
  // launches: the combining CTA resets it), then the partials
  unsigned int* counters = reinterpret_cast<unsigned int*>(static_cast<char*>(scratch) + 256);
  const size_t counter_bytes = ((size_t)batch * hkv * sizeof(unsigned int) + 255) / 256 * 256;
  float* partials = reinterpret_cast<float*>(static_cast<char*>(scratch) + 256 + counter_bytes);
  const dim3 grid((unsigned)(batch * hkv), (unsigned)n_split);
  const float scale = 1.0f / sqrtf((float)head_dim);
  auto q = static_cast<const __nv_bfloat16*>(qkv);
  auto kc = static_cast<__nv_bfloat16*>(k_cache);
  auto vc = static_cast<__nv_bfloat16*>(v_cache);
  auto o = static_cast<__nv_bfloat16*>(out);
  if (head_dim == 128)
    decode_attention_kernel<4><<<grid, kAttnWarps * 32, 0, stream>>>(q, kc, vc, o, partials, counters, hq, hkv, s_max,
                                                                      pos0, pos_dev, scale, log2_theta);
  else
    decode_attention_kernel<2><<<grid, kAttnWarps * 32, 0, stream>>>(q, kc, vc, o, partials, counters, hq, hkv, s_max,
                                                                      pos0, pos_dev, scale, log2_theta);
  return (int)cudaGetLastError();
}

}  // namespace smr
