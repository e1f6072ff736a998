// Rank-local pieces of a Llama-style decoder layer that sit between the fused
// GEMM + collective kernels: RMSNorm (optionally fused with the residual add
// that precedes it), rotary embedding in place on the QKV buffer, and
// SiLU(gate) * up.  Each is one pass over its operand in bf16 with fp32 math;
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

}  // namespace smr
