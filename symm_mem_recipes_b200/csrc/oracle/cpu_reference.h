// CPU oracles: the arithmetic contract of every kernel, in plain C++.
//
//  * ordered bf16 sum: acc = +0; acc = bf16(acc + x_r) for r = 0..WS-1, one
//    round-to-nearest-even per add.  Bit-for-bit what the one-shot and
//    two-shot kernels (and symm_mem_recipes/triton_one_shot_all_reduce.py:84-89)
//    compute.
//  * fp32 sum: accumulate in fp32 in rank order, round to bf16 once (what the
//    NVSwitch does for multimem.ld_reduce with .acc::f32, up to its own
//    summation order).
//  * GEMM / GEMV: fp32 accumulate over K, round to bf16 once.
//  * RMSNorm, rotary embedding, SiLU-mul: fp32 math on bf16 data, rounding
//    where the kernels round.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace smr {

inline float bf16_to_f32(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  __builtin_memcpy(&f, &u, 4);
  return f;
}
// round to nearest even; NaN stays NaN
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  __builtin_memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

// out[i] = ordered bf16 sum over srcs[0..n_src)
void ordered_sum_bf16(const uint16_t* const* srcs, int n_src, uint16_t* out, size_t numel);
// out[i] = bf16( sum_r float(srcs[r][i]) )
void fp32_sum_bf16(const uint16_t* const* srcs, int n_src, uint16_t* out, size_t numel);
// C[M,N] = A[M,K] * B[N,K]^T, bf16 in, fp32 accumulate, bf16 out (row-major)
void gemm_nt_bf16(const uint16_t* a, const uint16_t* b, uint16_t* c, int M, int N, int K);
// y[B,N] (fp32) = x[B,K] * w[K,N]
void gemv_f32(const uint16_t* x, const uint16_t* w, float* y, int B, int K, int N);

// Layer glue (kernels/layer_glue.cu), same rounding points as the kernels:
// s = x (+ r, rounded to bf16, stored to sum_out when given);
// out = bf16( bf16(s * rsqrt(mean(s^2) + eps)) * w )
void rms_norm_bf16(const uint16_t* x, const uint16_t* residual, const uint16_t* w, uint16_t* sum_out,
                   uint16_t* out, int rows, int H, float eps);
// in place: heads [0, n_heads) of every row of `row_stride` elements, pairs (i, i + D/2),
// angle = (pos0 + t % seq) * theta^(-2i/D)
void rope_bf16(uint16_t* qkv, long long tokens, int row_stride, int n_heads, int D, int seq, int pos0, float theta);
// out[T, F] = bf16( silu(gu[:, :F]) * gu[:, F:] )
void silu_mul_bf16(const uint16_t* gu, uint16_t* out, long long rows, int F);
// One decode step of attention for this rank's heads.  qkv [B, (hq + 2 hkv) * D] holds the new
// token's (already rotated) queries and keys and its values; caches are [B, s_max, hkv, D].  Writes
// the new key / value rows into the caches at `pos`, then out[b, h] = softmax(q_h . K[0..pos] /
// sqrt(D)) V[0..pos] for every query head h (head h reads KV head h / (hq / hkv)); fp32 math, bf16 out.
void decode_attention_bf16(const uint16_t* qkv, uint16_t* k_cache, uint16_t* v_cache, uint16_t* out, int B, int hq,
                           int hkv, int D, int s_max, int pos);

}  // namespace smr
