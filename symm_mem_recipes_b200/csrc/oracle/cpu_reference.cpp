#include "cpu_reference.h"

#include <vector>

namespace smr {

void ordered_sum_bf16(const uint16_t* const* srcs, int n_src, uint16_t* out, size_t numel) {
  for (size_t i = 0; i < numel; ++i) {
    uint16_t acc = 0;  // +0
    for (int r = 0; r < n_src; ++r) acc = f32_to_bf16(bf16_to_f32(acc) + bf16_to_f32(srcs[r][i]));
    out[i] = acc;
  }
}

void fp32_sum_bf16(const uint16_t* const* srcs, int n_src, uint16_t* out, size_t numel) {
  for (size_t i = 0; i < numel; ++i) {
    float acc = 0.f;
    for (int r = 0; r < n_src; ++r) acc += bf16_to_f32(srcs[r][i]);
    out[i] = f32_to_bf16(acc);
  }
}

void gemm_nt_bf16(const uint16_t* a, const uint16_t* b, uint16_t* c, int M, int N, int K) {
  std::vector<float> af((size_t)M * K), bf((size_t)N * K);
  for (size_t i = 0; i < af.size(); ++i) af[i] = bf16_to_f32(a[i]);
  for (size_t i = 0; i < bf.size(); ++i) bf[i] = bf16_to_f32(b[i]);
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      const float* ar = &af[(size_t)m * K];
      const float* br = &bf[(size_t)n * K];
      float acc = 0.f;
      for (int k = 0; k < K; ++k) acc += ar[k] * br[k];
      c[(size_t)m * N + n] = f32_to_bf16(acc);
    }
}

void gemv_f32(const uint16_t* x, const uint16_t* w, float* y, int B, int K, int N) {
  for (int b = 0; b < B; ++b) {
    float* yr = y + (size_t)b * N;
    for (int n = 0; n < N; ++n) yr[n] = 0.f;
    for (int k = 0; k < K; ++k) {
      float xv = bf16_to_f32(x[(size_t)b * K + k]);
      const uint16_t* wr = w + (size_t)k * N;
      for (int n = 0; n < N; ++n) yr[n] += xv * bf16_to_f32(wr[n]);
    }
  }
}

}  // namespace smr
