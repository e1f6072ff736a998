#include "cpu_reference.h"

#include <cmath>
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

void rms_norm_bf16(const uint16_t* x, const uint16_t* residual, const uint16_t* w, uint16_t* sum_out,
                   uint16_t* out, int rows, int H, float eps) {
  std::vector<float> s((size_t)H);
  for (int r = 0; r < rows; ++r) {
    const size_t o = (size_t)r * H;
    double ss = 0.0;
    for (int i = 0; i < H; ++i) {
      float v = bf16_to_f32(x[o + i]);
      if (residual != nullptr) {
        uint16_t sum = f32_to_bf16(v + bf16_to_f32(residual[o + i]));
        if (sum_out != nullptr) sum_out[o + i] = sum;
        v = bf16_to_f32(sum);
      }
      s[i] = v;
      ss += (double)v * v;
    }
    const float scale = 1.0f / std::sqrt((float)(ss / H) + eps);
    for (int i = 0; i < H; ++i) {
      const float n = bf16_to_f32(f32_to_bf16(s[i] * scale));
      out[o + i] = f32_to_bf16(n * bf16_to_f32(w[i]));
    }
  }
}

void rope_bf16(uint16_t* qkv, long long tokens, int row_stride, int n_heads, int D, int seq, int pos0, float theta) {
  const int half = D / 2;
  for (long long t = 0; t < tokens; ++t) {
    const double pos = (double)(pos0 + (int)(t % seq));
    for (int h = 0; h < n_heads; ++h) {
      uint16_t* base = qkv + t * row_stride + (long long)h * D;
      for (int i = 0; i < half; ++i) {
        const double ang = pos * std::pow((double)theta, -2.0 * i / D);
        const float cs = (float)std::cos(ang), sn = (float)std::sin(ang);
        const float x1 = bf16_to_f32(base[i]), x2 = bf16_to_f32(base[i + half]);
        base[i] = f32_to_bf16(x1 * cs - x2 * sn);
        base[i + half] = f32_to_bf16(x2 * cs + x1 * sn);
      }
    }
  }
}

void silu_mul_bf16(const uint16_t* gu, uint16_t* out, long long rows, int F) {
  for (long long r = 0; r < rows; ++r)
    for (int c = 0; c < F; ++c) {
      const float g = bf16_to_f32(gu[r * 2 * F + c]), u = bf16_to_f32(gu[r * 2 * F + F + c]);
      out[r * F + c] = f32_to_bf16(g / (1.0f + std::exp(-g)) * u);
    }
}

void decode_attention_bf16(const uint16_t* qkv, uint16_t* k_cache, uint16_t* v_cache, uint16_t* out, int B, int hq,
                           int hkv, int D, int s_max, int pos) {
  const int row = (hq + 2 * hkv) * D, G = hq / hkv;
  const float scale = 1.0f / std::sqrt((float)D);
  std::vector<float> score((size_t)pos + 1), acc((size_t)D);
  for (int b = 0; b < B; ++b) {
    const uint16_t* r = qkv + (size_t)b * row;
    for (int kvh = 0; kvh < hkv; ++kvh) {
      uint16_t* kc = k_cache + (((size_t)b * s_max + pos) * hkv + kvh) * D;
      uint16_t* vc = v_cache + (((size_t)b * s_max + pos) * hkv + kvh) * D;
      for (int d = 0; d < D; ++d) {
        kc[d] = r[(size_t)hq * D + (size_t)kvh * D + d];
        vc[d] = r[(size_t)(hq + hkv) * D + (size_t)kvh * D + d];
      }
    }
    for (int h = 0; h < hq; ++h) {
      const int kvh = h / G;
      const uint16_t* q = r + (size_t)h * D;
      float m = -INFINITY;
      for (int p = 0; p <= pos; ++p) {
        const uint16_t* k = k_cache + (((size_t)b * s_max + p) * hkv + kvh) * D;
        float s = 0.f;
        for (int d = 0; d < D; ++d) s += bf16_to_f32(q[d]) * bf16_to_f32(k[d]);
        score[p] = s * scale;
        m = std::max(m, score[p]);
      }
      float l = 0.f;
      std::fill(acc.begin(), acc.end(), 0.f);
      for (int p = 0; p <= pos; ++p) {
        const float w = std::exp(score[p] - m);
        const uint16_t* v = v_cache + (((size_t)b * s_max + p) * hkv + kvh) * D;
        l += w;
        for (int d = 0; d < D; ++d) acc[d] += w * bf16_to_f32(v[d]);
      }
      for (int d = 0; d < D; ++d) out[((size_t)b * hq + h) * D + d] = f32_to_bf16(acc[d] / l);
    }
  }
}

}  // namespace smr
