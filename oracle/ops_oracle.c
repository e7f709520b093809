/*
 * CPU oracle, half 2: the operator arithmetic of the fused pairs, as plain loops
 * (OpenMP over rows / output tiles).  TEST INFRASTRUCTURE ONLY -- never linked
 * into the shipped library; it is the checker for the CUDA path and the timed
 * CPU baseline of the benchmark.
 *
 * Parity unpinned: the reference ships no CPU implementation and no golden
 * outputs for any operator (its own check is fused-vs-unfused on the GPU,
 * test-utils/test-suite-files/utils_cc.py:52-86), so these loops follow the op
 * definitions in the reference's Relay dumps (cited per function in the header).
 */
#include "bfuse_oracle.h"

#include <float.h>
#include <math.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

float orc_bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round to nearest even, NaN kept quiet */
uint16_t orc_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline float tf32_trunc(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u &= 0xffffe000u;
  memcpy(&f, &u, 4);
  return f;
}

void orc_softmax_f32(const float *x, float *y, int rows, int cols, float scale) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float *xr = x + (size_t)r * cols;
    float *yr = y + (size_t)r * cols;
    float m = -INFINITY;
    for (int c = 0; c < cols; ++c) m = fmaxf(m, xr[c] * scale);
    float s = 0.f;
    for (int c = 0; c < cols; ++c) {
      yr[c] = expf(xr[c] * scale - m);
      s += yr[c];
    }
    float inv = 1.f / s;
    for (int c = 0; c < cols; ++c) yr[c] *= inv;
  }
}

void orc_layernorm_f32(const float *x, const float *res, const float *gamma, const float *beta,
                       float *y, int rows, int cols, float eps) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float *xr = x + (size_t)r * cols;
    const float *rr = res ? res + (size_t)r * cols : NULL;
    float *yr = y + (size_t)r * cols;
    double sum = 0.0;
    for (int c = 0; c < cols; ++c) sum += rr ? xr[c] + rr[c] : xr[c];
    float mean = (float)(sum / cols);
    double sq = 0.0;
    for (int c = 0; c < cols; ++c) {
      float v = (rr ? xr[c] + rr[c] : xr[c]) - mean;
      sq += (double)v * v;
    }
    float rstd = 1.f / sqrtf((float)(sq / cols) + eps);
    for (int c = 0; c < cols; ++c) {
      float v = rr ? xr[c] + rr[c] : xr[c];
      yr[c] = (v - mean) * rstd * gamma[c] + beta[c];
    }
  }
}

void orc_rmsnorm_bf16(const uint16_t *x, const uint16_t *w, uint16_t *y, int rows, int cols, float eps) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const uint16_t *xr = x + (size_t)r * cols;
    uint16_t *yr = y + (size_t)r * cols;
    double sq = 0.0;
    for (int c = 0; c < cols; ++c) {
      float v = orc_bf16_to_f32(xr[c]);
      sq += (double)v * v;
    }
    float rinv = 1.f / sqrtf((float)(sq / cols) + eps);
    for (int c = 0; c < cols; ++c)
      yr[c] = orc_f32_to_bf16(orc_bf16_to_f32(xr[c]) * rinv * orc_bf16_to_f32(w[c]));
  }
}

void orc_rope_bf16(const uint16_t *q, const float *inv_freq, uint16_t *y, int seq, int heads, int dim) {
  int half = dim / 2;
#pragma omp parallel for schedule(static)
  for (int s = 0; s < seq; ++s) {
    for (int i = 0; i < half; ++i) {
      float ang = (float)s * inv_freq[i];
      float cs = cosf(ang), sn = sinf(ang);
      for (int h = 0; h < heads; ++h) {
        size_t o = ((size_t)s * heads + h) * dim;
        float a = orc_bf16_to_f32(q[o + i]);
        float b = orc_bf16_to_f32(q[o + i + half]);
        /* x*cos + rotate_half(x)*sin, rotate_half = concat(-x[half:], x[:half]) */
        y[o + i] = orc_f32_to_bf16(a * cs - b * sn);
        y[o + i + half] = orc_f32_to_bf16(b * cs + a * sn);
      }
    }
  }
}

void orc_gemm_nt_f32(const float *A, const float *W, const float *bias, float *out,
                     int batch, int M, int N, int K, int causal, int tf32) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batch; ++b) {
    for (int m = 0; m < M; ++m) {
      const float *a = A + ((size_t)b * M + m) * K;
      float *o = out + ((size_t)b * M + m) * N;
      for (int n = 0; n < N; ++n) {
        if (causal && n > m) {
          o[n] = -FLT_MAX;
          continue;
        }
        const float *w = W + ((size_t)b * N + n) * K;
        float acc = 0.f;
        if (tf32) {
#pragma omp simd reduction(+ : acc)
          for (int k = 0; k < K; ++k) acc += tf32_trunc(a[k]) * tf32_trunc(w[k]);
        } else {
#pragma omp simd reduction(+ : acc)
          for (int k = 0; k < K; ++k) acc += a[k] * w[k];
        }
        o[n] = bias ? acc + bias[n] : acc;
      }
    }
  }
}

void orc_gemm_nt_bf16(const uint16_t *A, const uint16_t *W, uint16_t *out, int batch, int M, int N, int K) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batch; ++b) {
    for (int m = 0; m < M; ++m) {
      const uint16_t *a = A + ((size_t)b * M + m) * K;
      uint16_t *o = out + ((size_t)b * M + m) * N;
      for (int n = 0; n < N; ++n) {
        const uint16_t *w = W + ((size_t)b * N + n) * K;
        float acc = 0.f;
#pragma omp simd reduction(+ : acc)
        for (int k = 0; k < K; ++k) {
          uint32_t ua = (uint32_t)a[k] << 16, uw = (uint32_t)w[k] << 16;
          float fa, fw;
          memcpy(&fa, &ua, 4);
          memcpy(&fw, &uw, 4);
          acc += fa * fw;
        }
        o[n] = orc_f32_to_bf16(acc);
      }
    }
  }
}

void orc_conv2d_nchw_f32(const float *x, const float *w, float *y, int n, int ci, int h, int wd,
                         int co, int kh, int kw, int stride, int pad, int tf32) {
  int oh = (h + 2 * pad - kh) / stride + 1;
  int ow = (wd + 2 * pad - kw) / stride + 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < n; ++b) {
    for (int oc = 0; oc < co; ++oc) {
      for (int y0 = 0; y0 < oh; ++y0) {
        for (int x0 = 0; x0 < ow; ++x0) {
          float acc = 0.f;
          for (int c = 0; c < ci; ++c) {
            for (int r = 0; r < kh; ++r) {
              int iy = y0 * stride + r - pad;
              if (iy < 0 || iy >= h) continue;
              for (int s = 0; s < kw; ++s) {
                int ix = x0 * stride + s - pad;
                if (ix < 0 || ix >= wd) continue;
                float xv = x[(((size_t)b * ci + c) * h + iy) * wd + ix];
                float wv = w[(((size_t)oc * ci + c) * kh + r) * kw + s];
                if (tf32) {
                  xv = tf32_trunc(xv);
                  wv = tf32_trunc(wv);
                }
                acc += xv * wv;
              }
            }
          }
          y[(((size_t)b * co + oc) * oh + y0) * ow + x0] = acc;
        }
      }
    }
  }
}
