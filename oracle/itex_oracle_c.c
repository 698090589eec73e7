/*
 * CPU restatement (plain C + OpenMP) of the ITEX quantized-inference device arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY: the checker and the timed CPU baseline.  The CUDA library
 * never links or calls this file.  It restates what the reference executes through
 * oneDNN for the hot path (scalar host math stays in oracle/itex_oracle.py):
 *   - reorder f32 -> s8/u8 with a source scale         itex/core/kernels/common/quantize_op.h:256-275,394
 *   - reorder s8/u8 -> f32                             itex/core/kernels/common/dequantize_op.h:143-169
 *   - int8 inner product, scale on weights, bias after itex/core/kernels/common/quantized_matmul_common.h:223-226,92
 *   - int8 NHWC convolution with the same tail         itex/core/kernels/common/conv_ops.h:953-957,801
 * Build with -ffp-contract=off: fp32 multiply and add stay separate.
 * Parity: pinned against the NumPy twin (itself pinned to the reference's known-answer
 * tests and to real oneDNN) by tests/test_oracle_c.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define EXPORT __attribute__((visibility("default")))

EXPORT int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

static inline int sat_rne(float f, float lo, float hi) {
  if (f != f) return 0;
  if (f < lo) f = lo;
  if (f > hi) f = hi;
  return (int)nearbyintf(f);
}

/* q[i] = sat(rne(x[i] * scale[(i / inner) % nslice])) */
EXPORT void oracle_quantize_scaled(const float* x, int64_t n, int64_t inner, int64_t nslice, const float* scale,
                                   int is_signed, uint8_t* q) {
  const float lo = is_signed ? -128.f : 0.f, hi = is_signed ? 127.f : 255.f;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const float s = nslice > 1 ? scale[(i / inner) % nslice] : scale[0];
    q[i] = (uint8_t)sat_rne(x[i] * s, lo, hi);
  }
}

/* y[i] = (float(q[i]) - zp) * scale */
EXPORT void oracle_dequantize(const uint8_t* q, int64_t n, int64_t inner, int64_t nslice, const float* scale,
                              const float* zp, int is_signed, float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const int64_t c = nslice > 1 ? (i / inner) % nslice : 0;
    const float f = is_signed ? (float)(int8_t)q[i] : (float)q[i];
    y[i] = (f - (zp ? zp[c] : 0.f)) * scale[c];
  }
}

/* acc[m][n] = sum_k a[m][k] * b_nk[n][k]   (a unsigned or signed 8-bit, b signed 8-bit; exact) */
EXPORT void oracle_gemm_acc(const uint8_t* a, int a_signed, const int8_t* b_nk, int64_t m, int64_t n, int64_t k,
                            int32_t* acc) {
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t i = 0; i < m; ++i) {
    const uint8_t* ar = a + i * k;
    for (int64_t j = 0; j < n; ++j) {
      const int8_t* br = b_nk + j * k;
      int32_t s = 0;
      if (a_signed) {
        for (int64_t t = 0; t < k; ++t) s += (int32_t)(int8_t)ar[t] * (int32_t)br[t];
      } else {
        for (int64_t t = 0; t < k; ++t) s += (int32_t)ar[t] * (int32_t)br[t];
      }
      acc[i * n + j] = s;
    }
  }
}

/* The primitive's tail: f = float(acc) * scale[n|0]; f += bias[n]; relu; convert.
 * out_kind: 0 f32, 1 u8, 2 s8, 3 s32.  scale_count 0 = no multiply. */
EXPORT void oracle_epilogue(const int32_t* acc, int64_t m, int64_t n, const float* scale, int64_t scale_count,
                            const float* bias, int relu, int out_kind, void* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      float f = (float)acc[i * n + j];
      if (scale_count > 0) f = f * scale[scale_count > 1 ? j : 0];
      if (bias) f = f + bias[j];
      if (relu && f < 0.f) f = 0.f;
      const int64_t o = i * n + j;
      switch (out_kind) {
        case 0: ((float*)out)[o] = f; break;
        case 1: ((uint8_t*)out)[o] = (uint8_t)sat_rne(f, 0.f, 255.f); break;
        case 2: ((int8_t*)out)[o] = (int8_t)sat_rne(f, -128.f, 127.f); break;
        default: {
          double d = f != f ? 0.0 : (double)f;
          if (d < -2147483648.0) d = -2147483648.0;
          if (d > 2147483647.0) d = 2147483647.0;
          ((int32_t*)out)[o] = (int32_t)nearbyint(d);
        }
      }
    }
  }
}

/* Fused convenience for timing: quantize-free GEMM + tail without materialising acc for all rows at once. */
EXPORT void oracle_gemm_fused(const uint8_t* a, int a_signed, const int8_t* b_nk, int64_t m, int64_t n, int64_t k,
                              const float* scale, int64_t scale_count, const float* bias, int relu, int out_kind, void* out) {
  int32_t* acc = (int32_t*)malloc((size_t)m * n * sizeof(int32_t));
  oracle_gemm_acc(a, a_signed, b_nk, m, n, k, acc);
  oracle_epilogue(acc, m, n, scale, scale_count, bias, relu, out_kind, out);
  free(acc);
}

/* NHWC x [co][kh][kw][c] (filter packed output-channel major) int32 convolution, zero padding. */
EXPORT void oracle_conv_acc(const uint8_t* x, int x_signed, const int8_t* f_okkc, int64_t nb, int64_t h, int64_t w, int64_t c,
                            int64_t kh, int64_t kw, int64_t co, int64_t sh, int64_t sw, int64_t dh, int64_t dw, int64_t pt,
                            int64_t pl, int64_t oh, int64_t ow, int32_t* acc) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < nb; ++b)
    for (int64_t oy = 0; oy < oh; ++oy)
      for (int64_t ox = 0; ox < ow; ++ox) {
        int32_t* dst = acc + ((b * oh + oy) * ow + ox) * co;
        for (int64_t o = 0; o < co; ++o) {
          int32_t s = 0;
          for (int64_t ky = 0; ky < kh; ++ky) {
            const int64_t iy = oy * sh + ky * dh - pt;
            if (iy < 0 || iy >= h) continue;
            for (int64_t kx = 0; kx < kw; ++kx) {
              const int64_t ix = ox * sw + kx * dw - pl;
              if (ix < 0 || ix >= w) continue;
              const uint8_t* xp = x + ((b * h + iy) * w + ix) * c;
              const int8_t* fp = f_okkc + ((o * kh + ky) * kw + kx) * c;
              if (x_signed) {
                for (int64_t ci = 0; ci < c; ++ci) s += (int32_t)(int8_t)xp[ci] * (int32_t)fp[ci];
              } else {
                for (int64_t ci = 0; ci < c; ++ci) s += (int32_t)xp[ci] * (int32_t)fp[ci];
              }
            }
          }
          dst[o] = s;
        }
      }
}
