/*
 * CPU oracle for the quantized-linear path of onnx-mlir: see oracle.h.
 *
 * TEST INFRASTRUCTURE ONLY: used by tests/, the smoke check and the
 * cpu_baseline / reference arm of the benchmark as the checker and the timed
 * CPU side.  The CUDA library never calls into this file.
 *
 * Build with: gcc -O2 -fno-fast-math -ffp-contract=off -fopenmp -fPIC -shared
 * (contraction must stay off: the reference emits separate arith.mulf /
 * arith.addf and nothing in its pipeline fuses them).
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* Scalar pieces                                                             */
/* ------------------------------------------------------------------------ */

/* arith.minnumf / arith.maxnumf (src/Dialect/Mlir/DialectBuilder.cpp:462-484):
 * if one operand is NaN the other is returned.  C's fminf/fmaxf have the same
 * rule. */
static inline float minnum(float a, float b) { return fminf(a, b); }
static inline float maxnum(float a, float b) { return fmaxf(a, b); }

/* MathBuilder::clip (DialectBuilder.cpp:355-360): max with lb, then min with
 * ub. */
static inline float clipf(float v, float lb, float ub) {
  v = maxnum(v, lb);
  return minnum(v, ub);
}

/* MathBuilder::roundEvenEmulation (DialectBuilder.cpp:291-335); the op
 * sequence is the one the lit test
 * test/mlir/conversion/onnx_to_krnl/Quantization/DynamicQuantizeLinear_with_canonicalize.mlir:95-108
 * pins. */
float orc_round_even(float x) {
  float y = floorf(x);
  float r = x - y;
  float y1 = (r > 0.5f) ? (y + 1.0f) : y;
  float y2 = 0.5f * y;
  y2 = floorf(y2);
  y2 = y2 * 2.0f;
  float rr = y - y2;
  y2 = (rr == 1.0f) ? (y + 1.0f) : y;
  return (r == 0.5f) ? y2 : y1;
}

/* ------------------------------------------------------------------------ */
/* DynamicQuantizeLinear                                                     */
/* ------------------------------------------------------------------------ */

/* The reference's two non-default arithmetic modes, compile-time flags there:
 *   ORC_MODE_NO_ZERO_POINT  --disable-quantization-zero-point: zero point 0 in
 *       DynamicQuantizeLinear (DynamicQuantizeLinear.cpp:72-83,142), a given
 *       zero point ignored by QuantizeLinear (QuantizeLinear.cpp:231-237) and
 *       by DequantizeLinear (Math/Elementwise.cpp:1453);
 *   ORC_MODE_FAST_MATH  convert-onnx-to-krnl=enable-fast-math: x / scale
 *       becomes x * (1 / scale) (QuantizeLinear.cpp:43-44,117-131).
 * The lit tests Quantization/QuantizationWithoutZeroPoint.mlir and
 * QuantizeLinear_with_fast_math_canonicalize.mlir pin both. */
static int g_quant_mode = 0;
void orc_set_quant_mode(int flags) { g_quant_mode = flags; }

void orc_minmax_f32(const float *x, int64_t n, float *mn, float *mx) {
  float lo = INFINITY, hi = -INFINITY;
  for (int64_t i = 0; i < n; ++i) {
    lo = minnum(lo, x[i]);
    hi = maxnum(hi, x[i]);
  }
  *mn = lo;
  *mx = hi;
}

void orc_dql_params(
    float mn, float mx, float *scale, float *zp_f, uint8_t *zp) {
  const float qmin = 0.0f, qmax = 255.0f;
  float xmax = maxnum(mx, 0.0f);
  float xmin = minnum(mn, 0.0f);
  float xdiff = xmax - xmin;
  float bound = qmax - qmin;
  float s = xdiff / bound;
  float inter = qmin - xmin / s;
  float sat = clipf(inter, qmin, qmax); /* saturate first ... */
  float z = orc_round_even(sat);        /* ... then round (:77-79) */
  if (g_quant_mode & ORC_MODE_NO_ZERO_POINT)
    z = 0.0f;
  *scale = s;
  *zp_f = z;
  /* math.cast f32 -> ui8: fptoui to 32 bits, then truncate
   * (DialectBuilder.cpp:951-966,1028-1032). */
  *zp = (uint8_t)(uint32_t)z;
}

void orc_quantize_u8(
    const float *x, int64_t n, float scale, float zp_f, uint8_t *y) {
  const int fast = (g_quant_mode & ORC_MODE_FAST_MATH) != 0;
  const int no_zp = (g_quant_mode & ORC_MODE_NO_ZERO_POINT) != 0;
  const float rcp = 1.0f / scale;
  for (int64_t i = 0; i < n; ++i) {
    float q = fast ? x[i] * rcp : x[i] / scale;
    float r = orc_round_even(q);
    float a = no_zp ? r : r + zp_f;
    float s = clipf(a, 0.0f, 255.0f);
    y[i] = (uint8_t)(uint32_t)s;
  }
}

void orc_quantize_i8(
    const float *x, int64_t n, float scale, float zp_f, int8_t *y) {
  const int fast = (g_quant_mode & ORC_MODE_FAST_MATH) != 0;
  const int no_zp = (g_quant_mode & ORC_MODE_NO_ZERO_POINT) != 0;
  const float rcp = 1.0f / scale;
  for (int64_t i = 0; i < n; ++i) {
    float q = fast ? x[i] * rcp : x[i] / scale;
    float r = orc_round_even(q);
    float a = no_zp ? r : r + zp_f;
    float s = clipf(a, -128.0f, 127.0f);
    y[i] = (int8_t)(int32_t)s;
  }
}

void orc_dynamic_quantize_linear(
    const float *x, int64_t n, uint8_t *y, float *scale, uint8_t *zp) {
  float mn, mx, zf;
  orc_minmax_f32(x, n, &mn, &mx);
  orc_dql_params(mn, mx, scale, &zf, zp);
  orc_quantize_u8(x, n, *scale, zf, y);
}

/* ------------------------------------------------------------------------ */
/* MatMulInteger / QLinearMatMul                                             */
/* ------------------------------------------------------------------------ */

static inline int32_t widen8(const void *p, int64_t i, int is_signed) {
  return is_signed ? (int32_t)((const int8_t *)p)[i]
                   : (int32_t)((const uint8_t *)p)[i];
}

void orc_matmul_integer(const void *A, int a_signed, const void *B,
    int b_signed, int64_t M, int64_t N, int64_t K, const void *a_zp,
    int64_t a_zp_len, const void *b_zp, int64_t b_zp_len, int32_t *Y) {
  /* BInt32 = Cast(B) - Cast(b_zp), materialised once like the lowering does
   * (:78-84).  Unsigned arithmetic below gives the two's-complement wrap of
   * arith.muli / arith.addi. */
  uint32_t *Bs = (uint32_t *)malloc((size_t)(K * N) * sizeof(uint32_t) + 4);
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < K; ++k) {
    for (int64_t n = 0; n < N; ++n) {
      int32_t bz = 0;
      if (b_zp_len == 1)
        bz = widen8(b_zp, 0, b_signed);
      else if (b_zp_len > 1)
        bz = widen8(b_zp, n, b_signed);
      Bs[k * N + n] = (uint32_t)(widen8(B, k * N + n, b_signed) - bz);
    }
  }
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    int32_t az = 0;
    if (a_zp_len == 1)
      az = widen8(a_zp, 0, a_signed);
    else if (a_zp_len > 1)
      az = widen8(a_zp, m, a_signed);
    uint32_t *acc = (uint32_t *)(Y + m * N);
    for (int64_t n = 0; n < N; ++n)
      acc[n] = 0u;
    for (int64_t k = 0; k < K; ++k) {
      uint32_t a = (uint32_t)(widen8(A, m * K + k, a_signed) - az);
      const uint32_t *brow = Bs + k * N;
      for (int64_t n = 0; n < N; ++n)
        acc[n] += a * brow[n];
    }
  }
  free(Bs);
}

/* OnnxBuilder::getOrCastToI8 (src/Dialect/ONNX/DialectBuilder.cpp:916-932):
 * unsigned 8-bit values are shifted by -128 through i16 and truncated to i8;
 * signed values pass through. */
static inline int32_t to_i8_domain(int32_t v, int is_signed) {
  if (is_signed)
    return v;
  return (int32_t)(int8_t)(int16_t)(v - 128);
}

void orc_qlinear_matmul(const void *A, int a_signed, float a_scale,
    int32_t a_zp, const void *B, int b_signed, const float *b_scale,
    const void *b_zp, int64_t b_q_len, float y_scale, int32_t y_zp,
    int y_signed, int64_t M, int64_t N, int64_t K, void *Y) {
  int32_t az = to_i8_domain(a_zp, a_signed);
  int32_t yz = to_i8_domain(y_zp, y_signed);
  /* BI32 = Cast(getOrCastToI8(B)) - Cast(getOrCastToI8(b_zp)) (:111-117). */
  uint32_t *Bs = (uint32_t *)malloc((size_t)(K * N) * sizeof(uint32_t) + 4);
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < K; ++k) {
    for (int64_t n = 0; n < N; ++n) {
      int64_t qi = (b_q_len > 1) ? n : 0;
      int32_t bz = to_i8_domain(widen8(b_zp, qi, b_signed), b_signed);
      int32_t b8 = to_i8_domain(widen8(B, k * N + n, b_signed), b_signed);
      Bs[k * N + n] = (uint32_t)(b8 - bz);
    }
  }
#pragma omp parallel
  {
    uint32_t *acc = (uint32_t *)malloc((size_t)N * sizeof(uint32_t) + 4);
#pragma omp for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
      for (int64_t n = 0; n < N; ++n)
        acc[n] = 0u;
      for (int64_t k = 0; k < K; ++k) {
        int32_t a8 = to_i8_domain(widen8(A, m * K + k, a_signed), a_signed);
        uint32_t a = (uint32_t)(a8 - az);
        const uint32_t *brow = Bs + k * N;
        for (int64_t n = 0; n < N; ++n)
          acc[n] += a * brow[n];
      }
      for (int64_t n = 0; n < N; ++n) {
        int64_t qi = (b_q_len > 1) ? n : 0;
        /* scale = (a_scale * b_scale) / y_scale, elementwise f32 (:127). */
        float s = (a_scale * b_scale[qi]) / y_scale;
        float f = (float)(int32_t)acc[n] * s;
        float r = orc_round_even(f);
        /* onnx.Cast f32 -> i32 is arith.fptosi; r is integral. */
        uint32_t t = (uint32_t)(int32_t)r + (uint32_t)yz;
        if (!y_signed)
          t += 128u; /* back to the unsigned domain, then trunc to 8 bits */
        ((uint8_t *)Y)[m * N + n] = (uint8_t)(t & 0xFFu);
      }
    }
    free(acc);
  }
  free(Bs);
}

/* ------------------------------------------------------------------------ */
/* Dequantization                                                            */
/* ------------------------------------------------------------------------ */

void orc_dequant_tail(const int32_t *acc, int64_t M, int64_t N, float s0,
    float s1, int form, const float *bias, float *y) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t n = 0; n < N; ++n) {
      float f = (float)acc[m * N + n]; /* arith.sitofp */
      float v = f * s0;
      if (form == 1)
        v = v * s1;
      if (bias)
        v = v + bias[n];
      y[m * N + n] = v;
    }
  }
}

void orc_dequantize_linear(
    const void *x, int dtype, int64_t n, float scale, int32_t zp, float *y) {
  float zf = (g_quant_mode & ORC_MODE_NO_ZERO_POINT) ? 0.0f : (float)zp;
  for (int64_t i = 0; i < n; ++i) {
    float xf;
    if (dtype == 0)
      xf = (float)((const uint8_t *)x)[i];
    else if (dtype == 1)
      xf = (float)((const int8_t *)x)[i];
    else
      xf = (float)((const int32_t *)x)[i];
    y[i] = (xf - zf) * scale;
  }
}

/* ------------------------------------------------------------------------ */
/* fp32 encoder ops                                                          */
/* ------------------------------------------------------------------------ */

void orc_softmax_lastdim(const float *x, int64_t rows, int64_t cols, float *y) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *yr = y + r * cols;
    float mx = -INFINITY;
    for (int64_t c = 0; c < cols; ++c)
      mx = maxnum(mx, xr[c]);
    float sum = 0.0f;
    for (int64_t c = 0; c < cols; ++c) {
      float e = expf(xr[c] - mx);
      sum = sum + e;
      yr[c] = e;
    }
    for (int64_t c = 0; c < cols; ++c)
      yr[c] = yr[c] / sum;
  }
}

void orc_layernorm(const float *x, int64_t rows, int64_t cols,
    const float *gamma, const float *beta, float eps, float *y) {
  float nf = (float)cols;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    float *yr = y + r * cols;
    float s = 0.0f, s2 = 0.0f;
    for (int64_t c = 0; c < cols; ++c) {
      s = s + xr[c];
      s2 = s2 + xr[c] * xr[c];
    }
    float mean = s / nf;
    float mean2 = s2 / nf;
    float var = mean2 - mean * mean;
    float inv = 1.0f / sqrtf(var + eps);
    for (int64_t c = 0; c < cols; ++c) {
      float v = (xr[c] - mean) * inv;
      v = v * gamma[c];
      if (beta)
        v = v + beta[c];
      yr[c] = v;
    }
  }
}

void orc_gelu(const float *x, int64_t n, float *y) {
  const float inv_sqrt2 = (float)(1.0 / sqrt(2.0));
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float h = 0.5f * x[i];
    float e = erff(x[i] * inv_sqrt2);
    y[i] = h * (1.0f + e);
  }
}

void orc_add(const float *a, const float *b, int64_t n, float *y) {
  for (int64_t i = 0; i < n; ++i)
    y[i] = a[i] + b[i];
}

void orc_transpose_0213(
    const float *x, int64_t B, int64_t S, int64_t H, int64_t D, float *y) {
  for (int64_t b = 0; b < B; ++b)
    for (int64_t s = 0; s < S; ++s)
      for (int64_t h = 0; h < H; ++h)
        memcpy(y + ((b * H + h) * S + s) * D, x + ((b * S + s) * H + h) * D,
            (size_t)D * sizeof(float));
}

void orc_matmul_f32(const float *A, const float *B, int64_t batch, int64_t M,
    int64_t N, int64_t K, float *C) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < batch; ++b) {
    for (int64_t m = 0; m < M; ++m) {
      const float *a = A + (b * M + m) * K;
      const float *bm = B + b * K * N;
      float *c = C + (b * M + m) * N;
      for (int64_t n = 0; n < N; ++n)
        c[n] = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        float av = a[k];
        for (int64_t n = 0; n < N; ++n)
          c[n] = c[n] + av * bm[k * N + n];
      }
    }
  }
}

void orc_attention(const float *Q, const float *K, const float *V, int64_t B,
    int64_t S, int64_t heads, int64_t dh, float scale, float *out) {
  int64_t H = heads * dh;
#pragma omp parallel
  {
    float *sc = (float *)malloc((size_t)S * sizeof(float));
#pragma omp for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b) {
      for (int64_t h = 0; h < heads; ++h) {
        for (int64_t i = 0; i < S; ++i) {
          const float *q = Q + (b * S + i) * H + h * dh;
          /* scores = Q K^T (sequential over d), then Mul by the constant. */
          for (int64_t j = 0; j < S; ++j) {
            const float *k = K + (b * S + j) * H + h * dh;
            float acc = 0.0f;
            for (int64_t d = 0; d < dh; ++d)
              acc = acc + q[d] * k[d];
            sc[j] = acc * scale;
          }
          float mx = -INFINITY;
          for (int64_t j = 0; j < S; ++j)
            mx = maxnum(mx, sc[j]);
          float sum = 0.0f;
          for (int64_t j = 0; j < S; ++j) {
            float e = expf(sc[j] - mx);
            sum = sum + e;
            sc[j] = e;
          }
          for (int64_t j = 0; j < S; ++j)
            sc[j] = sc[j] / sum;
          float *o = out + (b * S + i) * H + h * dh;
          for (int64_t d = 0; d < dh; ++d)
            o[d] = 0.0f;
          for (int64_t j = 0; j < S; ++j) {
            const float *v = V + (b * S + j) * H + h * dh;
            float p = sc[j];
            for (int64_t d = 0; d < dh; ++d)
              o[d] = o[d] + p * v[d];
          }
        }
      }
    }
    free(sc);
  }
}

void orc_dyn_quant_linear(const float *X, int64_t M, int64_t K,
    const int8_t *W, int64_t N, float w_scale, const float *bias, float *Y,
    uint8_t *xq, float *x_scale, uint8_t *x_zp, int32_t *acc) {
  uint8_t *q = xq ? xq : (uint8_t *)malloc((size_t)(M * K));
  int32_t *a = acc ? acc : (int32_t *)malloc((size_t)(M * N) * sizeof(int32_t));
  float s;
  uint8_t z;
  orc_dynamic_quantize_linear(X, M * K, q, &s, &z);
  orc_matmul_integer(q, 0, W, 1, M, N, K, &z, 1, NULL, 0, a);
  float s0 = s * w_scale; /* onnx.Mul of the two scalars, rounded once */
  orc_dequant_tail(a, M, N, s0, 0.0f, 0, bias, Y);
  if (x_scale)
    *x_scale = s;
  if (x_zp)
    *x_zp = z;
  if (!xq)
    free(q);
  if (!acc)
    free(a);
}

void orc_encoder_layer(const float *x, int64_t B, int64_t S, int64_t H,
    int64_t heads, int64_t F, const orc_encoder_layer_weights *w, float eps,
    float *y) {
  int64_t T = B * S;
  int64_t dh = H / heads;
  size_t th = (size_t)(T * H), tf = (size_t)(T * F);
  float *q = (float *)malloc(th * 4), *k = (float *)malloc(th * 4);
  float *v = (float *)malloc(th * 4), *ctx = (float *)malloc(th * 4);
  float *a = (float *)malloc(th * 4), *h1 = (float *)malloc(th * 4);
  float *f = (float *)malloc(tf * 4), *o = (float *)malloc(th * 4);
  orc_dyn_quant_linear(x, T, H, w->wq, H, w->sc[0], w->bq, q, 0, 0, 0, 0);
  orc_dyn_quant_linear(x, T, H, w->wk, H, w->sc[1], w->bk, k, 0, 0, 0, 0);
  orc_dyn_quant_linear(x, T, H, w->wv, H, w->sc[2], w->bv, v, 0, 0, 0, 0);
  float scale = 1.0f / sqrtf((float)dh);
  orc_attention(q, k, v, B, S, heads, dh, scale, ctx);
  orc_dyn_quant_linear(ctx, T, H, w->wo, H, w->sc[3], w->bo, a, 0, 0, 0, 0);
  orc_add(x, a, T * H, a);
  orc_layernorm(a, T, H, w->ln1g, w->ln1b, eps, h1);
  orc_dyn_quant_linear(h1, T, H, w->w1, F, w->sc[4], w->b1, f, 0, 0, 0, 0);
  orc_gelu(f, T * F, f);
  orc_dyn_quant_linear(f, T, F, w->w2, H, w->sc[5], w->b2, o, 0, 0, 0, 0);
  orc_add(h1, o, T * H, o);
  orc_layernorm(o, T, H, w->ln2g, w->ln2b, eps, y);
  free(q); free(k); free(v); free(ctx); free(a); free(h1); free(f); free(o);
}

/* ------------------------------------------------------------------------ */
/* Reference-shaped CPU baseline                                             */
/* ------------------------------------------------------------------------ */

void orc_ref_shaped_matmul_integer(const uint8_t *A, const int8_t *B, int64_t M,
    int64_t N, int64_t K, int32_t a_zp, int32_t *Y, int threads) {
  /* Four elementwise nests first (widen A, subtract, widen B; the b zero
   * point is absent in the config graphs), as the -O3 lit test shows
   * (test/mlir/conversion/onnx_to_krnl/Math/MatMulInteger_with_canonicalize_O3.mlir:33-105). */
  int32_t *A32 = (int32_t *)malloc((size_t)(M * K) * 4);
  int32_t *As = (int32_t *)malloc((size_t)(M * K) * 4);
  int32_t *B32 = (int32_t *)malloc((size_t)(K * N) * 4);
  if (threads < 1)
    threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads)
  for (int64_t i = 0; i < M * K; ++i)
    A32[i] = (int32_t)A[i];
#pragma omp parallel for schedule(static) num_threads(threads)
  for (int64_t i = 0; i < M * K; ++i)
    As[i] = A32[i] - a_zp;
#pragma omp parallel for schedule(static) num_threads(threads)
  for (int64_t i = 0; i < K * N; ++i)
    B32[i] = (int32_t)B[i];
  memset(Y, 0, (size_t)(M * N) * 4);
  /* i blocked by 4, j by 8 (the SIMD dimension), k by 8; loop order after the
   * permute is i-block, j-block, k-block (Math/MatMul.cpp:310-326). */
#pragma omp parallel for schedule(static) num_threads(threads)
  for (int64_t i0 = 0; i0 < M; i0 += 4) {
    int64_t ie = (i0 + 4 < M) ? i0 + 4 : M;
    for (int64_t j0 = 0; j0 < N; j0 += 8) {
      int64_t je = (j0 + 8 < N) ? j0 + 8 : N;
      for (int64_t k0 = 0; k0 < K; k0 += 8) {
        int64_t ke = (k0 + 8 < K) ? k0 + 8 : K;
        for (int64_t i = i0; i < ie; ++i) {
          uint32_t c[8];
          for (int64_t j = j0; j < je; ++j)
            c[j - j0] = (uint32_t)Y[i * N + j];
          for (int64_t k = k0; k < ke; ++k) {
            uint32_t a = (uint32_t)As[i * K + k];
            for (int64_t j = j0; j < je; ++j)
              c[j - j0] += a * (uint32_t)B32[k * N + j];
          }
          for (int64_t j = j0; j < je; ++j)
            Y[i * N + j] = (int32_t)c[j - j0];
        }
      }
    }
  }
  free(A32);
  free(As);
  free(B32);
}

void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0)
    omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

int64_t orc_selftest_round_even_exhaustive(void) {
  int64_t bad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
  for (int64_t bits = 0; bits < (1ll << 32); ++bits) {
    uint32_t u = (uint32_t)bits;
    float x;
    memcpy(&x, &u, 4);
    if (!isfinite(x))
      continue;
    float a = orc_round_even(x);
    float b = rintf(x); /* default rounding mode: to nearest even */
    if (a != b) /* +0 == -0 compares equal */
      ++bad;
  }
  return bad;
}
