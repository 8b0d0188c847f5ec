// Shared host/device helpers for libomcuda (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "omcuda.h"

namespace omcuda {

// ---- host side -------------------------------------------------------------

// Records a failure in the calling thread's sticky status (and errno) and
// returns the code, so call sites can `return fail(...)`.
int fail(int code, const char *fmt, ...);
int check_cuda(cudaError_t e, const char *what);
void count_launch(int n = 1);
int sm_count();

#define OMCUDA_CHECK(expr)                                                     \
  do {                                                                         \
    int _st = ::omcuda::check_cuda((expr), #expr);                             \
    if (_st != OMCUDA_OK)                                                      \
      return _st;                                                              \
  } while (0)

#define OMCUDA_CHECK_LAUNCH(name)                                              \
  do {                                                                         \
    ::omcuda::count_launch();                                                  \
    int _st = ::omcuda::check_cuda(cudaGetLastError(), name);                  \
    if (_st != OMCUDA_OK)                                                      \
      return _st;                                                              \
  } while (0)

#ifdef __CUDACC__
__host__ __device__
#endif
static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device side -----------------------------------------------------------

#ifdef __CUDACC__

// Round half to even, the result of onnx-mlir's floor-based emulation
// (src/Dialect/Mlir/DialectBuilder.cpp:291-335).  That sequence equals
// IEEE roundToIntegralTiesToEven for every finite float except that it yields
// +0 where rint yields -0; every caller adds a non-negative-zero value or
// converts to an integer next, which erases the difference.
__device__ __forceinline__ float round_even(float x) { return rintf(x); }

// The emulation itself, op for op, for tests that compare the two on device.
__device__ __forceinline__ float round_even_emulated(float x) {
  float y = floorf(x);
  float r = __fsub_rn(x, y);
  float y1 = (r > 0.5f) ? __fadd_rn(y, 1.0f) : y;
  float y2 = __fmul_rn(floorf(__fmul_rn(0.5f, y)), 2.0f);
  float rr = __fsub_rn(y, y2);
  float yt = (rr == 1.0f) ? __fadd_rn(y, 1.0f) : y;
  return (r == 0.5f) ? yt : y1;
}

// MathBuilder::clip (DialectBuilder.cpp:355-360) with arith.maxnumf/minnumf;
// fmaxf/fminf return the non-NaN operand like maxnum/minnum.
__device__ __forceinline__ float clipf(float v, float lo, float hi) {
  return fminf(fmaxf(v, lo), hi);
}

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Gelu with the exact (erf) formula of the reference,
// 0.5 * x * (1 + erf(x / sqrt(2))) (src/Conversion/ONNXToKrnl/Math/Elementwise.cpp:358-388),
// evaluated without a branch and without the cancellation of 1 + erf for
// negative x.  With t = min(|x| / sqrt(2), 4) and E(t) = 2^(t * Q(t)) an
// approximation of erfc(t) (Q a degree-8 polynomial fitted to
// log2(erfc(t)) / t on [0, 4] so that the error of the exponent t * Q(t), i.e.
// the relative error of E, is uniform: 8e-7),
//   x >= 0:  0.5 x (1 + erf)  = x - (t / sqrt(2)) E(t)
//   x <  0:  0.5 x erfc(|x|/sqrt(2)) = - (t / sqrt(2)) E(t)
// both of which are  max(x, 0) - (t / sqrt(2)) E(t)  (one fused multiply-add).
// Relative error against the exactly rounded formula: below 4e-6 everywhere
// the reference's own result is meaningful.  For x < 0 the reference rounds
// erff to fp32 before adding 1, which quantizes its result to multiples of
// 0.5 |x| 2^-24; this function does not reproduce that rounding step, so the
// two differ by up to half such a step there (and the reference's result is
// exactly -0 below x = -5.6, where this one is about -4e-8).  NaN gives NaN,
// +inf gives +inf; -inf gives -4e-8 where the reference's 0 * inf gives NaN.
// About 14 instructions against the 35-40 of the library erff with both of
// its branches taken in a warp, which matters in the GEMM epilogue.  Every
// Gelu of the library (fused tail and standalone op) goes through this
// function or its two-lane form below.
#define OMCUDA_GELU_Q0 -1.627946138381958f
#define OMCUDA_GELU_Q1 -0.9180199503898621f
#define OMCUDA_GELU_Q2 -0.14988861978054047f
#define OMCUDA_GELU_Q3 0.030609266832470894f
#define OMCUDA_GELU_Q4 -0.002864620415493846f
#define OMCUDA_GELU_Q5 -0.0004925866960547864f
#define OMCUDA_GELU_Q6 0.00021463484154082835f
#define OMCUDA_GELU_Q7 -3.0283568776212633e-05f
#define OMCUDA_GELU_Q8 1.6220828911173157e-06f

// max(x, 0) that keeps a NaN (fmaxf would drop it).
__device__ __forceinline__ float relu_keep_nan(float x) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(x), "f"(0.0f));
  return r;
}

__device__ __forceinline__ float gelu_erf(float x) {
  const float c = 0.70710678118654752440f;
  const float t = fminf(fabsf(__fmul_rn(x, c)), 4.0f);
  float q = OMCUDA_GELU_Q8;
  q = __fmaf_rn(q, t, OMCUDA_GELU_Q7);
  q = __fmaf_rn(q, t, OMCUDA_GELU_Q6);
  q = __fmaf_rn(q, t, OMCUDA_GELU_Q5);
  q = __fmaf_rn(q, t, OMCUDA_GELU_Q4);
  q = __fmaf_rn(q, t, OMCUDA_GELU_Q3);
  q = __fmaf_rn(q, t, OMCUDA_GELU_Q2);
  q = __fmaf_rn(q, t, OMCUDA_GELU_Q1);
  q = __fmaf_rn(q, t, OMCUDA_GELU_Q0);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(q, t)));
  return __fmaf_rn(__fmul_rn(t, -c), e, relu_keep_nan(x));
}

// Three-input fp32 min / max of sm_100 (same result as two fminf / fmaxf:
// NaN operands are dropped).
__device__ __forceinline__ float min3f(float a, float b, float c) {
  float r;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Two Gelus at once on the packed-fp32 instructions of sm_100
// (mul / add / fma .f32x2: two independent, individually rounded fp32
// operations per instruction, so each lane gets exactly the bits gelu_erf
// gives it).  Halves the FMA-pipe instructions of the polynomial, which
// matters where the GEMM tail is bound by instruction issue.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ void gelu_erf_x2(float &x0, float &x1) {
#define OMCUDA_C2(c) pack_f32x2(c, c)
  const float c = 0.70710678118654752440f;
  float t0, t1;
  unpack_f32x2(mul_f32x2(pack_f32x2(x0, x1), OMCUDA_C2(c)), t0, t1);
  const uint64_t t = pack_f32x2(fminf(fabsf(t0), 4.0f), fminf(fabsf(t1), 4.0f));
  uint64_t q = OMCUDA_C2(OMCUDA_GELU_Q8);
  q = fma_f32x2(q, t, OMCUDA_C2(OMCUDA_GELU_Q7));
  q = fma_f32x2(q, t, OMCUDA_C2(OMCUDA_GELU_Q6));
  q = fma_f32x2(q, t, OMCUDA_C2(OMCUDA_GELU_Q5));
  q = fma_f32x2(q, t, OMCUDA_C2(OMCUDA_GELU_Q4));
  q = fma_f32x2(q, t, OMCUDA_C2(OMCUDA_GELU_Q3));
  q = fma_f32x2(q, t, OMCUDA_C2(OMCUDA_GELU_Q2));
  q = fma_f32x2(q, t, OMCUDA_C2(OMCUDA_GELU_Q1));
  q = fma_f32x2(q, t, OMCUDA_C2(OMCUDA_GELU_Q0));
  float a0, a1;
  unpack_f32x2(mul_f32x2(q, t), a0, a1);
  float e0, e1;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(a0));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(a1));
  // max(x, 0) - (t / sqrt(2)) e
  const uint64_t na = mul_f32x2(t, OMCUDA_C2(-c));
  const uint64_t m = pack_f32x2(relu_keep_nan(x0), relu_keep_nan(x1));
#undef OMCUDA_C2
  unpack_f32x2(fma_f32x2(na, pack_f32x2(e0, e1), m), x0, x1);
}

// Order-preserving float <-> uint mapping so running min/max can use integer
// atomics.  NaNs never reach these (callers filter with fminf/fmaxf).
__device__ __forceinline__ uint32_t f32_to_ordered(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_f32(uint32_t u) {
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// Folds a warp's {min,max} into a running range (two ordered uints).  The
// range only ever widens, so a plain (possibly stale) read that already covers
// the warp's values makes the atomic unnecessary; after the first few warps of
// a launch almost none is issued, which matters because they all target one
// address.  lo > hi (nothing but NaNs seen) commits nothing.
__device__ __forceinline__ void range_commit_warp(
    uint32_t *range, float lo, float hi) {
  lo = warp_min(lo);
  hi = warp_max(hi);
  if ((threadIdx.x & 31) == 0 && lo <= hi) {
    const uint32_t ol = f32_to_ordered(lo), oh = f32_to_ordered(hi);
    volatile uint32_t *vr = range;
    if (ol < vr[0])
      atomicMin(range, ol);
    if (oh > vr[1])
      atomicMax(range + 1, oh);
  }
}

#endif // __CUDACC__

} // namespace omcuda
