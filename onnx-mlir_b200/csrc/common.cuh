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
// with erf evaluated without a branch as
//   erf(t) = 1 - 2^(t * Q(t)),  t = min(|x| / sqrt(2), 4),  sign restored,
// Q a degree-7 polynomial fitted (weighted least squares on [0, 4], weights
// following the sensitivity of erf to Q) to log2(erfc(t)) / t.  Absolute
// error of erf below 2e-7 (polynomial 8.5e-8 plus the 2^x approximation), of
// Gelu below 4e-7 on [-8, 8]; beyond t = 4 erf is 1 in fp32.  About 15
// instructions against the 35-40 of the library erff with both of its
// branches taken in a warp, which matters in the GEMM epilogue.  Every Gelu
// of the library (fused tail and standalone op) goes through this function.
__device__ __forceinline__ float gelu_erf(float x) {
  const float t = fminf(fabsf(__fmul_rn(x, 0.70710678118654752440f)), 4.0f);
  float q = -4.5358585339272395e-05f;
  q = __fmaf_rn(q, t, 0.00044550743768922985f);
  q = __fmaf_rn(q, t, -0.0014894406776875257f);
  q = __fmaf_rn(q, t, -0.0007746315677650273f);
  q = __fmaf_rn(q, t, 0.02825368382036686f);
  q = __fmaf_rn(q, t, -0.14848162233829498f);
  q = __fmaf_rn(q, t, -0.9184163808822632f);
  q = __fmaf_rn(q, t, -1.6279085874557495f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(q, t)));
  const float r = copysignf(__fsub_rn(1.0f, e), x);
  return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, r));
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
  const uint64_t x = pack_f32x2(x0, x1);
  float t0, t1;
  unpack_f32x2(mul_f32x2(x, pack_f32x2(0.70710678118654752440f, 0.70710678118654752440f)),
      t0, t1);
  const uint64_t t = pack_f32x2(fminf(fabsf(t0), 4.0f), fminf(fabsf(t1), 4.0f));
#define OMCUDA_C2(c) pack_f32x2(c, c)
  uint64_t q = OMCUDA_C2(-4.5358585339272395e-05f);
  q = fma_f32x2(q, t, OMCUDA_C2(0.00044550743768922985f));
  q = fma_f32x2(q, t, OMCUDA_C2(-0.0014894406776875257f));
  q = fma_f32x2(q, t, OMCUDA_C2(-0.0007746315677650273f));
  q = fma_f32x2(q, t, OMCUDA_C2(0.02825368382036686f));
  q = fma_f32x2(q, t, OMCUDA_C2(-0.14848162233829498f));
  q = fma_f32x2(q, t, OMCUDA_C2(-0.9184163808822632f));
  q = fma_f32x2(q, t, OMCUDA_C2(-1.6279085874557495f));
  float a0, a1;
  unpack_f32x2(mul_f32x2(q, t), a0, a1);
  float e0, e1;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(a0));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(a1));
  // 1 - e, sign of x restored, then 0.5 x (1 + r)
  const float r0 = copysignf(__fsub_rn(1.0f, e0), x0);
  const float r1 = copysignf(__fsub_rn(1.0f, e1), x1);
  const uint64_t h = mul_f32x2(OMCUDA_C2(0.5f), x);
  const uint64_t s = add_f32x2(OMCUDA_C2(1.0f), pack_f32x2(r0, r1));
#undef OMCUDA_C2
  unpack_f32x2(mul_f32x2(h, s), x0, x1);
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
