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

// Order-preserving float <-> uint mapping so running min/max can use integer
// atomics.  NaNs never reach these (callers filter with fminf/fmaxf).
__device__ __forceinline__ uint32_t f32_to_ordered(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_f32(uint32_t u) {
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

#endif // __CUDACC__

} // namespace omcuda
