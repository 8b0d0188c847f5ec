// Scalar arithmetic of DynamicQuantizeLinear / QuantizeLinear shared by the
// quantize kernels and by the GEMM tail that quantizes its own output.
//
// Semantics follow onnx-mlir's lowering:
//   params    src/Conversion/ONNXToKrnl/Quantization/DynamicQuantizeLinear.cpp:43-84
//   quantize  src/Conversion/ONNXToKrnl/Quantization/QuantizeLinear.cpp:122-145
#pragma once

#include "../common.cuh"

namespace omcuda {

// fp32 arithmetic below uses the _rn intrinsics so that nothing is contracted
// into an fma: the reference emits separate arith ops.
// mode: OMCUDA_MODE_* flags (omcuda.h), the reference's compile-time options
// --disable-quantization-zero-point (zero point 0,
// DynamicQuantizeLinear.cpp:72-83) and enable-fast-math (x * (1 / scale)
// instead of x / scale, QuantizeLinear.cpp:43-44,117-131).
__device__ __forceinline__ void dql_params_from_range(
    float mn, float mx, float *scale, float *zp_f, int mode = 0) {
  float xmax = fmaxf(mx, 0.0f);
  float xmin = fminf(mn, 0.0f);
  float s = __fdiv_rn(__fsub_rn(xmax, xmin), 255.0f);
  float inter = __fsub_rn(0.0f, __fdiv_rn(xmin, s));
  float z = round_even(clipf(inter, 0.0f, 255.0f));
  *scale = s;
  *zp_f = (mode & OMCUDA_MODE_NO_ZERO_POINT) ? 0.0f : z;
}

// One element exactly as the reference computes it
// (QuantizeLinear.cpp:124-145): IEEE divide, round half even, add the zero
// point, clip, convert.
template <bool kSigned>
__device__ __forceinline__ uint32_t quantize_one_exact(
    float x, float scale, float zp_f, bool use_rcp = false) {
  float q = use_rcp ? __fmul_rn(x, __fdiv_rn(1.0f, scale)) : __fdiv_rn(x, scale);
  float r = round_even(q);
  float a = __fadd_rn(r, zp_f);
  if (kSigned) {
    float s = clipf(a, -128.0f, 127.0f);
    return (uint32_t)(int32_t)s & 0xffu; // fptosi, then trunc to 8 bits
  }
  float s = clipf(a, 0.0f, 255.0f);
  return (uint32_t)s; // fptoui; already within 8 bits
}

// Per-launch constants of the fast path.
struct QuantConsts {
  float scale, rcp, zp_f;
  bool fast;
  bool use_rcp; // fast-math mode: the reference multiplies by RN(1 / scale)
};

__device__ __forceinline__ QuantConsts make_quant_consts(
    float scale, float zp_f, int mode = 0) {
  QuantConsts c;
  c.scale = scale;
  c.zp_f = (mode & OMCUDA_MODE_NO_ZERO_POINT) ? 0.0f : zp_f;
  c.use_rcp = (mode & OMCUDA_MODE_FAST_MATH) != 0;
  c.rcp = __fdiv_rn(1.0f, scale);
  // The shortcut needs a normal, finite reciprocal; anything else (scale 0
  // from an all-zero tensor, denormal or huge scales) takes the exact path.
  const float as = fabsf(scale);
  c.fast = (as > 1e-30f) && (as < 1e30f);
  return c;
}

// Same result as quantize_one_exact with no divide or convert instruction on
// the common path (those run on the quarter-rate special-function pipe and
// would bound the kernel instead of HBM):
//  * t = fma(x, RN(1/scale), 1.5 * 2^23) rounds the product half-even to an
//    integer held in the mantissa (exact while |product| < 2^22); r = t - 1.5 *
//    2^23 is that integer and d = fma(x, RN(1/scale), -r) the exact distance
//    of the product from it.
//  * x * RN(1/scale) is within 2.5 ulp of the IEEE quotient q = x / scale.
//    Where |q| <= 512 that is below 2e-4, so unless |d| > 0.499 (the product
//    lies within 1e-3 of a tie) q rounds to the same integer r; the rare
//    near-tie element is redone with the exact divide.  Where |q| > 512 the
//    result saturates whatever the rounding (zero point and bounds lie in
//    [-128, 255]), and |d| <= 0.499 still holds or the exact path runs.
//  * the zero point is added and the clip applied while the value still
//    carries the 1.5 * 2^23 offset (integers below 2^24, or large values that
//    the clip cuts off either way), and the result is the low byte of the
//    mantissa (two's complement for the signed type).
// In fast-math mode the reference's quotient is RN(x * RN(1/scale)), the
// rounded value of the very product the fma holds exactly: away from a tie it
// rounds to the same integer, near one the redo uses that product.
// +-inf saturate through the clip; a NaN product fails the |d| test, passes
// through fmaxf as the lower clip bound, which is where maxnum/minnum send a
// NaN in the reference as well.
template <bool kSigned>
__device__ __forceinline__ uint32_t quantize_one(float x, const QuantConsts &c) {
  if (!c.fast)
    return quantize_one_exact<kSigned>(x, c.scale, c.zp_f, c.use_rcp);
  const float kMagic = 12582912.0f; // 1.5 * 2^23
  float t = __fmaf_rn(x, c.rcp, kMagic);
  const float r = __fsub_rn(t, kMagic);
  const float d = __fmaf_rn(x, c.rcp, -r);
  if (fabsf(d) > 0.499f) // near a tie, or too large for the mantissa trick
    t = __fadd_rn(round_even(c.use_rcp ? __fmul_rn(x, c.rcp) : __fdiv_rn(x, c.scale)),
        kMagic);
  const float u = __fadd_rn(t, c.zp_f);
  const float s = kSigned ? clipf(u, kMagic - 128.0f, kMagic + 127.0f)
                          : clipf(u, kMagic, kMagic + 255.0f);
  return __float_as_uint(s) & 0xffu;
}

// Four elements by the exact formula, out of line: the fast path below calls
// it for the rare float4 that holds a near-tie element, and must not carry the
// divide's instructions as predicated code.
template <bool kSigned>
__device__ __noinline__ uint32_t quantize_four_exact(
    float4 v, float scale, float zp_f, bool use_rcp) {
  return quantize_one_exact<kSigned>(v.x, scale, zp_f, use_rcp) |
         (quantize_one_exact<kSigned>(v.y, scale, zp_f, use_rcp) << 8) |
         (quantize_one_exact<kSigned>(v.z, scale, zp_f, use_rcp) << 16) |
         (quantize_one_exact<kSigned>(v.w, scale, zp_f, use_rcp) << 24);
}

// quantize_one on the four elements of a float4 with one near-tie test for
// all of them.
template <bool kSigned>
__device__ __forceinline__ uint32_t quantize_four(float4 v, const QuantConsts &c) {
  if (!c.fast)
    return quantize_four_exact<kSigned>(v, c.scale, c.zp_f, c.use_rcp);
  const float kMagic = 12582912.0f; // 1.5 * 2^23
  const float t0 = __fmaf_rn(v.x, c.rcp, kMagic), t1 = __fmaf_rn(v.y, c.rcp, kMagic);
  const float t2 = __fmaf_rn(v.z, c.rcp, kMagic), t3 = __fmaf_rn(v.w, c.rcp, kMagic);
  const float d0 = __fmaf_rn(v.x, c.rcp, -__fsub_rn(t0, kMagic));
  const float d1 = __fmaf_rn(v.y, c.rcp, -__fsub_rn(t1, kMagic));
  const float d2 = __fmaf_rn(v.z, c.rcp, -__fsub_rn(t2, kMagic));
  const float d3 = __fmaf_rn(v.w, c.rcp, -__fsub_rn(t3, kMagic));
  // NaN distances (infinite or NaN inputs) fall through fmaxf and take the
  // fast path, which saturates them as the exact formula does.
  const float dmax = fmaxf(fmaxf(fabsf(d0), fabsf(d1)), fmaxf(fabsf(d2), fabsf(d3)));
  if (dmax > 0.499f) // a near tie, or a value too large for the mantissa trick
    return quantize_four_exact<kSigned>(v, c.scale, c.zp_f, c.use_rcp);
  const float lo = kSigned ? kMagic - 128.0f : kMagic;
  const float hi = kSigned ? kMagic + 127.0f : kMagic + 255.0f;
  const uint32_t b0 = __float_as_uint(clipf(__fadd_rn(t0, c.zp_f), lo, hi)) & 0xffu;
  const uint32_t b1 = __float_as_uint(clipf(__fadd_rn(t1, c.zp_f), lo, hi)) & 0xffu;
  const uint32_t b2 = __float_as_uint(clipf(__fadd_rn(t2, c.zp_f), lo, hi)) & 0xffu;
  const uint32_t b3 = __float_as_uint(clipf(__fadd_rn(t3, c.zp_f), lo, hi));
  return b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
}

} // namespace omcuda
