// DynamicQuantizeLinear / QuantizeLinear / DequantizeLinear kernels.
//
// Semantics follow onnx-mlir's lowering:
//   min/max   src/Conversion/ONNXToKrnl/Math/Reduction.cpp:394-548 (minnum/maxnum,
//             identities +inf/-inf)
//   params    src/Conversion/ONNXToKrnl/Quantization/DynamicQuantizeLinear.cpp:43-84
//   quantize  src/Conversion/ONNXToKrnl/Quantization/QuantizeLinear.cpp:122-145
//   dequant   src/Conversion/ONNXToKrnl/Math/Elementwise.cpp:1438-1461
//
// Layout: tensors are flat, dense, row-major.  The reduction runs as a
// single-pass grid reduction: every block leaves its partial min/max in
// scratch, takes a ticket, and the block that draws the last ticket folds the
// partials and derives scale and zero point, so no block ever waits on
// another.  The quantize pass is a second launch that reads the two scalars
// from device memory; for tensors that fit in L2 its read of x is served from
// there.
#include "../common.cuh"

namespace omcuda {

static constexpr int kDqlThreads = 256;
static constexpr int kDqlMaxBlocks = 2048;
static constexpr int kQuantUnroll = 8;

struct DqlScratch {
  unsigned int ticket;
  unsigned int pad[15];
  float part_min[kDqlMaxBlocks];
  float part_max[kDqlMaxBlocks];
  float params[4]; // scale, zero point as float
};

// fp32 arithmetic below uses the _rn intrinsics so that nothing is contracted
// into an fma: the reference emits separate arith ops.
__device__ __forceinline__ void dql_params_from_range(
    float mn, float mx, float *scale, float *zp_f) {
  float xmax = fmaxf(mx, 0.0f);
  float xmin = fminf(mn, 0.0f);
  float s = __fdiv_rn(__fsub_rn(xmax, xmin), 255.0f);
  float inter = __fsub_rn(0.0f, __fdiv_rn(xmin, s));
  float z = round_even(clipf(inter, 0.0f, 255.0f));
  *scale = s;
  *zp_f = z;
}

__global__ void __launch_bounds__(kDqlThreads)
    dql_minmax_kernel(const float *__restrict__ x, int64_t n,
        DqlScratch *__restrict__ scr, float *__restrict__ y_scale,
        uint8_t *__restrict__ y_zp) {
  float lo = INFINITY, hi = -INFINITY;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const bool aligned = ((uintptr_t)x & 15u) == 0;
  if (aligned) {
    const int64_t n4 = n >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    // Eight independent 16-byte loads in flight per thread per trip: with all
    // 2048 threads of an SM resident that is 256 KiB outstanding per SM, well
    // above what HBM latency times bandwidth asks for.
    int64_t i = tid;
    for (; i + 7 * nthreads < n4; i += 8 * nthreads) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = __ldcs(x4 + i + u * nthreads);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        lo = fminf(lo, fminf(fminf(v[u].x, v[u].y), fminf(v[u].z, v[u].w)));
        hi = fmaxf(hi, fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w)));
      }
    }
    for (; i < n4; i += nthreads) {
      float4 a = __ldcs(x4 + i);
      lo = fminf(lo, fminf(fminf(a.x, a.y), fminf(a.z, a.w)));
      hi = fmaxf(hi, fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)));
    }
    for (int64_t j = (n4 << 2) + tid; j < n; j += nthreads) {
      float v = x[j];
      lo = fminf(lo, v);
      hi = fmaxf(hi, v);
    }
  } else {
    for (int64_t j = tid; j < n; j += nthreads) {
      float v = x[j];
      lo = fminf(lo, v);
      hi = fmaxf(hi, v);
    }
  }
  lo = warp_min(lo);
  hi = warp_max(hi);
  __shared__ float s_lo[kDqlThreads / 32], s_hi[kDqlThreads / 32];
  __shared__ bool s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_lo[warp] = lo;
    s_hi[warp] = hi;
  }
  __syncthreads();
  if (warp == 0) {
    lo = lane < kDqlThreads / 32 ? s_lo[lane] : INFINITY;
    hi = lane < kDqlThreads / 32 ? s_hi[lane] : -INFINITY;
    lo = warp_min(lo);
    hi = warp_max(hi);
    if (lane == 0) {
      scr->part_min[blockIdx.x] = lo;
      scr->part_max[blockIdx.x] = hi;
      __threadfence();
      unsigned int t = atomicAdd(&scr->ticket, 1u);
      s_last = (t == gridDim.x - 1);
    }
  }
  __syncthreads();
  if (!s_last)
    return;
  // Last block: fold the partials (order does not matter for min/max).
  __threadfence();
  lo = INFINITY;
  hi = -INFINITY;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
    lo = fminf(lo, __ldcg(&scr->part_min[i]));
    hi = fmaxf(hi, __ldcg(&scr->part_max[i]));
  }
  lo = warp_min(lo);
  hi = warp_max(hi);
  __syncthreads();
  if (lane == 0) {
    s_lo[warp] = lo;
    s_hi[warp] = hi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kDqlThreads / 32; ++w) {
      lo = fminf(lo, s_lo[w]);
      hi = fmaxf(hi, s_hi[w]);
    }
    float s, z;
    dql_params_from_range(lo, hi, &s, &z);
    scr->params[0] = s;
    scr->params[1] = z;
    if (y_scale)
      *y_scale = s;
    if (y_zp)
      *y_zp = (uint8_t)(unsigned int)z; // fptoui then trunc; z is in [0,255]
    scr->ticket = 0; // leave the scratch ready for the next call
  }
}

// One element exactly as the reference computes it
// (QuantizeLinear.cpp:124-145): IEEE divide, round half even, add the zero
// point, clip, convert.
template <bool kSigned>
__device__ __forceinline__ uint32_t quantize_one_exact(
    float x, float scale, float zp_f) {
  float q = __fdiv_rn(x, scale);
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
};

__device__ __forceinline__ QuantConsts make_quant_consts(float scale, float zp_f) {
  QuantConsts c;
  c.scale = scale;
  c.zp_f = zp_f;
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
// +-inf saturate through the clip; a NaN product fails the |d| test, passes
// through fmaxf as the lower clip bound, which is where maxnum/minnum send a
// NaN in the reference as well.
template <bool kSigned>
__device__ __forceinline__ uint32_t quantize_one(float x, const QuantConsts &c) {
  if (!c.fast)
    return quantize_one_exact<kSigned>(x, c.scale, c.zp_f);
  const float kMagic = 12582912.0f; // 1.5 * 2^23
  float t = __fmaf_rn(x, c.rcp, kMagic);
  const float r = __fsub_rn(t, kMagic);
  const float d = __fmaf_rn(x, c.rcp, -r);
  if (fabsf(d) > 0.499f) // near a tie, or too large for the mantissa trick
    t = __fadd_rn(round_even(__fdiv_rn(x, c.scale)), kMagic);
  const float u = __fadd_rn(t, c.zp_f);
  const float s = kSigned ? clipf(u, kMagic - 128.0f, kMagic + 127.0f)
                          : clipf(u, kMagic, kMagic + 255.0f);
  return __float_as_uint(s) & 0xffu;
}

// Four elements by the exact formula, out of line: the fast path below calls
// it for the rare float4 that holds a near-tie element, and must not carry the
// divide's instructions as predicated code.
template <bool kSigned>
__device__ __noinline__ uint32_t quantize_four_exact(float4 v, float scale, float zp_f) {
  return quantize_one_exact<kSigned>(v.x, scale, zp_f) |
         (quantize_one_exact<kSigned>(v.y, scale, zp_f) << 8) |
         (quantize_one_exact<kSigned>(v.z, scale, zp_f) << 16) |
         (quantize_one_exact<kSigned>(v.w, scale, zp_f) << 24);
}

// quantize_one on the four elements of a float4 with one near-tie test for
// all of them.
template <bool kSigned>
__device__ __forceinline__ uint32_t quantize_four(float4 v, const QuantConsts &c) {
  if (!c.fast)
    return quantize_four_exact<kSigned>(v, c.scale, c.zp_f);
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
    return quantize_four_exact<kSigned>(v, c.scale, c.zp_f);
  const float lo = kSigned ? kMagic - 128.0f : kMagic;
  const float hi = kSigned ? kMagic + 127.0f : kMagic + 255.0f;
  const uint32_t b0 = __float_as_uint(clipf(__fadd_rn(t0, c.zp_f), lo, hi)) & 0xffu;
  const uint32_t b1 = __float_as_uint(clipf(__fadd_rn(t1, c.zp_f), lo, hi)) & 0xffu;
  const uint32_t b2 = __float_as_uint(clipf(__fadd_rn(t2, c.zp_f), lo, hi)) & 0xffu;
  const uint32_t b3 = __float_as_uint(clipf(__fadd_rn(t3, c.zp_f), lo, hi));
  return b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
}

// Where the range-driven form of the kernel leaves its scalars.
struct QuantOutputs {
  float *params;  // {scale, zero point as float}
  float *y_scale; // the op's y_scale output, may be null
  uint8_t *y_zp;  // the op's y_zero_point output, may be null
};

// params: {scale, zp as float}.  If zp8 is non-NULL the zero point is read
// from it instead (QuantizeLinear with a given 8-bit zero point).  If range is
// non-NULL, scale and zero point are derived from that running {min,max}
// (ordered-uint encoding, see f32_to_ordered) as DynamicQuantizeLinear does.
template <bool kSigned>
__global__ void __launch_bounds__(kDqlThreads)
    quantize_kernel(const float *__restrict__ x, int64_t n,
        uint8_t *__restrict__ y, const float *__restrict__ params,
        const float *__restrict__ scale_ptr, const void *__restrict__ zp8,
        int has_zp, const uint32_t *__restrict__ range, QuantOutputs outs) {
  float scale, zp_f;
  if (range) {
    // Scale and zero point straight from a producer's running range (every
    // thread derives the same two scalars; block 0 also publishes them for
    // the ops that follow).
    dql_params_from_range(ordered_to_f32(__ldg(range)), ordered_to_f32(__ldg(range + 1)),
        &scale, &zp_f);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      outs.params[0] = scale;
      outs.params[1] = zp_f;
      if (outs.y_scale)
        *outs.y_scale = scale;
      if (outs.y_zp)
        *outs.y_zp = (uint8_t)(unsigned int)zp_f; // fptoui; zp_f is in [0,255]
    }
  } else if (params) {
    scale = __ldg(params);
    zp_f = __ldg(params + 1);
  } else {
    scale = __ldg(scale_ptr);
    if (!has_zp)
      zp_f = 0.0f;
    else if (kSigned)
      zp_f = (float)*reinterpret_cast<const int8_t *>(zp8);
    else
      zp_f = (float)*reinterpret_cast<const uint8_t *>(zp8);
  }
  const QuantConsts qc = make_quant_consts(scale, zp_f);
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  const bool aligned = (((uintptr_t)x & 15u) == 0) && (((uintptr_t)y & 3u) == 0);
  if (aligned) {
    const int64_t n4 = n >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    uint32_t *y4 = reinterpret_cast<uint32_t *>(y);
    int64_t i = tid;
    // kQuantUnroll float4 loads in flight per thread; each is a fully
    // coalesced 512-byte warp access, each store a 128-byte one.
    for (; i + (kQuantUnroll - 1) * nthreads < n4; i += kQuantUnroll * nthreads) {
      float4 v[kQuantUnroll];
#pragma unroll
      for (int u = 0; u < kQuantUnroll; ++u)
        v[u] = __ldcs(x4 + i + u * nthreads);
#pragma unroll
      for (int u = 0; u < kQuantUnroll; ++u)
        __stcs(y4 + i + u * nthreads, quantize_four<kSigned>(v[u], qc));
    }
    for (; i < n4; i += nthreads)
      y4[i] = quantize_four<kSigned>(__ldcs(x4 + i), qc);
    for (int64_t j = (n4 << 2) + tid; j < n; j += nthreads)
      y[j] = (uint8_t)quantize_one<kSigned>(x[j], qc);
  } else {
    for (int64_t j = tid; j < n; j += nthreads)
      y[j] = (uint8_t)quantize_one<kSigned>(x[j], qc);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
    dequantize_kernel(const T *__restrict__ x, int64_t n,
        const float *__restrict__ scale, const T *__restrict__ zp,
        float *__restrict__ y) {
  const float s = __ldg(scale);
  const float zf = zp ? (float)*zp : 0.0f;
  const bool has_zp = zp != nullptr;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float xf = (float)x[i];
    float d = has_zp ? __fsub_rn(xf, zf) : xf;
    y[i] = __fmul_rn(d, s);
  }
}

static int grid_for(int64_t work_items, int per_block) {
  int64_t want = ceil_div(work_items, per_block);
  int64_t cap = (int64_t)sm_count() * 8;
  if (cap > kDqlMaxBlocks)
    cap = kDqlMaxBlocks;
  if (want < 1)
    want = 1;
  return (int)(want < cap ? want : cap);
}

int launch_quantize_with_params(const float *x, int64_t n, uint8_t *y,
    const float *params, cudaStream_t st) {
  int grid = grid_for(n, kDqlThreads * 16);
  quantize_kernel<false><<<grid, kDqlThreads, 0, st>>>(
      x, n, y, params, nullptr, nullptr, 1, nullptr, QuantOutputs{});
  OMCUDA_CHECK_LAUNCH("quantize_kernel");
  return OMCUDA_OK;
}

} // namespace omcuda

using namespace omcuda;

extern "C" int64_t omcudaDevDqlScratchBytes(int64_t) {
  return (int64_t)sizeof(DqlScratch);
}

extern "C" int omcudaDevDynamicQuantizeLinear(const float *x, int64_t n,
    uint8_t *y, float *y_scale, uint8_t *y_zp, void *scratch, void *stream) {
  if (n < 0 || (n > 0 && (!x || !y)) || !scratch)
    return fail(OMCUDA_EINVAL, "DynamicQuantizeLinear: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  DqlScratch *scr = (DqlScratch *)scratch;
  int grid = grid_for(n, kDqlThreads * 16);
  dql_minmax_kernel<<<grid, kDqlThreads, 0, st>>>(x, n, scr, y_scale, y_zp);
  OMCUDA_CHECK_LAUNCH("dql_minmax_kernel");
  if (n > 0)
    return launch_quantize_with_params(x, n, y, scr->params, st);
  return OMCUDA_OK;
}

extern "C" int omcudaDevQuantizeFromRange(const float *x, int64_t n, void *range,
    uint8_t *y, float *params, float *y_scale, uint8_t *y_zp, void *stream) {
  if (n < 0 || (n > 0 && (!x || !y)) || !range || !params)
    return fail(OMCUDA_EINVAL, "QuantizeFromRange: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  // One launch: every block derives the scalars from the range itself (a
  // block of its own when there is nothing to quantize).
  int grid = grid_for(n, kDqlThreads * 16);
  QuantOutputs outs{params, y_scale, y_zp};
  quantize_kernel<false><<<grid, kDqlThreads, 0, st>>>(
      x, n, y, nullptr, nullptr, nullptr, 1, (const uint32_t *)range, outs);
  OMCUDA_CHECK_LAUNCH("quantize_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevQuantizeLinear(const float *x, int64_t n, void *y,
    int y_signed, const float *scale, const void *zp, void *stream) {
  if (n < 0 || (n > 0 && (!x || !y)) || !scale)
    return fail(OMCUDA_EINVAL, "QuantizeLinear: bad argument");
  if (n == 0)
    return OMCUDA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  int grid = grid_for(n, kDqlThreads * 16);
  if (y_signed)
    quantize_kernel<true><<<grid, kDqlThreads, 0, st>>>(
        x, n, (uint8_t *)y, nullptr, scale, zp, zp != nullptr, nullptr, QuantOutputs{});
  else
    quantize_kernel<false><<<grid, kDqlThreads, 0, st>>>(
        x, n, (uint8_t *)y, nullptr, scale, zp, zp != nullptr, nullptr, QuantOutputs{});
  OMCUDA_CHECK_LAUNCH("quantize_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevDequantizeLinear(const void *x, int dtype, int64_t n,
    const float *scale, const void *zp, float *y, void *stream) {
  if (n < 0 || (n > 0 && (!x || !y)) || !scale || dtype < 0 || dtype > 2)
    return fail(OMCUDA_EINVAL, "DequantizeLinear: bad argument");
  if (n == 0)
    return OMCUDA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  int grid = grid_for(n, 256 * 4);
  if (dtype == 0)
    dequantize_kernel<uint8_t><<<grid, 256, 0, st>>>(
        (const uint8_t *)x, n, scale, (const uint8_t *)zp, y);
  else if (dtype == 1)
    dequantize_kernel<int8_t><<<grid, 256, 0, st>>>(
        (const int8_t *)x, n, scale, (const int8_t *)zp, y);
  else
    dequantize_kernel<int32_t><<<grid, 256, 0, st>>>(
        (const int32_t *)x, n, scale, (const int32_t *)zp, y);
  OMCUDA_CHECK_LAUNCH("dequantize_kernel");
  return OMCUDA_OK;
}
