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
#include "../runtime/internal.h"
#include "quantize.cuh"

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

__global__ void __launch_bounds__(kDqlThreads)
    dql_minmax_kernel(const float *__restrict__ x, int64_t n,
        DqlScratch *__restrict__ scr, float *__restrict__ y_scale,
        uint8_t *__restrict__ y_zp, int mode) {
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
    dql_params_from_range(lo, hi, &s, &z, mode);
    scr->params[0] = s;
    scr->params[1] = z;
    if (y_scale)
      *y_scale = s;
    if (y_zp)
      *y_zp = (uint8_t)(unsigned int)z; // fptoui then trunc; z is in [0,255]
    scr->ticket = 0; // leave the scratch ready for the next call
  }
}

// Folds the min / max of x into a running range (the encoding and the commit
// rule of range_commit_warp): the reduction of DynamicQuantizeLinear in the
// form the producers of the encoder harness use, for a tensor that has no
// producer on the device.
__global__ void __launch_bounds__(kDqlThreads)
    range_fold_kernel(const float *__restrict__ x, int64_t n, uint32_t *__restrict__ range) {
  float lo = INFINITY, hi = -INFINITY;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if ((((uintptr_t)x) & 15u) == 0) {
    const int64_t n4 = n >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    for (int64_t i = tid; i < n4; i += nthreads) {
      const float4 a = __ldcs(x4 + i);
      lo = fminf(lo, fminf(fminf(a.x, a.y), fminf(a.z, a.w)));
      hi = fmaxf(hi, fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)));
    }
    for (int64_t j = (n4 << 2) + tid; j < n; j += nthreads) {
      lo = fminf(lo, x[j]);
      hi = fmaxf(hi, x[j]);
    }
  } else {
    for (int64_t j = tid; j < n; j += nthreads) {
      lo = fminf(lo, x[j]);
      hi = fmaxf(hi, x[j]);
    }
  }
  range_commit_warp(range, lo, hi);
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
        int has_zp, const uint32_t *__restrict__ range, QuantOutputs outs, int mode) {
  float scale, zp_f;
  if (range) {
    // Scale and zero point straight from a producer's running range (every
    // thread derives the same two scalars; block 0 also publishes them for
    // the ops that follow).
    dql_params_from_range(ordered_to_f32(__ldg(range)), ordered_to_f32(__ldg(range + 1)),
        &scale, &zp_f, mode);
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
  const QuantConsts qc = make_quant_consts(scale, zp_f, mode);
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
      x, n, y, params, nullptr, nullptr, 1, nullptr, QuantOutputs{}, quant_mode());
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
  dql_minmax_kernel<<<grid, kDqlThreads, 0, st>>>(x, n, scr, y_scale, y_zp, quant_mode());
  OMCUDA_CHECK_LAUNCH("dql_minmax_kernel");
  if (n > 0)
    return launch_quantize_with_params(x, n, y, scr->params, st);
  return OMCUDA_OK;
}

extern "C" int omcudaDevRangeFold(const float *x, int64_t n, void *range, void *stream) {
  if (n < 0 || (n > 0 && !x) || !range)
    return fail(OMCUDA_EINVAL, "RangeFold: bad argument");
  if (n == 0)
    return OMCUDA_OK;
  int grid = grid_for(n, kDqlThreads * 16);
  range_fold_kernel<<<grid, kDqlThreads, 0, (cudaStream_t)stream>>>(x, n, (uint32_t *)range);
  OMCUDA_CHECK_LAUNCH("range_fold_kernel");
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
      x, n, y, nullptr, nullptr, nullptr, 1, (const uint32_t *)range, outs, quant_mode());
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
        x, n, (uint8_t *)y, nullptr, scale, zp, zp != nullptr, nullptr, QuantOutputs{},
        quant_mode());
  else
    quantize_kernel<false><<<grid, kDqlThreads, 0, st>>>(
        x, n, (uint8_t *)y, nullptr, scale, zp, zp != nullptr, nullptr, QuantOutputs{},
        quant_mode());
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
  if (quant_mode() & OMCUDA_MODE_NO_ZERO_POINT)
    zp = nullptr; // the reference drops the subtraction (Math/Elementwise.cpp:1453)
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
