// fp32 kernels for the ops a dynamic-quantized encoder graph holds between its
// quantized linears, so that activations never leave HBM:
//   Softmax             src/Conversion/ONNXToKrnl/Math/Softmax.cpp:25-134
//   LayerNormalization  src/Conversion/ONNXToKrnl/NN/Normalization.cpp:748-880
//   Gelu (erf)          src/Conversion/ONNXToKrnl/Math/Elementwise.cpp:358-388
//   Add                 src/Conversion/ONNXToKrnl/Math/Elementwise.cpp
//   Transpose (0,2,1,3) src/Conversion/ONNXToKrnl/Tensor/Transpose.cpp
//   MatMul fp32         src/Conversion/ONNXToKrnl/Math/MatMul.cpp:488-507
// Reductions are reordered relative to the reference's sequential loops; the
// parity tolerance for these ops is 1e-3 relative.
#include <cstdlib>
#include <cstring>

#include "../runtime/internal.h"
#include "../common.cuh"

namespace omcuda {

// ---- Softmax over the last axis: one warp per row --------------------------------

__global__ void __launch_bounds__(256)
    softmax_rows_kernel(const float *__restrict__ x, int64_t rows, int64_t cols,
        float *__restrict__ y) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows)
    return;
  const float *xr = x + r * cols;
  float *yr = y + r * cols;
  float mx = -INFINITY;
  for (int64_t c = lane; c < cols; c += 32)
    mx = fmaxf(mx, xr[c]);
  mx = warp_max(mx);
  float sum = 0.0f;
  for (int64_t c = lane; c < cols; c += 32) {
    float e = expf(__fsub_rn(xr[c], mx));
    yr[c] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  for (int64_t c = lane; c < cols; c += 32)
    yr[c] = __fdiv_rn(yr[c], sum);
}

// ---- LayerNorm (optionally of x + residual): one warp per row ----------------------

__global__ void __launch_bounds__(256)
    layernorm_rows_kernel(const float *__restrict__ x,
        const float *__restrict__ residual, int64_t rows, int64_t cols,
        const float *__restrict__ gamma, const float *__restrict__ beta,
        float eps, float *__restrict__ y, uint32_t *__restrict__ out_range) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  float lo = INFINITY, hi = -INFINITY;
  if (r < rows) {
    const float *xr = x + r * cols;
    const float *rr = residual ? residual + r * cols : nullptr;
    float *yr = y + r * cols;
    float s = 0.0f, s2 = 0.0f;
    for (int64_t c = lane; c < cols; c += 32) {
      float v = xr[c];
      if (rr)
        v = __fadd_rn(v, rr[c]);
      s += v;
      s2 += __fmul_rn(v, v);
    }
    s = warp_sum(s);
    s2 = warp_sum(s2);
    const float nf = (float)cols;
    const float mean = __fdiv_rn(s, nf);
    const float mean2 = __fdiv_rn(s2, nf);
    const float var = __fsub_rn(mean2, __fmul_rn(mean, mean));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
    for (int64_t c = lane; c < cols; c += 32) {
      float v = xr[c];
      if (rr)
        v = __fadd_rn(v, rr[c]);
      float o = __fmul_rn(__fmul_rn(__fsub_rn(v, mean), inv), gamma[c]);
      if (beta)
        o = __fadd_rn(o, beta[c]);
      yr[c] = o;
      lo = fminf(lo, o);
      hi = fmaxf(hi, o);
    }
  }
  if (out_range)
    range_commit_warp(out_range, lo, hi);
}

// Same function for rows of NV * 128 floats (hidden sizes 768 and 1024): one
// warp per row, the row held in registers as NV float4 per lane, so x and the
// residual are read from HBM exactly once, with 16-byte accesses.
template <int NV>
__global__ void __launch_bounds__(256)
    layernorm_rows_vec_kernel(const float *__restrict__ x,
        const float *__restrict__ residual, int64_t rows,
        const float *__restrict__ gamma, const float *__restrict__ beta,
        float eps, float *__restrict__ y, uint32_t *__restrict__ out_range) {
  constexpr int64_t cols = (int64_t)NV * 128;
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  float lo = INFINITY, hi = -INFINITY;
  if (r < rows) {
    const float4 *xr = reinterpret_cast<const float4 *>(x + r * cols);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i)
      v[i] = __ldcs(xr + lane + 32 * i);
    if (residual) {
      const float4 *rr = reinterpret_cast<const float4 *>(residual + r * cols);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const float4 q = __ldcs(rr + lane + 32 * i);
        v[i].x = __fadd_rn(v[i].x, q.x);
        v[i].y = __fadd_rn(v[i].y, q.y);
        v[i].z = __fadd_rn(v[i].z, q.z);
        v[i].w = __fadd_rn(v[i].w, q.w);
      }
    }
    float s = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      s2 += (__fmul_rn(v[i].x, v[i].x) + __fmul_rn(v[i].y, v[i].y)) +
            (__fmul_rn(v[i].z, v[i].z) + __fmul_rn(v[i].w, v[i].w));
    }
    s = warp_sum(s);
    s2 = warp_sum(s2);
    const float nf = (float)cols;
    const float mean = __fdiv_rn(s, nf);
    const float mean2 = __fdiv_rn(s2, nf);
    const float var = __fsub_rn(mean2, __fmul_rn(mean, mean));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
    const float4 *g4 = reinterpret_cast<const float4 *>(gamma);
    const float4 *b4 = reinterpret_cast<const float4 *>(beta);
    float4 *yr = reinterpret_cast<float4 *>(y + r * cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const float4 g = __ldg(g4 + lane + 32 * i);
      float4 o;
      o.x = __fmul_rn(__fmul_rn(__fsub_rn(v[i].x, mean), inv), g.x);
      o.y = __fmul_rn(__fmul_rn(__fsub_rn(v[i].y, mean), inv), g.y);
      o.z = __fmul_rn(__fmul_rn(__fsub_rn(v[i].z, mean), inv), g.z);
      o.w = __fmul_rn(__fmul_rn(__fsub_rn(v[i].w, mean), inv), g.w);
      if (beta) {
        const float4 bb = __ldg(b4 + lane + 32 * i);
        o.x = __fadd_rn(o.x, bb.x);
        o.y = __fadd_rn(o.y, bb.y);
        o.z = __fadd_rn(o.z, bb.z);
        o.w = __fadd_rn(o.w, bb.w);
      }
      yr[lane + 32 * i] = o;
      lo = fminf(lo, fminf(fminf(o.x, o.y), fminf(o.z, o.w)));
      hi = fmaxf(hi, fmaxf(fmaxf(o.x, o.y), fmaxf(o.z, o.w)));
    }
  }
  if (out_range)
    range_commit_warp(out_range, lo, hi);
}

// ---- elementwise -------------------------------------------------------------------

__global__ void __launch_bounds__(256)
    gelu_kernel(const float *__restrict__ x, int64_t n, float *__restrict__ y) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if ((((uintptr_t)x | (uintptr_t)y) & 15u) == 0) {
    const int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += stride) {
      float4 v = reinterpret_cast<const float4 *>(x)[i];
      v.x = gelu_erf(v.x);
      v.y = gelu_erf(v.y);
      v.z = gelu_erf(v.z);
      v.w = gelu_erf(v.w);
      reinterpret_cast<float4 *>(y)[i] = v;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride)
      y[i] = gelu_erf(x[i]);
  } else {
    for (int64_t i = tid; i < n; i += stride)
      y[i] = gelu_erf(x[i]);
  }
}

__global__ void __launch_bounds__(256)
    add_kernel(const float *__restrict__ a, const float *__restrict__ b,
        int64_t n, float *__restrict__ y) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)y) & 15u) == 0) {
    const int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += stride) {
      float4 u = reinterpret_cast<const float4 *>(a)[i];
      float4 v = reinterpret_cast<const float4 *>(b)[i];
      reinterpret_cast<float4 *>(y)[i] = make_float4(__fadd_rn(u.x, v.x),
          __fadd_rn(u.y, v.y), __fadd_rn(u.z, v.z), __fadd_rn(u.w, v.w));
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride)
      y[i] = __fadd_rn(a[i], b[i]);
  } else {
    for (int64_t i = tid; i < n; i += stride)
      y[i] = __fadd_rn(a[i], b[i]);
  }
}

// [B,S,H,D] -> [B,H,S,D]: rows of D floats move as units.
__global__ void __launch_bounds__(256)
    transpose_0213_kernel(const float *__restrict__ x, int64_t B, int64_t S,
        int64_t H, int64_t D, float *__restrict__ y) {
  const int64_t total = B * S * H * D;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (int64_t)gridDim.x * blockDim.x) {
    int64_t d = o % D;
    int64_t s = (o / D) % S;
    int64_t h = (o / (D * S)) % H;
    int64_t b = o / (D * S * H);
    y[o] = x[((b * S + s) * H + h) * D + d];
  }
}

// ---- batched fp32 matmul: 64x64 tile, 16-deep, 4x4 per thread ----------------------

__global__ void __launch_bounds__(256)
    matmul_f32_kernel(const float *__restrict__ A, const float *__restrict__ Bm,
        int64_t M, int64_t N, int64_t K, float *__restrict__ C) {
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64 + 1];
  const int64_t batch = blockIdx.z;
  A += batch * M * K;
  Bm += batch * K * N;
  C += batch * M * N;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      int r = i >> 4, c = i & 15; // A tile: 64 rows x 16 k
      int64_t m = m0 + r, k = k0 + c;
      As[c][r] = (m < M && k < K) ? A[m * K + k] : 0.0f;
    }
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      int r = i >> 6, c = i & 63; // B tile: 16 k x 64 cols
      int64_t k = k0 + r, n = n0 + c;
      Bs[r][c] = (k < K && n < N) ? Bm[k * N + n] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[k][ty * 4 + i];
        b[i] = Bs[k][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      int64_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N)
        C[m * N + n] = acc[i][j];
    }
}

// ---- attention: softmax(Q K^T * scale) V per (batch, head) ---------------------------
//
// Q, K, V, out are [B, S, heads*dh] (the layout the linears produce), so the
// Reshape/Transpose pairs of the graph are folded into the addressing.  One
// block serves one (b, h) and kRows query rows per warp; keys stream through
// shared memory in tiles of 32.  Scores for a query row stay in shared memory
// (S floats), so the three softmax passes never touch HBM.
constexpr int kAttWarps = 4;
constexpr int kAttRows = 4; // query rows per warp

template <int DH>
__global__ void __launch_bounds__(kAttWarps * 32)
    attention_kernel(const float *__restrict__ Q, const float *__restrict__ Kt,
        const float *__restrict__ V, int64_t S, int64_t heads, float scale,
        float *__restrict__ out, int64_t ld_in, int64_t ld_out,
        uint32_t *__restrict__ out_range) {
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t bh = blockIdx.y;
  const int64_t b = bh / heads, h = bh % heads;
  const int64_t H = ld_in;   // row pitch of Q, K, V in floats
  const int64_t Ho = ld_out; // row pitch of out
  const int64_t q0 = ((int64_t)blockIdx.x * kAttWarps + warp) * kAttRows;
  // smem: Ktile[DH][33] | Vtile[32][DH] | q[warps][rows][DH] | p[warps][rows][S]
  float *ktile = smem;
  float *vtile = ktile + DH * 33;
  float *qs = vtile + 32 * DH + (warp * kAttRows) * DH;
  float *ps = vtile + 32 * DH + kAttWarps * kAttRows * DH +
              (int64_t)(warp * kAttRows) * S;
  for (int r = 0; r < kAttRows; ++r) {
    int64_t qi = q0 + r;
    for (int d = lane; d < DH; d += 32)
      qs[r * DH + d] = (qi < S) ? Q[(b * S + qi) * H + h * DH + d] : 0.0f;
  }
  // Pass 1: scores.
  for (int64_t j0 = 0; j0 < S; j0 += 32) {
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * DH; i += blockDim.x) {
      int j = i / DH, d = i % DH;
      int64_t kj = j0 + j;
      ktile[d * 33 + j] = (kj < S) ? Kt[(b * S + kj) * H + h * DH + d] : 0.0f;
    }
    __syncthreads();
    float acc[kAttRows];
#pragma unroll
    for (int r = 0; r < kAttRows; ++r)
      acc[r] = 0.0f;
#pragma unroll 8
    for (int d = 0; d < DH; ++d) {
      float kv = ktile[d * 33 + lane];
#pragma unroll
      for (int r = 0; r < kAttRows; ++r)
        acc[r] = __fadd_rn(acc[r], __fmul_rn(qs[r * DH + d], kv));
    }
    if (j0 + lane < S) {
#pragma unroll
      for (int r = 0; r < kAttRows; ++r)
        ps[(int64_t)r * S + j0 + lane] = __fmul_rn(acc[r], scale);
    }
  }
  __syncwarp();
  // Softmax per row (max, exp and sum, divide).
  for (int r = 0; r < kAttRows; ++r) {
    float *p = ps + (int64_t)r * S;
    float mx = -INFINITY;
    for (int64_t j = lane; j < S; j += 32)
      mx = fmaxf(mx, p[j]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int64_t j = lane; j < S; j += 32) {
      float e = expf(__fsub_rn(p[j], mx));
      p[j] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    for (int64_t j = lane; j < S; j += 32)
      p[j] = __fdiv_rn(p[j], sum);
  }
  // Pass 2: P V.  Lane owns output dims lane, lane+32, ...
  constexpr int kDPer = (DH + 31) / 32;
  float o[kAttRows][kDPer];
#pragma unroll
  for (int r = 0; r < kAttRows; ++r)
#pragma unroll
    for (int i = 0; i < kDPer; ++i)
      o[r][i] = 0.0f;
  for (int64_t j0 = 0; j0 < S; j0 += 32) {
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * DH; i += blockDim.x) {
      int j = i / DH, d = i % DH;
      int64_t kj = j0 + j;
      vtile[j * DH + d] = (kj < S) ? V[(b * S + kj) * H + h * DH + d] : 0.0f;
    }
    __syncthreads();
    const int jn = (int)((S - j0) < 32 ? (S - j0) : 32);
    for (int j = 0; j < jn; ++j) {
#pragma unroll
      for (int i = 0; i < kDPer; ++i) {
        int d = lane + 32 * i;
        float vv = (d < DH) ? vtile[j * DH + d] : 0.0f;
#pragma unroll
        for (int r = 0; r < kAttRows; ++r)
          o[r][i] = __fadd_rn(o[r][i],
              __fmul_rn(ps[(int64_t)r * S + j0 + j], vv));
      }
    }
  }
  float lo = INFINITY, hi = -INFINITY;
  for (int r = 0; r < kAttRows; ++r) {
    int64_t qi = q0 + r;
    if (qi >= S)
      continue;
#pragma unroll
    for (int i = 0; i < kDPer; ++i) {
      int d = lane + 32 * i;
      if (d < DH) {
        out[(b * S + qi) * Ho + h * DH + d] = o[r][i];
        lo = fminf(lo, o[r][i]);
        hi = fmaxf(hi, o[r][i]);
      }
    }
  }
  if (out_range)
    range_commit_warp(out_range, lo, hi);
}

// Arms running {min,max} ranges (ordered-uint encoding): min side all ones,
// max side zero, so that the first value folded in replaces both.
__global__ void range_init_kernel(uint32_t *ranges, int count) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) {
    ranges[2 * i] = 0xffffffffu;
    ranges[2 * i + 1] = 0u;
  }
}

static int ew_grid(int64_t n, int per_thread) {
  int64_t want = ceil_div(n, 256 * per_thread);
  int64_t cap = (int64_t)sm_count() * 8;
  if (want < 1)
    want = 1;
  return (int)(want < cap ? want : cap);
}

} // namespace omcuda

using namespace omcuda;

extern "C" int omcudaDevSoftmax(
    const float *x, int64_t rows, int64_t cols, float *y, void *stream) {
  if (rows < 0 || cols <= 0 || (rows > 0 && (!x || !y)))
    return fail(OMCUDA_EINVAL, "Softmax: bad argument");
  if (rows == 0)
    return OMCUDA_OK;
  softmax_rows_kernel<<<(unsigned)ceil_div(rows, 8), 256, 0,
      (cudaStream_t)stream>>>(x, rows, cols, y);
  OMCUDA_CHECK_LAUNCH("softmax_rows_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevLayerNorm(const float *x, const float *residual,
    int64_t rows, int64_t cols, const float *gamma, const float *beta,
    float eps, float *y, void *out_minmax, void *stream) {
  if (rows < 0 || cols <= 0 || (rows > 0 && (!x || !y)) || !gamma)
    return fail(OMCUDA_EINVAL, "LayerNormalization: bad argument");
  if (rows == 0)
    return OMCUDA_OK;
  const bool vec_ok = ((((uintptr_t)x | (uintptr_t)residual | (uintptr_t)gamma |
                            (uintptr_t)beta | (uintptr_t)y) & 15u) == 0);
  const unsigned grid = (unsigned)ceil_div(rows, 8);
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t *rng = reinterpret_cast<uint32_t *>(out_minmax);
  if (vec_ok && cols == 768)
    layernorm_rows_vec_kernel<6><<<grid, 256, 0, st>>>(
        x, residual, rows, gamma, beta, eps, y, rng);
  else if (vec_ok && cols == 1024)
    layernorm_rows_vec_kernel<8><<<grid, 256, 0, st>>>(
        x, residual, rows, gamma, beta, eps, y, rng);
  else
    layernorm_rows_kernel<<<grid, 256, 0, st>>>(
        x, residual, rows, cols, gamma, beta, eps, y, rng);
  OMCUDA_CHECK_LAUNCH("layernorm_rows_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevGelu(const float *x, int64_t n, float *y, void *stream) {
  if (n < 0 || (n > 0 && (!x || !y)))
    return fail(OMCUDA_EINVAL, "Gelu: bad argument");
  if (n == 0)
    return OMCUDA_OK;
  gelu_kernel<<<ew_grid(n, 8), 256, 0, (cudaStream_t)stream>>>(x, n, y);
  OMCUDA_CHECK_LAUNCH("gelu_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevAdd(
    const float *a, const float *b, int64_t n, float *y, void *stream) {
  if (n < 0 || (n > 0 && (!a || !b || !y)))
    return fail(OMCUDA_EINVAL, "Add: bad argument");
  if (n == 0)
    return OMCUDA_OK;
  add_kernel<<<ew_grid(n, 8), 256, 0, (cudaStream_t)stream>>>(a, b, n, y);
  OMCUDA_CHECK_LAUNCH("add_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevTranspose0213(const float *x, int64_t B, int64_t S,
    int64_t H, int64_t D, float *y, void *stream) {
  int64_t n = B * S * H * D;
  if (n < 0 || (n > 0 && (!x || !y)))
    return fail(OMCUDA_EINVAL, "Transpose: bad argument");
  if (n == 0)
    return OMCUDA_OK;
  transpose_0213_kernel<<<ew_grid(n, 4), 256, 0, (cudaStream_t)stream>>>(
      x, B, S, H, D, y);
  OMCUDA_CHECK_LAUNCH("transpose_0213_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevMatMulF32(const float *A, const float *B, int64_t batch,
    int64_t M, int64_t N, int64_t K, float *C, void *stream) {
  if (batch < 0 || M < 0 || N <= 0 || K <= 0 || !A || !B || !C)
    return fail(OMCUDA_EINVAL, "MatMul: bad argument");
  if (batch == 0 || M == 0)
    return OMCUDA_OK;
  if (batch > 65535)
    return fail(OMCUDA_ENOTSUP, "MatMul: more than 65535 batches");
  dim3 grid((unsigned)ceil_div(N, 64), (unsigned)ceil_div(M, 64), (unsigned)batch);
  matmul_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, B, M, N, K, C);
  OMCUDA_CHECK_LAUNCH("matmul_f32_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevRangeInit(void *ranges, int64_t count, void *stream) {
  if (!ranges || count <= 0)
    return fail(OMCUDA_EINVAL, "RangeInit: bad argument");
  range_init_kernel<<<(unsigned)ceil_div(count, 128), 128, 0,
      (cudaStream_t)stream>>>((uint32_t *)ranges, (int)count);
  OMCUDA_CHECK_LAUNCH("range_init_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevAttention(const float *Q, const float *K, const float *V,
    int64_t B, int64_t S, int64_t heads, int64_t dh, float scale, float *out,
    void *stream) {
  return omcudaDevAttentionEx(Q, K, V, B, S, heads, dh, scale, out, heads * dh,
      heads * dh, nullptr, stream);
}

extern "C" int omcudaDevAttentionEx(const float *Q, const float *K,
    const float *V, int64_t B, int64_t S, int64_t heads, int64_t dh,
    float scale, float *out, int64_t ld_in, int64_t ld_out, void *out_range,
    void *stream) {
  if (B < 0 || S <= 0 || heads <= 0 || !Q || !K || !V || !out ||
      ld_in < heads * dh || ld_out < heads * dh)
    return fail(OMCUDA_EINVAL, "Attention: bad argument");
  if (B == 0)
    return OMCUDA_OK;
  if (dh != 64 && dh != 32 && dh != 128)
    return fail(OMCUDA_ENOTSUP, "Attention: head size must be 32, 64 or 128");
  if (B * heads > 65535)
    return fail(OMCUDA_ENOTSUP, "Attention: batch*heads exceeds 65535");
  // Tensor-core kernel unless the rows are not aligned for it or the SIMT
  // kernel is asked for (OMCUDA_ATTENTION=simt, used to cross-check the two).
  static const bool force_simt = [] {
    const char *s = getenv("OMCUDA_ATTENTION");
    return s && strcmp(s, "simt") == 0;
  }();
  if (!force_simt && attention_mma_supported(Q, K, V, out, dh, ld_in, ld_out))
    return launch_attention_mma(Q, K, V, B, S, heads, dh, scale, out, ld_in,
        ld_out, out_range, (cudaStream_t)stream);
  size_t smem = (size_t)(dh * 33 + 32 * dh + kAttWarps * kAttRows * dh +
                         (int64_t)kAttWarps * kAttRows * S) *
                sizeof(float);
  if (smem > 200 * 1024)
    return fail(OMCUDA_ENOTSUP, "Attention: sequence too long for this kernel");
  dim3 grid((unsigned)ceil_div(S, kAttWarps * kAttRows), (unsigned)(B * heads));
  cudaStream_t st = (cudaStream_t)stream;
#define OMCUDA_LAUNCH_ATT(DH)                                                  \
  do {                                                                         \
    OMCUDA_CHECK(cudaFuncSetAttribute(attention_kernel<DH>,                    \
        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));              \
    attention_kernel<DH><<<grid, kAttWarps * 32, smem, st>>>(Q, K, V, S,       \
        heads, scale, out, ld_in, ld_out, (uint32_t *)out_range);              \
  } while (0)
  if (dh == 64)
    OMCUDA_LAUNCH_ATT(64);
  else if (dh == 32)
    OMCUDA_LAUNCH_ATT(32);
  else
    OMCUDA_LAUNCH_ATT(128);
#undef OMCUDA_LAUNCH_ATT
  OMCUDA_CHECK_LAUNCH("attention_kernel");
  return OMCUDA_OK;
}
