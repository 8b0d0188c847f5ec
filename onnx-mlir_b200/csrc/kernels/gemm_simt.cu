// Operand preparation for the int8 GEMMs and the SIMT (dp4a) GEMM.
//
// prepare_b: B arrives [K,N] row-major (the ONNX layout of a MatMulInteger /
// QLinearMatMul weight).  Both GEMM kernels consume it K-major, so it is
// copied once into Bt[N][kp] (kp = K rounded up to 16, zero padded) together
// with its column sums, which carry the A zero point through the epilogue
// (see gemm_epilogue.cuh).
//
// gemm_i8_warp_kernel: one warp per output column n and per group of MT rows;
// the 32 lanes split K in 16-byte chunks (coalesced 512-byte reads of the Bt
// row), accumulate with dp4a, and fold with shuffles.  It is the path for
// small M, where the GEMM is bound by reading the weight once from HBM, and
// for shapes the tensor-core kernel does not take (K not a multiple of 16,
// unaligned bases).  Integer accumulation wraps in 32 bits in any order, so
// its results are bit-identical to the tensor-core kernel's.
#include <cstdlib>

#include "../runtime/internal.h"
#include "gemm_epilogue.cuh"

namespace omcuda {

// ---- B preparation -----------------------------------------------------------

__global__ void __launch_bounds__(256)
    transpose_b_kernel(const uint8_t *__restrict__ B, int64_t K, int64_t N,
        int64_t kp, uint8_t *__restrict__ Bt) {
  // 64(k) x 64(n) byte tile through shared memory; reads are coalesced along
  // n, writes along k.
  __shared__ uint8_t tile[64][65];
  const int64_t k0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6; // 64 x 4
  for (int r = ty; r < 64; r += 4) {
    int64_t k = k0 + r, n = n0 + tx;
    tile[r][tx] = (k < K && n < N) ? B[k * N + n] : (uint8_t)0;
  }
  __syncthreads();
  for (int r = ty; r < 64; r += 4) {
    int64_t n = n0 + r, k = k0 + tx;
    if (n < N && k < kp)
      Bt[n * kp + k] = tile[tx][r];
  }
}

template <bool kSigned>
__global__ void __launch_bounds__(256)
    colsum_kernel(const uint8_t *__restrict__ B, int64_t K, int64_t N,
        int32_t *__restrict__ colsum) {
  // blockDim = (64, 4): 64 columns per block, K split four ways.
  __shared__ int32_t part[4][64];
  const int64_t n = (int64_t)blockIdx.x * 64 + threadIdx.x;
  int32_t s = 0;
  if (n < N) {
    for (int64_t k = threadIdx.y; k < K; k += 4) {
      uint8_t b = B[k * N + n];
      s += kSigned ? (int32_t)(int8_t)b : (int32_t)b;
    }
  }
  part[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && n < N)
    colsum[n] = part[0][threadIdx.x] + part[1][threadIdx.x] +
                part[2][threadIdx.x] + part[3][threadIdx.x];
}

template <bool kSigned>
__global__ void __launch_bounds__(256)
    rowsum_kernel(const uint8_t *__restrict__ A, int64_t M, int64_t K,
        int32_t *__restrict__ rowsum) {
  // One warp per row.
  const int64_t m = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= M)
    return;
  const int lane = threadIdx.x & 31;
  int32_t s = 0;
  for (int64_t k = lane; k < K; k += 32) {
    uint8_t a = A[m * K + k];
    s += kSigned ? (int32_t)(int8_t)a : (int32_t)a;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0)
    rowsum[m] = s;
}

__global__ void requant_scale_kernel(const float *__restrict__ a_scale,
    const float *__restrict__ b_scale, int64_t len,
    const float *__restrict__ y_scale, float *__restrict__ S) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < len)
    S[i] = __fdiv_rn(__fmul_rn(*a_scale, b_scale[i]), *y_scale);
}

// ---- SIMT GEMM ----------------------------------------------------------------

template <bool kASigned, bool kBSigned>
__device__ __forceinline__ int32_t dp4a_mixed(uint32_t a, uint32_t b, int32_t c) {
  int32_t d;
  if (kASigned && kBSigned)
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  else if (kASigned && !kBSigned)
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  else if (!kASigned && kBSigned)
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  else
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__device__ __forceinline__ uint4 load_a_chunk(const uint8_t *__restrict__ A,
    int64_t m, int64_t M, int64_t K, int64_t k0, bool vec_ok) {
  uint4 v = make_uint4(0, 0, 0, 0);
  if (m >= M)
    return v;
  if (vec_ok && k0 + 16 <= K)
    return __ldg(reinterpret_cast<const uint4 *>(A + m * K + k0));
  uint32_t w[4] = {0, 0, 0, 0};
  for (int j = 0; j < 16; ++j) {
    int64_t k = k0 + j;
    if (k < K)
      w[j >> 2] |= (uint32_t)A[m * K + k] << (8 * (j & 3));
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <int MT, bool kASigned, bool kBSigned>
__global__ void __launch_bounds__(256)
    gemm_i8_warp_kernel(const uint8_t *__restrict__ A,
        const uint8_t *__restrict__ Bt, int64_t kp, EpiParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t m0 = (int64_t)blockIdx.y * MT;
  if (n >= p.N)
    return; // whole warp leaves together
  const bool vec_ok = ((p.K & 15) == 0) && (((uintptr_t)A & 15u) == 0);
  int32_t acc[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i)
    acc[i] = 0;
  const uint4 *brow = reinterpret_cast<const uint4 *>(Bt + n * kp);
  const int64_t chunks = kp >> 4;
  for (int64_t c = lane; c < chunks; c += 32) {
    uint4 b = __ldg(brow + c);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      uint4 a = load_a_chunk(A, m0 + i, p.M, p.K, c << 4, vec_ok);
      int32_t s = acc[i];
      s = dp4a_mixed<kASigned, kBSigned>(a.x, b.x, s);
      s = dp4a_mixed<kASigned, kBSigned>(a.y, b.y, s);
      s = dp4a_mixed<kASigned, kBSigned>(a.z, b.z, s);
      s = dp4a_mixed<kASigned, kBSigned>(a.w, b.w, s);
      acc[i] = s;
    }
  }
#pragma unroll
  for (int i = 0; i < MT; ++i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  }
  // Lane i finishes row m0+i (MT <= 32).
  const EpiScalars sc = epi_scalars(p);
  float lo = INFINITY, hi = -INFINITY;
  int32_t mine = 0;
#pragma unroll
  for (int i = 0; i < MT; ++i)
    if (lane == i)
      mine = acc[i];
  const int64_t m = m0 + lane;
  if (lane < MT && m < p.M) {
    EpiRow row = epi_row(p, m);
    int32_t v = epi_int(p, row, mine, n);
    if (p.kind == OMCUDA_EPI_I32) {
      reinterpret_cast<int32_t *>(p.Y)[m * p.N + n] = v;
    } else if (p.kind == OMCUDA_EPI_DEQUANT) {
      float y = epi_dequant(p, sc, v, n);
      if (p.residual)
        y = __fadd_rn(y, __ldg(p.residual + m * p.N + n));
      reinterpret_cast<float *>(p.Y)[m * p.N + n] = y;
      lo = fminf(lo, y);
      hi = fmaxf(hi, y);
    } else {
      reinterpret_cast<uint8_t *>(p.Y)[m * p.N + n] =
          (uint8_t)epi_requant(p, sc, v, n);
    }
  }
  if (p.out_range && p.kind == OMCUDA_EPI_DEQUANT)
    epi_range_commit(p.out_range, lo, hi);
}


// ---- GEMV-shaped GEMM for M <= 16 ----------------------------------------------
//
// With a handful of rows the GEMM is one pass over the K*N bytes of the
// weight: HBM bound.  A block of kGemvWarps warps owns CB adjacent output
// columns (CB rows of Bt) and MT rows of A, and splits K between its warps:
// chunk c (16 bytes of K) goes to thread c mod (32 * kGemvWarps), so that a
// warp-wide load of Bt is one coalesced 512-byte access and every SM keeps
// tens of kilobytes of weight reads in flight (CB loads per thread and trip,
// trips unrolled by two).  A is tiny (M*K bytes) and is served by L1; loading
// one A chunk for CB columns keeps the L1 traffic per weight byte at MT / CB.
// The partial sums are folded with shuffles inside each warp and through
// shared memory between the warps (no global workspace, no atomics); the
// first MT * CB threads of the block run the epilogue.  Integer addition is
// exact in any order, so the result equals the other kernels' bit for bit.
constexpr int kGemvWarps = 4;

template <int MT, int CB, bool kASigned, bool kBSigned>
__global__ void __launch_bounds__(32 * kGemvWarps)
    gemm_i8_gemv_kernel(const uint8_t *__restrict__ A,
        const uint8_t *__restrict__ Bt, int64_t kp, EpiParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t m0 = (int64_t)blockIdx.y * MT;
  const bool vec_ok = ((p.K & 15) == 0) && (((uintptr_t)A & 15u) == 0);
  const int64_t chunks = kp >> 4;
  constexpr int kStep = 32 * kGemvWarps;
  __shared__ int32_t part[kGemvWarps][MT * CB];
  static_assert(MT * CB <= 32, "the epilogue runs in the first warp");
  const EpiScalars sc = epi_scalars(p);
  float lo = INFINITY, hi = -INFINITY;
  // A block walks column groups (grid-stride), so that a launch is a few
  // resident blocks per SM streaming the weight rather than thousands of
  // short-lived ones.
  const int64_t groups = ceil_div(p.N, CB);
  for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
    const int64_t n0 = g * CB;
    int32_t acc[MT][CB];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < CB; ++j)
        acc[i][j] = 0;
    const uint4 *brow[CB];
#pragma unroll
    for (int j = 0; j < CB; ++j) // columns past N re-read the last one; never stored
      brow[j] = reinterpret_cast<const uint4 *>(Bt + (n0 + j < p.N ? n0 + j : p.N - 1) * kp);
    auto consume = [&](int64_t c, const uint4 (&b)[CB]) {
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const uint4 a = load_a_chunk(A, m0 + i, p.M, p.K, c << 4, vec_ok);
#pragma unroll
        for (int j = 0; j < CB; ++j) {
          int32_t s = acc[i][j];
          s = dp4a_mixed<kASigned, kBSigned>(a.x, b[j].x, s);
          s = dp4a_mixed<kASigned, kBSigned>(a.y, b[j].y, s);
          s = dp4a_mixed<kASigned, kBSigned>(a.z, b[j].z, s);
          s = dp4a_mixed<kASigned, kBSigned>(a.w, b[j].w, s);
          acc[i][j] = s;
        }
      }
    };
    int64_t c = threadIdx.x;
    for (; c + kStep < chunks; c += 2 * kStep) {
      uint4 b0[CB], b1[CB];
#pragma unroll
      for (int j = 0; j < CB; ++j) {
        b0[j] = __ldcs(brow[j] + c);
        b1[j] = __ldcs(brow[j] + c + kStep);
      }
      consume(c, b0);
      consume(c + kStep, b1);
    }
    if (c < chunks) {
      uint4 b0[CB];
#pragma unroll
      for (int j = 0; j < CB; ++j)
        b0[j] = __ldcs(brow[j] + c);
      consume(c, b0);
    }
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < CB; ++j) {
        int32_t v = acc[i][j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
          v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0)
          part[warp][i * CB + j] = v;
      }
    __syncthreads();
    // Thread t of the first warp finishes output (row m0 + t / CB, column n0 + t % CB).
    if (warp == 0) {
      const int64_t m = m0 + lane / CB, n = n0 + lane % CB;
      if (lane < MT * CB && m < p.M && n < p.N) {
        int32_t sum = 0;
#pragma unroll
        for (int w = 0; w < kGemvWarps; ++w)
          sum += part[w][lane];
        const EpiRow row = epi_row(p, m);
        const int32_t v = epi_int(p, row, sum, n);
        if (p.kind == OMCUDA_EPI_I32) {
          reinterpret_cast<int32_t *>(p.Y)[m * p.N + n] = v;
        } else if (p.kind == OMCUDA_EPI_DEQUANT) {
          float y = epi_dequant(p, sc, v, n);
          if (p.residual)
            y = __fadd_rn(y, __ldg(p.residual + m * p.N + n));
          reinterpret_cast<float *>(p.Y)[m * p.N + n] = y;
          lo = fminf(lo, y);
          hi = fmaxf(hi, y);
        } else {
          reinterpret_cast<uint8_t *>(p.Y)[m * p.N + n] = (uint8_t)epi_requant(p, sc, v, n);
        }
      }
    }
    __syncthreads(); // part[] is rewritten by the next group
  }
  if (warp == 0 && p.out_range && p.kind == OMCUDA_EPI_DEQUANT)
    epi_range_commit(p.out_range, lo, hi);
}

// ---- GEMV-shaped GEMM for 2..16 rows on mma.sync ---------------------------------
//
// With more than one row the dp4a work per weight byte of the kernel above
// starts to outgrow the weight read.  This kernel keeps the same shape (a pass over the weight,
// HBM bound) and hands the arithmetic to mma.sync.m16n8k32: the 16 rows of
// the A fragment are the (up to) 16 rows of the problem, the 8 columns of the
// B fragment are 8 adjacent output columns, and a warp consumes the weight in
// 64-byte blocks of K: lane (g, q) (g = lane / 4 the column, q = lane % 4)
// loads the 16 bytes at offset 16 q of column g's block straight from global
// memory into its B registers.  The instruction's own K order is different
// (lane q holds K bytes 4q..4q+3 and 16+4q..16+4q+3), but a sum over K does not
// care in which order the bytes are paired as long as A and B agree, so A is
// loaded with the same permutation (the 16 bytes at offset 16 q of rows g and
// g + 8) and one 16-byte load feeds two MMAs.  The kGemvMmaWarps warps of a
// block split K between them and fold their fragments through shared memory;
// all threads then run the epilogue, consecutive threads on consecutive
// columns.  Integer sums are exact in any order: bit-identical to the other
// kernels.
constexpr int kGemvMmaWarps = 8;
constexpr int kGemvMmaUnroll = 4; // 64-byte blocks of K in flight per warp

template <bool kASigned, bool kBSigned>
__device__ __forceinline__ void mma_m16n8k32(int32_t (&c)[4], uint32_t a0,
    uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if (kASigned && kBSigned)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else if (kASigned && !kBSigned)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else if (!kASigned && kBSigned)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int CG, bool kASigned, bool kBSigned>
__global__ void __launch_bounds__(32 * kGemvMmaWarps)
    gemm_i8_gemv_mma_kernel(const uint8_t *__restrict__ A,
        const uint8_t *__restrict__ Bt, int64_t kp, EpiParams p) {
  constexpr int kCols = 8 * CG;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int64_t m0 = (int64_t)blockIdx.y * 16;
  const bool vec_ok = ((p.K & 15) == 0) && (((uintptr_t)A & 15u) == 0);
  const int64_t blocks64 = (kp + 63) >> 6;
  __shared__ int32_t part[kGemvMmaWarps][16][kCols + 1];
  const EpiScalars sc = epi_scalars(p);
  float lo = INFINITY, hi = -INFINITY;
  const int64_t groups = ceil_div(p.N, kCols);
  for (int64_t grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const int64_t n0 = grp * kCols;
    int32_t acc[CG][4];
#pragma unroll
    for (int j = 0; j < CG; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        acc[j][i] = 0;
    const uint8_t *brow[CG];
#pragma unroll
    for (int j = 0; j < CG; ++j) { // columns past N re-read the last one; never stored
      const int64_t n = n0 + 8 * j + g;
      brow[j] = Bt + (n < p.N ? n : p.N - 1) * kp + 16 * q;
    }
    // Warp w takes runs of kGemvMmaUnroll adjacent blocks (256 bytes of every
    // column), run r = w, w + kGemvMmaWarps, ...
    for (int64_t b0 = (int64_t)warp * kGemvMmaUnroll; b0 < blocks64;
         b0 += (int64_t)kGemvMmaWarps * kGemvMmaUnroll) {
      uint4 bw[kGemvMmaUnroll][CG];
#pragma unroll
      for (int u = 0; u < kGemvMmaUnroll; ++u) {
        const int64_t koff = ((b0 + u) << 6) + 16 * q;
#pragma unroll
        for (int j = 0; j < CG; ++j)
          bw[u][j] = koff < kp
                         ? __ldcs(reinterpret_cast<const uint4 *>(brow[j] + ((b0 + u) << 6)))
                         : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < kGemvMmaUnroll; ++u) {
        const int64_t koff = ((b0 + u) << 6) + 16 * q;
        const uint4 a_lo = load_a_chunk(A, m0 + g, p.M, p.K, koff, vec_ok);
        const uint4 a_hi = load_a_chunk(A, m0 + g + 8, p.M, p.K, koff, vec_ok);
#pragma unroll
        for (int j = 0; j < CG; ++j) {
          mma_m16n8k32<kASigned, kBSigned>(
              acc[j], a_lo.x, a_hi.x, a_lo.y, a_hi.y, bw[u][j].x, bw[u][j].y);
          mma_m16n8k32<kASigned, kBSigned>(
              acc[j], a_lo.z, a_hi.z, a_lo.w, a_hi.w, bw[u][j].z, bw[u][j].w);
        }
      }
    }
    // Accumulator fragment: c0,c1 = row g, columns 2q, 2q+1; c2,c3 = row g + 8.
#pragma unroll
    for (int j = 0; j < CG; ++j) {
      part[warp][g][8 * j + 2 * q] = acc[j][0];
      part[warp][g][8 * j + 2 * q + 1] = acc[j][1];
      part[warp][g + 8][8 * j + 2 * q] = acc[j][2];
      part[warp][g + 8][8 * j + 2 * q + 1] = acc[j][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * kCols; idx += 32 * kGemvMmaWarps) {
      const int r = idx / kCols, cidx = idx % kCols;
      const int64_t m = m0 + r, n = n0 + cidx;
      if (m < p.M && n < p.N) {
        int32_t sum = 0;
#pragma unroll
        for (int w = 0; w < kGemvMmaWarps; ++w)
          sum += part[w][r][cidx];
        const EpiRow row = epi_row(p, m);
        const int32_t v = epi_int(p, row, sum, n);
        if (p.kind == OMCUDA_EPI_I32) {
          reinterpret_cast<int32_t *>(p.Y)[m * p.N + n] = v;
        } else if (p.kind == OMCUDA_EPI_DEQUANT) {
          float y = epi_dequant(p, sc, v, n);
          if (p.residual)
            y = __fadd_rn(y, __ldg(p.residual + m * p.N + n));
          reinterpret_cast<float *>(p.Y)[m * p.N + n] = y;
          lo = fminf(lo, y);
          hi = fmaxf(hi, y);
        } else {
          reinterpret_cast<uint8_t *>(p.Y)[m * p.N + n] = (uint8_t)epi_requant(p, sc, v, n);
        }
      }
    }
    __syncthreads(); // part[] is rewritten by the next group
  }
  if (p.out_range && p.kind == OMCUDA_EPI_DEQUANT)
    epi_range_commit(p.out_range, lo, hi);
}

EpiParams make_epi_params(const omcudaGemmArgs &a) {
  EpiParams p;
  p.M = a.M;
  p.N = a.N;
  p.K = a.K;
  p.a_zp = a.a_zp;
  p.a_zp_len = a.a_zp ? (int)(a.a_zp_len > 1 ? 2 : a.a_zp_len) : 0;
  p.a_signed = a.a_signed;
  p.b_zp = a.b_zp;
  p.b_zp_len = a.b_zp ? (int)(a.b_zp_len > 1 ? 2 : a.b_zp_len) : 0;
  p.b_signed = a.B.b_signed;
  p.colsum = a.B.colsum;
  p.rowsum = a.a_rowsum;
  p.kind = a.epilogue;
  p.Y = a.Y;
  p.sa = a.sa;
  p.sb = a.sb;
  p.sb_len = a.sb_len > 1 ? 2 : (int)a.sb_len;
  p.form = a.scale_form;
  p.bias = a.bias;
  p.gelu = a.gelu;
  p.y_zp = a.y_zp;
  p.residual = (a.epilogue == OMCUDA_EPI_DEQUANT) ? a.residual : nullptr;
  p.res_vec_ok = ((((uintptr_t)a.residual) & 15u) == 0) && (a.N % 4 == 0);
  p.out_range = reinterpret_cast<uint32_t *>(a.out_minmax);
  p.q_range = reinterpret_cast<const uint32_t *>(a.q_range);
  p.q_params = a.q_params;
  p.q_scale = a.q_scale;
  p.q_zp = a.q_zp;
  // (a scalar scale is read with a scalar load wherever it lies)
  const uintptr_t sb_vec = a.sb_len > 1 ? (uintptr_t)a.sb : 0;
  p.vec_ok = ((((uintptr_t)a.B.colsum | (uintptr_t)a.bias | sb_vec) & 15u) == 0) &&
             (a.N % 4 == 0);
  p.line_store = 0;
  p.l2_hints = 0;
  p.quant_mode = quant_mode();
  p.split_k = 1;
  p.ws_rows = 0;
  return p;
}

template <int MT>
static void launch_warp_gemm(const omcudaGemmArgs &a, cudaStream_t st) {
  EpiParams p = make_epi_params(a);
  dim3 grid((unsigned)ceil_div(a.N, 8), (unsigned)ceil_div(a.M, MT));
  const uint8_t *A = (const uint8_t *)a.A;
  const uint8_t *Bt = (const uint8_t *)a.B.bt;
  int sel = (a.a_signed ? 2 : 0) | (a.B.b_signed ? 1 : 0);
  switch (sel) {
  case 0:
    gemm_i8_warp_kernel<MT, false, false><<<grid, 256, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  case 1:
    gemm_i8_warp_kernel<MT, false, true><<<grid, 256, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  case 2:
    gemm_i8_warp_kernel<MT, true, false><<<grid, 256, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  default:
    gemm_i8_warp_kernel<MT, true, true><<<grid, 256, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  }
}

template <int MT, int CB>
static void launch_gemv(const omcudaGemmArgs &a, cudaStream_t st) {
  EpiParams p = make_epi_params(a);
  // Up to 12 resident blocks of 128 threads per SM (1536 threads, 8 x 16-byte
  // loads in flight each with CB = 4).
  const int64_t groups = ceil_div(a.N, CB), resident = (int64_t)sm_count() * 12;
  dim3 grid((unsigned)(groups < resident ? groups : resident), (unsigned)ceil_div(a.M, MT));
  const uint8_t *A = (const uint8_t *)a.A;
  const uint8_t *Bt = (const uint8_t *)a.B.bt;
  const int threads = 32 * kGemvWarps;
  int sel = (a.a_signed ? 2 : 0) | (a.B.b_signed ? 1 : 0);
  switch (sel) {
  case 0:
    gemm_i8_gemv_kernel<MT, CB, false, false><<<grid, threads, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  case 1:
    gemm_i8_gemv_kernel<MT, CB, false, true><<<grid, threads, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  case 2:
    gemm_i8_gemv_kernel<MT, CB, true, false><<<grid, threads, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  default:
    gemm_i8_gemv_kernel<MT, CB, true, true><<<grid, threads, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  }
}

template <int CG>
static void launch_gemv_mma(const omcudaGemmArgs &a, cudaStream_t st) {
  EpiParams p = make_epi_params(a);
  // One block per 8 * CG columns (it reads 8 * CG * K bytes of the weight); very
  // wide weights wrap around a grid of 16 blocks per SM.
  const int64_t groups = ceil_div(a.N, 8 * CG), cap = (int64_t)sm_count() * 16;
  dim3 grid((unsigned)(groups < cap ? groups : cap), (unsigned)ceil_div(a.M, 16));
  const uint8_t *A = (const uint8_t *)a.A;
  const uint8_t *Bt = (const uint8_t *)a.B.bt;
  const int threads = 32 * kGemvMmaWarps;
  int sel = (a.a_signed ? 2 : 0) | (a.B.b_signed ? 1 : 0);
  switch (sel) {
  case 0:
    gemm_i8_gemv_mma_kernel<CG, false, false><<<grid, threads, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  case 1:
    gemm_i8_gemv_mma_kernel<CG, false, true><<<grid, threads, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  case 2:
    gemm_i8_gemv_mma_kernel<CG, true, false><<<grid, threads, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  default:
    gemm_i8_gemv_mma_kernel<CG, true, true><<<grid, threads, 0, st>>>(A, Bt, a.B.kp, p);
    break;
  }
}

// OMCUDA_GEMV=0 keeps the older warp-per-column kernel for every M, for
// experiments.
static bool gemv_wanted() {
  static const bool on = [] {
    const char *s = getenv("OMCUDA_GEMV");
    return !(s && atoi(s) == 0);
  }();
  return on;
}

// Largest M the mma.sync GEMV takes (row groups of 16 re-read the weight
// through L2).  OMCUDA_GEMV_MMA_MAX_M overrides it; 0 switches the kernel off.
static int64_t gemv_mma_max_m() {
  static const int64_t v = [] {
    const char *s = getenv("OMCUDA_GEMV_MMA_MAX_M");
    return s ? (int64_t)atoll(s) : (int64_t)16;
  }();
  return v;
}

static int64_t gemv_max_m() {
  if (!gemv_wanted())
    return 0;
  return gemv_mma_max_m() > 4 ? gemv_mma_max_m() : 4;
}

int launch_gemm_simt(const omcudaGemmArgs &a, cudaStream_t st) {
  // The GEMV-shaped kernels: dp4a up to 4 rows, mma.sync above (with more
  // rows the dp4a work per weight byte outgrows the weight read).
  // (OMCUDA_GEMV_MMA_MIN_M moves the hand-over from the dp4a kernel, for
  // experiments: measured on 4096 x 14336 the dp4a kernel reads one row's
  // weight in 19 us and four rows' in 29 us, the mma.sync kernel 22 and 24 us.)
  static const int64_t mma_min_m = [] {
    const char *s = getenv("OMCUDA_GEMV_MMA_MIN_M");
    return s ? (int64_t)atoll(s) : (int64_t)2;
  }();
  if (a.M >= mma_min_m && a.M <= gemv_mma_max_m() && gemv_wanted()) {
    launch_gemv_mma<2>(a, st);
    OMCUDA_CHECK_LAUNCH("gemm_i8_gemv_mma_kernel");
    return OMCUDA_OK;
  }
  if (a.M <= 16 && gemv_wanted()) {
    if (a.M <= 1)
      launch_gemv<1, 4>(a, st);
    else if (a.M <= 2)
      launch_gemv<2, 4>(a, st);
    else if (a.M <= 4)
      launch_gemv<4, 4>(a, st);
    else
      launch_gemv<8, 4>(a, st); // 9..16 rows: two row groups share the weight through L2
    OMCUDA_CHECK_LAUNCH("gemm_i8_gemv_kernel");
    return OMCUDA_OK;
  }
  if (a.M <= 1)
    launch_warp_gemm<1>(a, st);
  else if (a.M <= 4)
    launch_warp_gemm<4>(a, st);
  else if (a.M <= 8)
    launch_warp_gemm<8>(a, st);
  else
    launch_warp_gemm<16>(a, st);
  OMCUDA_CHECK_LAUNCH("gemm_i8_warp_kernel");
  return OMCUDA_OK;
}

} // namespace omcuda

using namespace omcuda;

extern "C" int64_t omcudaDevPreparedBBytes(int64_t K, int64_t N, int64_t *kp) {
  int64_t k16 = (K + 15) & ~int64_t(15);
  if (kp)
    *kp = k16;
  return N * k16;
}

extern "C" int omcudaDevPrepareB(const void *B, int b_signed, int64_t K,
    int64_t N, omcudaPreparedB *out, void *stream) {
  if (!B || !out || !out->bt || !out->colsum || K <= 0 || N <= 0)
    return fail(OMCUDA_EINVAL, "PrepareB: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  int64_t kp;
  omcudaDevPreparedBBytes(K, N, &kp);
  out->K = K;
  out->N = N;
  out->kp = kp;
  out->b_signed = b_signed;
  dim3 tgrid((unsigned)ceil_div(N, 64), (unsigned)ceil_div(kp, 64));
  transpose_b_kernel<<<tgrid, 256, 0, st>>>(
      (const uint8_t *)B, K, N, kp, (uint8_t *)out->bt);
  OMCUDA_CHECK_LAUNCH("transpose_b_kernel");
  dim3 cblock(64, 4);
  unsigned cgrid = (unsigned)ceil_div(N, 64);
  if (b_signed)
    colsum_kernel<true><<<cgrid, cblock, 0, st>>>(
        (const uint8_t *)B, K, N, out->colsum);
  else
    colsum_kernel<false><<<cgrid, cblock, 0, st>>>(
        (const uint8_t *)B, K, N, out->colsum);
  OMCUDA_CHECK_LAUNCH("colsum_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevRowSum(const void *A, int a_signed, int64_t M,
    int64_t K, int32_t *rowsum, void *stream) {
  if (!A || !rowsum || M <= 0 || K <= 0)
    return fail(OMCUDA_EINVAL, "RowSum: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  unsigned grid = (unsigned)ceil_div(M, 8);
  if (a_signed)
    rowsum_kernel<true><<<grid, 256, 0, st>>>((const uint8_t *)A, M, K, rowsum);
  else
    rowsum_kernel<false><<<grid, 256, 0, st>>>((const uint8_t *)A, M, K, rowsum);
  OMCUDA_CHECK_LAUNCH("rowsum_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevRequantScale(const float *a_scale, const float *b_scale,
    int64_t len, const float *y_scale, float *S, void *stream) {
  if (!a_scale || !b_scale || !y_scale || !S || len <= 0)
    return fail(OMCUDA_EINVAL, "RequantScale: bad argument");
  requant_scale_kernel<<<(unsigned)ceil_div(len, 256), 256, 0,
      (cudaStream_t)stream>>>(a_scale, b_scale, len, y_scale, S);
  OMCUDA_CHECK_LAUNCH("requant_scale_kernel");
  return OMCUDA_OK;
}

extern "C" int omcudaDevGemmI8(const omcudaGemmArgs *args, void *stream) {
  if (!args)
    return fail(OMCUDA_EINVAL, "GemmI8: null args");
  const omcudaGemmArgs &a = *args;
  if (a.M < 0 || a.N <= 0 || a.K <= 0 || !a.A || !a.B.bt ||
      (!a.Y && a.epilogue != OMCUDA_EPI_DEQUANT_RANGE))
    return fail(OMCUDA_EINVAL, "GemmI8: bad shape or null operand");
  if (a.M == 0)
    return OMCUDA_OK;
  if (a.B.K != a.K || a.B.N != a.N)
    return fail(OMCUDA_EINVAL, "GemmI8: prepared B does not match K,N");
  if (a.a_zp && a.a_zp_len != 1 && a.a_zp_len != a.M)
    return fail(OMCUDA_EINVAL, "GemmI8: a_zp length must be 1 or M");
  if (a.b_zp && a.b_zp_len != 1 && a.b_zp_len != a.N)
    return fail(OMCUDA_EINVAL, "GemmI8: b_zp length must be 1 or N");
  if (a.b_zp && a.b_zp_len != 0 && !a.a_rowsum)
    return fail(OMCUDA_EINVAL, "GemmI8: b_zp needs the row sums of A");
  if (a.a_zp && a.a_zp_len != 0 && !a.B.colsum)
    return fail(OMCUDA_EINVAL, "GemmI8: a_zp needs the column sums of B");
  if (a.residual && a.epilogue != OMCUDA_EPI_DEQUANT)
    return fail(OMCUDA_EINVAL, "GemmI8: a residual goes with the dequant epilogue only");
  if (a.epilogue < OMCUDA_EPI_I32 || a.epilogue > OMCUDA_EPI_DEQUANT_QUANT)
    return fail(OMCUDA_EINVAL, "GemmI8: unknown epilogue %d", a.epilogue);
  if (epi_is_dequant(a.epilogue) && (!a.sa || !a.sb))
    return fail(OMCUDA_EINVAL, "GemmI8: dequant epilogue needs both scales");
  if (a.epilogue == OMCUDA_EPI_DEQUANT_RANGE && !a.out_minmax)
    return fail(OMCUDA_EINVAL, "GemmI8: the range-only tail needs out_minmax");
  if (a.epilogue == OMCUDA_EPI_DEQUANT_QUANT && (!a.q_range || !a.q_params))
    return fail(OMCUDA_EINVAL, "GemmI8: the quantizing tail needs q_range and q_params");
  if (a.epilogue == OMCUDA_EPI_REQUANT && !a.sb)
    return fail(OMCUDA_EINVAL, "GemmI8: requant epilogue needs S");
  if (a.epilogue != OMCUDA_EPI_I32 && a.sb_len != 1 && a.sb_len != a.N)
    return fail(OMCUDA_EINVAL, "GemmI8: scale length must be 1 or N");
  cudaStream_t st = (cudaStream_t)stream;
  bool tc_ok = gemm_tc_supported(a);
  if (a.kernel_choice == 1 && !tc_ok)
    return fail(OMCUDA_ENOTSUP,
        "GemmI8: tensor-core kernel needs K %% 16 == 0 and 16-byte aligned A");
  const bool tc_only = a.epilogue == OMCUDA_EPI_DEQUANT_SPLIT ||
                       a.epilogue == OMCUDA_EPI_DEQUANT_RANGE ||
                       a.epilogue == OMCUDA_EPI_DEQUANT_QUANT;
  if (tc_only && (!tc_ok || a.kernel_choice == 2))
    return fail(OMCUDA_ENOTSUP,
        "GemmI8: the split-bf16, range-only and quantizing tails exist on the "
        "tensor-core kernel only (K %% 16 == 0, 16-byte aligned A)");
  // With a handful of rows the GEMM is one read of the weight, which the
  // GEMV-shaped kernels stream faster than 128-row tensor-core tiles on a few
  // SMs (measured: M = 1 19 us against 23-27 us on the 58 MB weights).
  bool use_tc = (a.kernel_choice == 1) || tc_only ||
                (a.kernel_choice == 0 && tc_ok && a.M > gemv_max_m());
  return use_tc ? launch_gemm_tc(a, st) : launch_gemm_simt(a, st);
}
