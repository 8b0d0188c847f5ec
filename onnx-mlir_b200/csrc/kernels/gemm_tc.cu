// int8 x int8 -> int32 GEMM on Blackwell tensor cores (tcgen05.mma kind::i8)
// with the zero-point / dequantize / requantize epilogues of
// gemm_epilogue.cuh.  It computes what onnx-mlir's MatMulInteger and
// QLinearMatMul lowerings compute with CPU loops
// (src/Conversion/ONNXToKrnl/Math/MatMulInteger.cpp:59-90,
//  src/Conversion/ONNXToKrnl/Math/QLinearMatMul.cpp:89-138,
//  src/Conversion/ONNXToKrnl/Math/MatMul.cpp:278-327).
//
// Data layout in HBM: A is [M,K] row-major 8-bit (K-major, as ONNX gives it);
// B is the prepared K-major copy Bt[N][kp] (gemm_simt.cu); Y is [M,N]
// row-major i32 / f32 / 8-bit.
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Warp roles:
//   warp 0     TMA producer: cp.async.bulk.tensor loads of a 128x128-byte A
//              tile and a BNx128-byte Bt tile per pipeline stage, 128-byte
//              swizzle, completion on an mbarrier.  Plain (non-multicast)
//              loads only.
//   warp 1     allocates tensor memory; its lane 0 issues tcgen05.mma
//              (M=128, N=BN, K=32 per instruction, four per stage) into one of
//              two TMEM accumulator buffers and commits to mbarriers to free
//              the smem stage / publish the accumulator.
//   warps 2-9  epilogue: tcgen05.ld the accumulator (a warp may read the 32
//              TMEM lanes its id modulo 4 selects; the two warps of a lane
//              quadrant split the tile's columns), apply the epilogue, stage
//              the results in shared memory and store whole 128-byte lines.
// The two accumulator buffers let the epilogue of tile i overlap the MMAs of
// tile i+1.
//
// Every wait on an mbarrier is bounded: after wait_ns (two seconds unless
// omcudaDevSetWaitLimitNs changed it) without progress of that one wait, the
// waiting thread raises a CTA-wide abort flag, the kernel writes a non-zero
// word to *status, releases its tensor memory and returns.
#include <cuda.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../runtime/internal.h"
#include "gemm_epilogue.cuh"
#include "quantize.cuh"
#include "tc_ptx.cuh"

namespace omcuda {

namespace {

constexpr int kBM = 128;       // rows of A per tile
constexpr int kBK = 128;       // bytes (= int8 elements) of K per stage
constexpr int kUmmaK = 32;     // K of one tcgen05.mma kind::i8
// The kernels are built with 8 or 16 epilogue warps (EW).  Sixteen hide the
// epilogue's latency better, which decides shapes with a short K loop; eight
// leave shared memory for a deeper operand pipeline, which decides long K.
// Columns of a tile that one epilogue warp drains: the EW/4 warps that may
// read a TMEM lane quadrant split the tile's columns, 32 columns at least.
__host__ __device__ constexpr int epi_cols_per_warp(int bn, int ew) {
  return bn / (ew / 4) >= 32 ? bn / (ew / 4) : 32;
}
__host__ __device__ constexpr int epi_active_warps(int bn, int ew) {
  return 4 * (bn / epi_cols_per_warp(bn, ew));
}
__host__ __device__ constexpr int tc_threads(int ew) { return 32 * (2 + ew); }
constexpr int kSmemBudget = 232448 - 1024 - 512; // per CTA, minus slack and barriers
__host__ __device__ constexpr int tc_stages(int stage_bytes, int ew) {
  return (kSmemBudget - ew * 4096) / stage_bytes < 8
             ? (kSmemBudget - ew * 4096) / stage_bytes
             : 8;
}

template <int BN, int EW>
struct TcConfig {
  static constexpr int kABytes = kBM * kBK;
  static constexpr int kBBytes = BN * kBK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = tc_stages(kStageBytes, EW);
  static constexpr int kTmemCols = 2 * BN; // two accumulator buffers
  // Output staging: per epilogue warp one slab of 32 rows x 128 bytes.
  static constexpr int kSlabBytes = 32 * 128;
  static constexpr int kStagingBytes = EW * kSlabBytes;
  static constexpr int kSmemBytes =
      kStages * kStageBytes + kStagingBytes + 1024; // + alignment slack
};

// ---- shared-memory staging helper ------------------------------------------------

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a,
    uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a),
               "r"(b), "r"(c), "r"(d)
               : "memory");
}

// ---- epilogue arithmetic on one 32-column chunk ---------------------------------------

// Loads 32 consecutive per-column values with 16-byte loads when allowed.
template <typename T>
__device__ __forceinline__ void load_cols32(
    const T *base, int64_t n, int valid, bool vec_ok, T (&out)[32]) {
  if (vec_ok && valid == 32) {
    const uint4 *p4 = reinterpret_cast<const uint4 *>(base + n);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4 q = __ldg(p4 + j);
      out[4 * j + 0] = *reinterpret_cast<T *>(&q.x);
      out[4 * j + 1] = *reinterpret_cast<T *>(&q.y);
      out[4 * j + 2] = *reinterpret_cast<T *>(&q.z);
      out[4 * j + 3] = *reinterpret_cast<T *>(&q.w);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      out[j] = (j < valid) ? __ldg(base + n + j) : T(0);
  }
}

// Turns 32 raw accumulators of one row into 32 output words (EPI_I32: the
// corrected i32; EPI_DEQUANT, EPI_DEQUANT_SPLIT and EPI_DEQUANT_RANGE: f32
// bits; EPI_REQUANT: one byte per word; EPI_DEQUANT_QUANT: words 0..7 hold
// the 32 output bytes, four to a word).
template <int EPI>
__device__ __forceinline__ void epilogue_chunk(const EpiParams &p,
    const EpiScalars &sc, const QuantConsts &qc, const EpiRow &row,
    const float *res_row, int64_t nc, int valid, uint32_t (&v)[32], float &lo,
    float &hi) {
  const bool vec = p.vec_ok != 0;
  if (p.b_zp_len != 0) {
    // - bz[n] * rowsum[m] + K * az * bz[n]  =  bz[n] * (K * az - rowsum[m])
    const uint32_t tr = (uint32_t)p.K * (uint32_t)row.az - (uint32_t)row.rs;
    if (p.b_zp_len == 1) {
      const uint32_t bz = (uint32_t)load_zp8(p.b_zp, 0, p.b_signed);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        v[j] += bz * tr;
    } else if (vec && valid == 32 && (((uintptr_t)p.b_zp + (uintptr_t)nc) & 15u) == 0) {
      const uint4 *src = reinterpret_cast<const uint4 *>(
          reinterpret_cast<const uint8_t *>(p.b_zp) + nc);
      const uint4 q0 = __ldg(src), q1 = __ldg(src + 1);
      const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const uint32_t byte = (w[j >> 2] >> (8 * (j & 3))) & 0xffu;
        const uint32_t bz = p.b_signed ? (uint32_t)(int32_t)(int8_t)byte : byte;
        v[j] += bz * tr;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < valid)
          v[j] += (uint32_t)load_zp8(p.b_zp, nc + j, p.b_signed) * tr;
    }
  }
  if (p.a_zp_len != 0) {
    int32_t cs[32];
    load_cols32(p.colsum, nc, valid, vec, cs);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      v[j] -= (uint32_t)row.az * (uint32_t)cs[j];
  }
  if (EPI == OMCUDA_EPI_I32)
    return;
  if (epi_is_dequant(EPI)) {
    float f[32];
#pragma unroll
    for (int j = 0; j < 32; ++j)
      f[j] = __int2float_rn((int32_t)v[j]);
    if (p.sb_len == 1) {
      if (p.form == 0) {
        // (packed fp32: two exactly rounded products per instruction)
        const uint64_t s2 = pack_f32x2(sc.s0, sc.s0);
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          unpack_f32x2(mul_f32x2(pack_f32x2(f[j], f[j + 1]), s2), f[j], f[j + 1]);
      } else {
        const float sb = __ldg(p.sb);
#pragma unroll
        for (int j = 0; j < 32; ++j)
          f[j] = __fmul_rn(__fmul_rn(f[j], sc.sa), sb);
      }
    } else {
      float sb[32];
      load_cols32(p.sb, nc, valid, vec, sb);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        f[j] = (p.form == 0) ? __fmul_rn(f[j], __fmul_rn(sc.sa, sb[j]))
                             : __fmul_rn(__fmul_rn(f[j], sc.sa), sb[j]);
    }
    if (p.bias) {
      float b[32];
      load_cols32(p.bias, nc, valid, vec, b);
#pragma unroll
      for (int j = 0; j < 32; j += 2)
        unpack_f32x2(add_f32x2(pack_f32x2(f[j], f[j + 1]), pack_f32x2(b[j], b[j + 1])),
            f[j], f[j + 1]);
    }
    if (p.gelu) {
#pragma unroll
      for (int j = 0; j < 32; j += 2)
        gelu_erf_x2(f[j], f[j + 1]);
    }
    if (EPI == OMCUDA_EPI_DEQUANT && res_row) {
      float r[32];
      load_cols32(res_row, nc, valid, p.res_vec_ok != 0, r);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        f[j] = __fadd_rn(f[j], r[j]);
    }
    if (p.out_range) {
      if (valid == 32) {
        // three-input min / max: one instruction per two values
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          lo = min3f(lo, f[j], f[j + 1]);
          hi = max3f(hi, f[j], f[j + 1]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < valid) {
            lo = fminf(lo, f[j]);
            hi = fmaxf(hi, f[j]);
          }
      }
    }
    if (EPI == OMCUDA_EPI_DEQUANT_QUANT) {
      // DynamicQuantizeLinear's quantize step on the values just computed.
#pragma unroll
      for (int j = 0; j < 8; ++j)
        v[j] = quantize_four<false>(
            make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]), qc);
      return;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j)
      v[j] = __float_as_uint(f[j]);
    return;
  }
  // EPI_REQUANT
  if (p.sb_len == 1) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float r = round_even(__fmul_rn(__int2float_rn((int32_t)v[j]), sc.s0));
      v[j] = ((uint32_t)__float2int_rz(r) + (uint32_t)p.y_zp) & 0xffu;
    }
  } else {
    float S[32];
    load_cols32(p.sb, nc, valid, vec, S);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float r = round_even(__fmul_rn(__int2float_rn((int32_t)v[j]), S[j]));
      v[j] = ((uint32_t)__float2int_rz(r) + (uint32_t)p.y_zp) & 0xffu;
    }
  }
}

// 32 f32 words -> words 0..15: bf16 hi of the pairs (v0,v1), (v2,v3), ...;
// words 16..31: bf16 lo, with hi = bf16(x), lo = bf16(x - hi), round to
// nearest even (the operand format of the tcgen05 attention kernel).
__device__ __forceinline__ void split_words_bf16(uint32_t (&v)[32]) {
  uint32_t h[16], l[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float a = __uint_as_float(v[2 * i]), b = __uint_as_float(v[2 * i + 1]);
    uint32_t hw;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hw) : "f"(b), "f"(a));
    // x - hi for both values in one packed instruction (hi * -1 + x: one
    // rounding, the subtraction's)
    float ra, rb;
    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(hw << 16),
                               __uint_as_float(hw & 0xffff0000u)),
                     pack_f32x2(-1.0f, -1.0f), pack_f32x2(a, b)),
        ra, rb);
    uint32_t lw;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lw) : "f"(rb), "f"(ra));
    h[i] = hw;
    l[i] = lw;
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = h[i];
    v[16 + i] = l[i];
  }
}

// EPI_DEQUANT_QUANT: scale and zero point as DynamicQuantizeLinear derives
// them from the range a range-only pass of the same product left behind.
// Every thread computes the same two scalars; one thread of the grid also
// publishes them for the operators that follow.
template <int EPI>
__device__ __forceinline__ QuantConsts epi_quant_consts(const EpiParams &p, bool publish) {
  if (EPI != OMCUDA_EPI_DEQUANT_QUANT)
    return QuantConsts{1.0f, 1.0f, 0.0f, true};
  float scale, zp_f;
  dql_params_from_range(ordered_to_f32(__ldg(p.q_range)),
      ordered_to_f32(__ldg(p.q_range + 1)), &scale, &zp_f, p.quant_mode);
  if (publish) {
    p.q_params[0] = scale;
    p.q_params[1] = zp_f;
    if (p.q_scale)
      *p.q_scale = scale;
    if (p.q_zp)
      *p.q_zp = (uint8_t)(unsigned int)zp_f; // fptoui; zp_f is in [0,255]
  }
  return make_quant_consts(scale, zp_f, p.quant_mode);
}

// Drains one accumulator tile half (this warp's 32 TMEM lanes x kHalfCols
// columns starting at taddr) through the epilogue into Y.
//   m_warp   first output row of this warp's 32 rows
//   n0       first output column of this warp's column range
//   slab0    this warp's 4 KiB staging slab in shared memory
//   release  called once, right after the last tensor-memory load of the
//            tile: the accumulator buffer is handed back to the MMA issuer
//            before the arithmetic and the stores of the last chunk, which
//            keeps those off the path that decides when the next tile's MMAs
//            may start
template <int BN, int EPI, int EW, typename Release>
__device__ __forceinline__ void epilogue_tile(const EpiParams &p,
    const EpiScalars &sc, const QuantConsts &qc, uint32_t taddr, int64_t m_warp,
    int64_t n0, uint32_t slab0, int lane, bool use_slab, float &lo, float &hi,
    const CUtensorMap *map_y, const CUtensorMap *map_y2, Release &&release,
    int32_t store_row_off = 0) {
  const bool hint_store = (p.l2_hints & 1) != 0;
  const uint64_t pol_out = hint_store ? l2_policy_evict_first() : 0;
  // EPI_DEQUANT_SPLIT stages like the 4-byte tails (32 columns per 128-byte
  // slab row: 16 words of bf16 hi pairs, then 16 words of lo pairs).
  constexpr bool kSplit = EPI == OMCUDA_EPI_DEQUANT_SPLIT;
  // EPI_DEQUANT_RANGE walks the tile like the f32 tail and stores nothing.
  constexpr bool kNoStore = EPI == OMCUDA_EPI_DEQUANT_RANGE;
  constexpr bool kPacked = EPI == OMCUDA_EPI_DEQUANT_QUANT; // bytes arrive four to a word
  constexpr int kOutBytes =
      (EPI == OMCUDA_EPI_REQUANT || EPI == OMCUDA_EPI_DEQUANT_QUANT) ? 1 : 4;
  constexpr int kHalfCols = epi_cols_per_warp(BN, EW);
  constexpr int kSlabCols =
      (128 / kOutBytes) < kHalfCols ? (128 / kOutBytes) : kHalfCols;
  constexpr int kSlabsPerHalf = kHalfCols / kSlabCols;
  static_assert(kHalfCols % 32 == 0 && kHalfCols % kSlabCols == 0, "tile shape");
  const int64_t m = m_warp + lane;
  const bool y4_ok = ((p.N & 3) == 0) && (((uintptr_t)p.Y & 15u) == 0);
  const bool row_ok = m < p.M;
  EpiRow row;
  row.az = 0;
  row.rs = 0;
  if (row_ok)
    row = epi_row(p, m);
  const float *res_row = (row_ok && p.residual) ? p.residual + m * p.N : nullptr;
  if (use_slab) {
    // Results pass through a shared-memory slab (32 rows per warp, rows of
    // kRowB bytes in the 128-byte-swizzle pattern) and leave with one TMA
    // store per slab, which writes whole lines and clips rows and columns
    // beyond the matrix.  EPI_DEQUANT_SPLIT uses the two halves of the slab
    // for the hi and the lo plane.
    constexpr int kRowB = kSplit ? 64 : kSlabCols * kOutBytes;
    static_assert(kRowB == 32 || kRowB == 64 || kRowB == 128,
        "slab rows span one swizzle width");
    // 16-byte piece index XOR address bits 7.. (3, 2 or 1 bits for the 128-,
    // 64- and 32-byte swizzle), as the store's tensor map expects.
    constexpr uint32_t kSwzMask = (uint32_t)kRowB / 16u - 1u;
    const uint32_t row_off = (uint32_t)lane * kRowB;
    // The XOR term of this thread's row (pieces of a row stay inside it).
    const uint32_t swz = ((row_off >> 7) & kSwzMask) << 4;
    const uint32_t my_row = slab0 + row_off;
    const bool warp_in = m_warp < p.M;
#pragma unroll 1
    for (int g = 0; g < kSlabsPerHalf; ++g) {
      const int64_t ng = n0 + (int64_t)g * kSlabCols;
#pragma unroll 1
      for (int cc = 0; cc < kSlabCols; cc += 32) {
        uint32_t v[32];
        __syncwarp(); // tcgen05.ld is warp-collective: enter it converged
        tmem_ld32(taddr + (uint32_t)(g * kSlabCols + cc), v);
        tmem_ld_wait();
        if (g == kSlabsPerHalf - 1 && cc + 32 >= kSlabCols)
          release();
        const int64_t nc = ng + cc;
        const int valid = (int)((p.N - nc) < 32 ? (p.N - nc) : 32);
        if (row_ok && valid > 0)
          epilogue_chunk<EPI>(p, sc, qc, row, res_row, nc, valid, v, lo, hi);
        if (kNoStore)
          continue;
        if (kSplit)
          split_words_bf16(v);
        if (cc == 0) {
          // The previous store must have read the slab before it is rewritten.
          if (lane == 0)
            tma_store_wait_read();
          __syncwarp();
        }
        if (kSplit) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t so = my_row + (((uint32_t)j * 16u) ^ swz);
            st_shared_v4(so, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            st_shared_v4(so + 2048u, v[16 + 4 * j], v[17 + 4 * j], v[18 + 4 * j],
                v[19 + 4 * j]);
          }
        } else if (kOutBytes == 4) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_shared_v4(my_row + (((uint32_t)j * 16u) ^ swz), v[4 * j], v[4 * j + 1],
                v[4 * j + 2], v[4 * j + 3]);
        } else {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            w[j] = kPacked ? v[j]
                           : (v[4 * j] | (v[4 * j + 1] << 8) | (v[4 * j + 2] << 16) |
                                 (v[4 * j + 3] << 24));
          st_shared_v4(my_row + ((uint32_t)cc ^ swz), w[0], w[1], w[2], w[3]);
          st_shared_v4(my_row + (((uint32_t)cc + 16u) ^ swz), w[4], w[5], w[6], w[7]);
        }
      }
      if (kNoStore)
        continue;
      fence_proxy_async_smem(); // the slab was written through the generic proxy
      __syncwarp();
      if (lane == 0 && warp_in && ng < p.N) {
        if (hint_store) {
          tma_store_2d_hint(map_y, slab0, (int32_t)ng, (int32_t)m_warp + store_row_off, pol_out);
          if (kSplit)
            tma_store_2d_hint(map_y2, slab0 + 2048u, (int32_t)ng, (int32_t)m_warp, pol_out);
        } else {
          tma_store_2d(map_y, slab0, (int32_t)ng, (int32_t)m_warp + store_row_off);
          if (kSplit)
            tma_store_2d(map_y2, slab0 + 2048u, (int32_t)ng, (int32_t)m_warp);
        }
        tma_store_commit();
      }
    }
  } else {
    // Fallback when the row pitch of Y is not a multiple of 16 bytes:
    // direct stores, one row per thread.
#pragma unroll 1
    for (int c = 0; c < kHalfCols; c += 32) {
      uint32_t v[32];
      __syncwarp();
      tmem_ld32(taddr + (uint32_t)c, v);
      tmem_ld_wait();
      if (c + 32 >= kHalfCols)
        release();
      const int64_t nc = n0 + c;
      const int valid = (int)((p.N - nc) < 32 ? (p.N - nc) : 32);
      if (!row_ok || valid <= 0)
        continue;
      epilogue_chunk<EPI>(p, sc, qc, row, res_row, nc, valid, v, lo, hi);
      if (kNoStore)
        continue;
      if (kSplit) {
        split_words_bf16(v);
        uint16_t *dhi = reinterpret_cast<uint16_t *>(p.Y) + m * p.N + nc;
        uint16_t *dlo = dhi + p.M * p.N;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < valid) {
            dhi[j] = (uint16_t)(v[j >> 1] >> (16 * (j & 1)));
            dlo[j] = (uint16_t)(v[16 + (j >> 1)] >> (16 * (j & 1)));
          }
      } else if (kOutBytes == 4) {
        uint32_t *dst = reinterpret_cast<uint32_t *>(p.Y) + m * p.N + nc;
        if (y4_ok && valid == 32) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            reinterpret_cast<uint4 *>(dst)[j] = make_uint4(
                v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < valid)
              dst[j] = v[j];
        }
      } else {
        uint8_t *dst = reinterpret_cast<uint8_t *>(p.Y) + m * p.N + nc;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < valid)
            dst[j] = kPacked ? (uint8_t)(v[j >> 2] >> (8 * (j & 3))) : (uint8_t)v[j];
      }
    }
  }
}

} // namespace

// ---- the kernel -------------------------------------------------------------------

template <int BN, int EPI, int EW>
__global__ void __launch_bounds__(tc_threads(EW), 1)
    gemm_i8_tc_kernel(const __grid_constant__ CUtensorMap map_a,
        const __grid_constant__ CUtensorMap map_b,
        const __grid_constant__ CUtensorMap map_y,
        const __grid_constant__ CUtensorMap map_y2, EpiParams p, uint32_t idesc,
        int *status, uint64_t wait_ns) {
  using Cfg = TcConfig<BN, EW>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kHalfCols = epi_cols_per_warp(BN, EW); // columns per epilogue warp of a lane quadrant

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[kStages];
  __shared__ uint64_t bar_empty[kStages];
  __shared__ uint64_t bar_acc_full[2];
  __shared__ uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // 128-byte-swizzled tiles must start on a 1024-byte boundary.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t staging_base = smem_base + kStages * Cfg::kStageBytes;

  const int64_t tiles_m = ceil_div(p.M, kBM);
  const int64_t tiles_n = ceil_div(p.N, BN);
  const int num_kb = (int)ceil_div(p.K, kBK);
  // Work units: tiles, or (split-K pass) the split_k K slices of every tile,
  // slices of one tile next to each other.
  const int split = p.split_k;
  const int64_t num_units = tiles_m * tiles_n * split;

  if (threadIdx.x == 32) { // (a thread that has nothing else to set up)
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    if (p.line_store) {
      prefetch_tensormap(&map_y);
      if (EPI == OMCUDA_EPI_DEQUANT_SPLIT)
        prefetch_tensormap(&map_y2);
    }
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_acc_full[b]), 1);
      mbar_init(smem_u32(&bar_acc_empty[b]), epi_active_warps(BN, EW)); // one arrive per active epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1)
    tmem_alloc(smem_u32(&tmem_base_slot), Cfg::kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int *abortp = &abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t pol_a = l2_policy_evict_first(), pol_b = l2_policy_evict_last();
      for (int64_t u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int64_t t = split > 1 ? u / split : u;
        const int ks = split > 1 ? (int)(u % split) : 0;
        const int kb0 = (int)((int64_t)ks * num_kb / split);
        const int kb1 = (int)((int64_t)(ks + 1) * num_kb / split);
        const int32_t m0 = (int32_t)((t / tiles_n) * kBM);
        const int32_t n0 = (int32_t)((t % tiles_n) * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp, wait_ns)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[stage]);
          const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sb = sa + Cfg::kABytes;
          mbar_expect_tx(full, Cfg::kStageBytes);
          if (p.l2_hints & 2)
            tma_load_2d_hint(sa, &map_a, kb * kBK, m0, full, pol_a);
          else
            tma_load_2d(sa, &map_a, kb * kBK, m0, full);
          if (p.l2_hints & 4)
            tma_load_2d_hint(sb, &map_b, kb * kBK, n0, full, pol_b);
          else
            tma_load_2d(sb, &map_b, kb * kBK, n0, full);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int64_t it = 0;
      // The issuing thread is a chain of dependent round trips (barrier poll,
      // MMA issue, commit); whether a stage has landed is therefore asked one
      // stage ahead, before the MMAs of the current stage are issued.
      bool landed = false;
      for (int64_t u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++it) {
        const int ks = split > 1 ? (int)(u % split) : 0;
        const int kb0 = (int)((int64_t)ks * num_kb / split);
        const int kb1 = (int)((int64_t)(ks + 1) * num_kb / split);
        const int buf = (int)(it & 1);
        const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
        if (!mbar_wait(smem_u32(&bar_acc_empty[buf]), acc_phase ^ 1u, abortp, wait_ns)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!landed && !mbar_wait(smem_u32(&bar_full[stage]), phase, abortp, wait_ns)) {
            ok = false;
            break;
          }
          const int nstage = stage + 1 == kStages ? 0 : stage + 1;
          const uint32_t nphase = nstage == 0 ? phase ^ 1u : phase;
          landed = mbar_test_wait(smem_u32(&bar_full[nstage]), nphase);
          tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sb = sa + Cfg::kABytes;
          static_assert(kBK / kUmmaK == 4, "four K slices per stage");
          umma_i8_x4(d_tmem, make_smem_desc(sa), make_smem_desc(sb), idesc,
              kb != kb0 ? 1u : 0u);
          umma_commit(smem_u32(&bar_empty[stage]));
          stage = nstage;
          phase = nphase;
        }
        if (ok)
          umma_commit(smem_u32(&bar_acc_full[buf]));
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    const int quad = warp & 3;       // TMEM lanes [32*quad, 32*quad+32)
    const int ew = warp - 2;         // 0..7
    const int c_lo = (ew >> 2) * kHalfCols; // this warp's share of the columns
    const bool active = c_lo < BN;          // narrow tiles leave some warps idle
    const EpiScalars sc = epi_scalars(p);
    const QuantConsts qc = epi_quant_consts<EPI>(p, warp == 2 && lane == 0 && blockIdx.x == 0);
    const bool use_slab = p.line_store != 0;
    const uint32_t slab0 = staging_base + (uint32_t)ew * Cfg::kSlabBytes;
    bool ok = active;
    int64_t it = 0;
    float lo = INFINITY, hi = -INFINITY; // range of this warp's f32 outputs
    for (int64_t u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++it) {
      const int64_t t = split > 1 ? u / split : u;
      const int32_t row_off = split > 1 ? (int32_t)((u % split) * p.ws_rows) : 0;
      const int buf = (int)(it & 1);
      const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
      const int64_t m_warp = (t / tiles_n) * kBM + quad * 32;
      const int64_t n0 = (t % tiles_n) * BN + c_lo;
      // While the MMAs of this tile are still running, pull the per-column
      // vectors this warp will need into L1.
      {
        const int line = lane & 7, which = lane >> 3;
        const int64_t nl = n0 + 32 * line;
        const void *src = nullptr;
        if (32 * line < kHalfCols && nl < p.N) {
          if (which == 0 && p.a_zp_len != 0)
            src = p.colsum + nl;
          else if (which == 1 && p.bias)
            src = p.bias + nl;
          else if (which == 2 && p.sb && p.sb_len != 1)
            src = p.sb + nl;
        }
        if (src)
          asm volatile("prefetch.global.L1 [%0];" ::"l"(src));
        // ... and this warp's block of the residual (32 rows x kHalfCols f32)
        // towards L2: the epilogue reads it one row per thread.
        if (p.residual && m_warp + lane < p.M) {
          const float *rr = p.residual + (m_warp + lane) * p.N + n0;
          for (int c = 0; c < kHalfCols && n0 + c < p.N; c += 32)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(rr + c));
        }
      }
      if (!mbar_wait(smem_u32(&bar_acc_full[buf]), acc_phase, abortp, wait_ns)) {
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const uint32_t taddr =
          tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN + c_lo);
      // The accumulator buffer may be overwritten once every warp has read
      // its share of it.
      epilogue_tile<BN, EPI, EW>(p, sc, qc, taddr, m_warp, n0, slab0, lane, use_slab,
          lo, hi, &map_y, &map_y2, [&] {
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0)
              mbar_arrive(smem_u32(&bar_acc_empty[buf]));
          }, row_off);
    }
    // One commit of the running range per warp, and every store of this warp
    // complete before the CTA may exit.
    if (active && p.out_range && epi_is_dequant(EPI) && EPI != OMCUDA_EPI_DEQUANT_QUANT)
      epi_range_commit(p.out_range, lo, hi);
    if (lane == 0)
      tma_store_wait_all();
  }

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && abort_flag)
    atomicExch(status, 1);
}


// ---- the 2-CTA kernel ----------------------------------------------------------------
//
// Same pipeline on a cluster of two CTAs (two SMs) that share one 256 x 256
// output tile: CTA r owns rows [128 r, 128 r + 128) of it.  Each CTA loads its
// own 128-row A tile but only half of the B tile (128 of the 256 columns);
// tcgen05.mma.cta_group::2 reads both halves.  Per SM that is 32 KiB of
// operands per 128-byte K step instead of 48 KiB, which matters because the
// single-CTA kernel is limited by how fast an SM can take operands in, not by
// the tensor pipe.  Only the leader CTA (rank 0) issues MMAs:
//   full[s]       (leader)  one arrive + 64 KiB of TMA bytes from both CTAs
//   empty[s]      (each)    tcgen05.commit to both CTAs when the MMAs are done
//   acc_full[b]   (each)    tcgen05.commit to both CTAs after the last K step
//   acc_empty[b]  (leader)  16 arrives: the 8 epilogue warps of both CTAs
//
// Work units.  Whole 256 x 256 tiles are dealt round-robin to the clusters.
// When the tiles left over after the last complete round would keep at most
// half of the clusters busy, each of them is cut into two 256 x 128 units
// (tcgen05.mma with N = 128, 64 B columns per CTA), so that the last round
// takes about half as long: units [0, full_units) are whole tiles, the rest
// alternate between the two halves of the remaining tiles.
struct PairUnit {
  int64_t tile;
  int narrow; // 1: a 128-column half tile
  int half;   // which half
};

__device__ __forceinline__ PairUnit pair_unit(int64_t u, int64_t full_units) {
  PairUnit r;
  if (u < full_units) {
    r.tile = u;
    r.narrow = 0;
    r.half = 0;
  } else {
    const int64_t k = u - full_units;
    r.tile = full_units + (k >> 1);
    r.narrow = 1;
    r.half = (int)(k & 1);
  }
  return r;
}

template <int EPI, int EW>
__global__ void __launch_bounds__(tc_threads(EW), 1)
    gemm_i8_tc2_kernel(const __grid_constant__ CUtensorMap map_a,
        const __grid_constant__ CUtensorMap map_b,
        const __grid_constant__ CUtensorMap map_b_half,
        const __grid_constant__ CUtensorMap map_y,
        const __grid_constant__ CUtensorMap map_y2, EpiParams p, uint32_t idesc,
        uint32_t idesc_half, int64_t full_units, int64_t num_units, int *status,
        uint64_t wait_ns) {
  constexpr int BN = 256;
  constexpr int kABytes = kBM * kBK;
  constexpr int kBHalfBytes = (BN / 2) * kBK;
  constexpr int kStageBytes = kABytes + kBHalfBytes; // 32 KiB per CTA
  constexpr int kStages = tc_stages(kStageBytes, EW);
  constexpr int kTmemCols = 2 * BN;
  constexpr int kSlabBytes = 32 * 128;
  constexpr int kHalfCols = epi_cols_per_warp(BN, EW);

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[kStages];
  __shared__ uint64_t bar_empty[kStages];
  __shared__ uint64_t bar_acc_full[2];
  __shared__ uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(); // 0 = leader
  const int64_t cluster_id = blockIdx.x >> 1;
  const int64_t num_clusters = gridDim.x >> 1;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t staging_base = smem_base + kStages * kStageBytes;

  const int64_t tiles_n = ceil_div(p.N, BN);
  const int num_kb = (int)ceil_div(p.K, kBK);
  // Split-K pass: unit u is K slice u % split of tile u / split (all units
  // whole tiles then).
  const int split = p.split_k;
  if (threadIdx.x == 32) { // (a thread that has nothing else to set up)
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    if (p.line_store) {
      prefetch_tensormap(&map_y);
      if (EPI == OMCUDA_EPI_DEQUANT_SPLIT)
        prefetch_tensormap(&map_y2);
    }
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_acc_full[b]), 1);
      mbar_init(smem_u32(&bar_acc_empty[b]), 2 * epi_active_warps(BN, EW));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1)
    tmem_alloc_pair(smem_u32(&tmem_base_slot), kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all(); // both CTAs' barriers exist before anyone signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int *abortp = &abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t pol_a = l2_policy_evict_first(), pol_b = l2_policy_evict_last();
      for (int64_t u = cluster_id; u < num_units && ok; u += num_clusters) {
        const PairUnit un = pair_unit(u, full_units);
        const int64_t t = split > 1 ? un.tile / split : un.tile;
        const int ks = split > 1 ? (int)(un.tile % split) : 0;
        const int kb0 = (int)((int64_t)ks * num_kb / split);
        const int kb1 = (int)((int64_t)(ks + 1) * num_kb / split);
        const int32_t m0 = (int32_t)((t / tiles_n) * (2 * kBM) + rank * kBM);
        // this CTA's share of the B columns: 128 of 256, or 64 of 128
        const int32_t n0 = un.narrow
                               ? (int32_t)((t % tiles_n) * BN + un.half * (BN / 2) + rank * (BN / 4))
                               : (int32_t)((t % tiles_n) * BN + rank * (BN / 2));
        const uint32_t stage_tx = un.narrow ? kABytes + kBHalfBytes / 2 : kStageBytes;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp, wait_ns)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = mapa_shared(smem_u32(&bar_full[stage]), 0);
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
          if (rank == 0)
            mbar_expect_tx(smem_u32(&bar_full[stage]), 2 * stage_tx);
          if (p.l2_hints & 2)
            tma_load_2d_pair_hint(sa, &map_a, kb * kBK, m0, full_leader, pol_a);
          else
            tma_load_2d_pair(sa, &map_a, kb * kBK, m0, full_leader);
          if (p.l2_hints & 4)
            tma_load_2d_pair_hint(sb, un.narrow ? &map_b_half : &map_b, kb * kBK, n0,
                full_leader, pol_b);
          else
            tma_load_2d_pair(sb, un.narrow ? &map_b_half : &map_b, kb * kBK, n0, full_leader);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int64_t it = 0;
      bool landed = false; // asked one stage ahead, see the single-CTA kernel
      for (int64_t u = cluster_id; u < num_units && ok; u += num_clusters, ++it) {
        const uint32_t unit_idesc = u < full_units ? idesc : idesc_half;
        const int ks = split > 1 ? (int)(u % split) : 0;
        const int kb0 = (int)((int64_t)ks * num_kb / split);
        const int kb1 = (int)((int64_t)(ks + 1) * num_kb / split);
        const int buf = (int)(it & 1);
        const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
        if (!mbar_wait(smem_u32(&bar_acc_empty[buf]), acc_phase ^ 1u, abortp, wait_ns)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!landed && !mbar_wait(smem_u32(&bar_full[stage]), phase, abortp, wait_ns)) {
            ok = false;
            break;
          }
          const int nstage = stage + 1 == kStages ? 0 : stage + 1;
          const uint32_t nphase = nstage == 0 ? phase ^ 1u : phase;
          landed = mbar_test_wait(smem_u32(&bar_full[nstage]), nphase);
          tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
          static_assert(kBK / kUmmaK == 4, "four K slices per stage");
          umma_i8_pair_x4(d_tmem, make_smem_desc(sa), make_smem_desc(sb), unit_idesc,
              kb != kb0 ? 1u : 0u);
          umma_commit_pair(smem_u32(&bar_empty[stage]), 3);
          stage = nstage;
          phase = nphase;
        }
        if (ok)
          umma_commit_pair(smem_u32(&bar_acc_full[buf]), 3);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9 of both CTAs) ----------------
    const int quad = warp & 3;
    const int ew = warp - 2;
    const int c_lo = (ew >> 2) * kHalfCols;
    const bool active = c_lo < BN;
    const EpiScalars sc = epi_scalars(p);
    const QuantConsts qc = epi_quant_consts<EPI>(p, warp == 2 && lane == 0 && blockIdx.x == 0);
    const bool use_slab = p.line_store != 0;
    const uint32_t slab0 = staging_base + (uint32_t)ew * kSlabBytes;
    bool ok = active;
    int64_t it = 0;
    float lo = INFINITY, hi = -INFINITY; // range of this warp's f32 outputs
    for (int64_t u = cluster_id; u < num_units && ok; u += num_clusters, ++it) {
      const PairUnit un = pair_unit(u, full_units);
      const int64_t t = split > 1 ? un.tile / split : un.tile;
      const int32_t row_off = split > 1 ? (int32_t)((un.tile % split) * p.ws_rows) : 0;
      const int buf = (int)(it & 1);
      const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
      const int64_t m_warp = (t / tiles_n) * (2 * kBM) + rank * kBM + quad * 32;
      const int64_t n0 = (t % tiles_n) * BN + un.half * (BN / 2) + c_lo;
      // a half tile keeps only the warps of accumulator columns 0..127 busy
      const bool mine = !un.narrow || c_lo < BN / 2;
      if (mine) {
        const int line = lane & 7, which = lane >> 3;
        const int64_t nl = n0 + 32 * line;
        const void *src = nullptr;
        if (32 * line < kHalfCols && nl < p.N) {
          if (which == 0 && p.a_zp_len != 0)
            src = p.colsum + nl;
          else if (which == 1 && p.bias)
            src = p.bias + nl;
          else if (which == 2 && p.sb && p.sb_len != 1)
            src = p.sb + nl;
        }
        if (src)
          asm volatile("prefetch.global.L1 [%0];" ::"l"(src));
        // ... and this warp's block of the residual (32 rows x kHalfCols f32)
        // towards L2: the epilogue reads it one row per thread.
        if (p.residual && m_warp + lane < p.M) {
          const float *rr = p.residual + (m_warp + lane) * p.N + n0;
          for (int c = 0; c < kHalfCols && n0 + c < p.N; c += 32)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(rr + c));
        }
      }
      if (!mbar_wait(smem_u32(&bar_acc_full[buf]), acc_phase, abortp, wait_ns)) {
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const uint32_t taddr =
          tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN + c_lo);
      auto release = [&] {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0)
          mbar_arrive_cluster(mapa_shared(smem_u32(&bar_acc_empty[buf]), 0));
      };
      if (mine)
        epilogue_tile<BN, EPI, EW>(p, sc, qc, taddr, m_warp, n0, slab0, lane, use_slab,
            lo, hi, &map_y, &map_y2, release, row_off);
      else
        release();
    }
    if (active && p.out_range && epi_is_dequant(EPI) && EPI != OMCUDA_EPI_DEQUANT_QUANT)
      epi_range_commit(p.out_range, lo, hi);
    if (lane == 0)
      tma_store_wait_all();
  }

  // ---------------- teardown ----------------
  // Neither CTA may leave (or free tensor memory) while its peer can still
  // signal its barriers or read its shared memory.
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && abort_flag)
    atomicExch(status, 1);
}

// ---- host side ----------------------------------------------------------------------

// 2-D tensor map over a row-major [rows, cols] matrix of esize-byte elements
// (1: u8, 2: bf16, 4: i32) whose row pitch is pitch bytes; box = box_cols x
// box_rows elements with box_cols * esize == swizzle_bytes (32, 64 or 128: the
// swizzle mode of that width); loads fill with zeros outside the matrix, stores
// clip.
int make_tma_map_2d(CUtensorMap *map, const void *base, int64_t rows,
    int64_t cols, int64_t pitch, int box_cols, int box_rows, int esize,
    int swizzle_bytes) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t,
      void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
      const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiledFn fn = nullptr;
  static std::once_flag looked_up;
  std::call_once(looked_up, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault,
            &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  if (!fn)
    return fail(OMCUDA_ECUDA, "cuTensorMapEncodeTiled is not available");
  // A box row must span exactly the swizzle width, so that rows are packed
  // densely in shared memory in the pattern the kernels assume.
  if (box_cols * esize != swizzle_bytes ||
      (swizzle_bytes != 32 && swizzle_bytes != 64 && swizzle_bytes != 128))
    return fail(OMCUDA_EINVAL, "tensor map: box row of %d bytes with a %d-byte swizzle",
        box_cols * esize, swizzle_bytes);
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = esize == 4   ? CU_TENSOR_MAP_DATA_TYPE_INT32
                                 : esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                              : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE,
      swizzle_bytes == 32   ? CU_TENSOR_MAP_SWIZZLE_32B
      : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(OMCUDA_ECUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return OMCUDA_OK;
}

// State the tensor-core launchers keep per device (the device current on the
// calling thread): the status word a CTA whose bounded wait gave up sets to
// non-zero, and which kernels already had their launch attributes set.
// Guarded by one mutex; the launch path takes it only for a table look-up.
static std::mutex g_dev_mutex;
static int *g_status_words[kMaxDevices] = {nullptr};
static std::atomic<uint64_t> g_wait_limit_ns{kWaitLimitNs};


int *tc_status_word() {
  const int dev = current_device_index();
  if (dev < 0)
    return nullptr;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_status_words[dev]) {
    int *w = nullptr;
    if (cudaMalloc(&w, sizeof(int)) != cudaSuccess)
      return nullptr;
    if (cudaMemset(w, 0, sizeof(int)) != cudaSuccess) {
      cudaFree(w);
      return nullptr;
    }
    g_status_words[dev] = w;
  }
  return g_status_words[dev];
}

uint64_t tc_wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }

namespace {

// 2-D map for the GEMM operands: box = 128 bytes x box_rows.
int make_map(CUtensorMap *map, const void *base, int64_t rows, int64_t cols,
    int64_t pitch, int box_rows, int esize = 1) {
  return make_tma_map_2d(map, base, rows, cols, pitch, kBK / esize, box_rows, esize, 128);
}

// Instruction descriptor of tcgen05.mma kind::i8: s32 accumulator, operand
// signedness per operand, both operands K-major, N and M of the instruction.
uint32_t make_idesc(int a_signed, int b_signed, int n) {
  uint32_t d = 0;
  d |= 2u << 4;                        // accumulator format: s32
  d |= (a_signed ? 1u : 0u) << 7;      // A: 0 = u8, 1 = s8
  d |= (b_signed ? 1u : 0u) << 10;     // B: 0 = u8, 1 = s8
  d |= (uint32_t)(n >> 3) << 17;       // N / 8
  d |= (uint32_t)(kBM >> 4) << 24;     // M / 16
  return d;
}

// 16-byte stores of whole lines need an aligned base and row pitch (the
// range-only tail stores nothing and walks the tile the same way).
template <int EPI>
bool y_takes_line_stores(const omcudaGemmArgs &a) {
  if (EPI == OMCUDA_EPI_DEQUANT_RANGE)
    return true;
  const int esize = (EPI == OMCUDA_EPI_REQUANT || EPI == OMCUDA_EPI_DEQUANT_QUANT)
                        ? 1
                        : (EPI == OMCUDA_EPI_DEQUANT_SPLIT ? 2 : 4);
  return (((uintptr_t)a.Y & 15u) == 0) && ((a.N * esize) % 16 == 0);
}

// Tensor maps of the output for the epilogue's TMA stores: boxes of 32 rows x
// one slab row (32 f32 / i32 columns; kHalfCols, at most 128, u8 columns; 32
// bf16 columns of the hi and of the lo plane).  Only encoded when Y can take
// them (16-byte aligned base and row pitch); otherwise the kernel stores
// directly and never reads the maps.
template <int EPI>
int make_y_maps(const omcudaGemmArgs &a, int half_cols, bool line_store,
    CUtensorMap *map_y, CUtensorMap *map_y2) {
  memset(map_y, 0, sizeof(*map_y));
  memset(map_y2, 0, sizeof(*map_y2));
  if (!line_store)
    return OMCUDA_OK;
  int rc;
  if (EPI == OMCUDA_EPI_DEQUANT_RANGE)
    return OMCUDA_OK; // nothing is stored
  if (EPI == OMCUDA_EPI_REQUANT || EPI == OMCUDA_EPI_DEQUANT_QUANT) {
    const int cols = half_cols < 128 ? half_cols : 128; // 32, 64 or 128
    rc = make_tma_map_2d(map_y, a.Y, a.M, a.N, a.N, cols, 32, 1, cols);
  } else if (EPI == OMCUDA_EPI_DEQUANT_SPLIT) {
    rc = make_tma_map_2d(map_y, a.Y, a.M, a.N, a.N * 2, 32, 32, 2, 64);
    if (rc == OMCUDA_OK)
      rc = make_tma_map_2d(map_y2, (const uint8_t *)a.Y + (size_t)a.M * a.N * 2, a.M,
          a.N, a.N * 2, 32, 32, 2, 64);
  } else {
    rc = make_tma_map_2d(map_y, a.Y, a.M, a.N, a.N * 4, 32, 32, 4, 128);
  }
  return rc;
}

// L2 eviction hints (EpiParams::l2_hints); OMCUDA_GEMM_L2_HINTS=0..7 overrides
// the default, for experiments.
inline int l2_hints_wanted() {
  static const int v = [] {
    const char *s = getenv("OMCUDA_GEMM_L2_HINTS");
    return s ? atoi(s) & 7 : 0;
  }();
  return v;
}

// ---- split-K -------------------------------------------------------------------------
//
// A GEMM with few output tiles and a long K loop leaves most SMs idle, and the
// ones that work are bound by how fast one SM takes operands in.  Split-K
// deals the K loop of every tile to `split` work units; each stores its raw
// 32-bit sums into its own slice of a workspace (the EPI_I32 tail without zero
// points, through the same TMA stores), and splitk_reduce_kernel adds the
// slices and runs the real tail.  Integer sums are exact in any order, so the
// result equals the unsplit kernel's bit for bit.
struct SplitPlan {
  int split = 1;
  int64_t ws_rows = 0;   // rows per slice: M rounded up to the 32 rows of a store slab
  int32_t *ws = nullptr; // [split][ws_rows][N]
};

// One thread per four adjacent outputs of a row.
__global__ void __launch_bounds__(256)
    splitk_reduce_kernel(const int32_t *__restrict__ ws, int split, int64_t ws_rows,
        EpiParams p) {
  const int64_t n4 = p.N >> 2; // the split path requires N % 4 == 0
  const int64_t total = p.M * n4;
  const EpiScalars sc = epi_scalars(p);
  float lo = INFINITY, hi = -INFINITY;
  const bool y16 = (((uintptr_t)p.Y) & 15u) == 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / n4, n = (i - m * n4) << 2;
    int4 acc = make_int4(0, 0, 0, 0);
    for (int k = 0; k < split; ++k) {
      const int4 v = __ldcs(reinterpret_cast<const int4 *>(
          ws + ((int64_t)k * ws_rows + m) * p.N + n));
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    const EpiRow row = epi_row(p, m);
    const int32_t v[4] = {epi_int(p, row, acc.x, n), epi_int(p, row, acc.y, n + 1),
        epi_int(p, row, acc.z, n + 2), epi_int(p, row, acc.w, n + 3)};
    if (p.kind == OMCUDA_EPI_I32) {
      int32_t *dst = reinterpret_cast<int32_t *>(p.Y) + m * p.N + n;
      if (y16)
        *reinterpret_cast<int4 *>(dst) = make_int4(v[0], v[1], v[2], v[3]);
      else
        for (int j = 0; j < 4; ++j)
          dst[j] = v[j];
    } else if (p.kind == OMCUDA_EPI_DEQUANT) {
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        y[j] = epi_dequant(p, sc, v[j], n + j);
        if (p.residual)
          y[j] = __fadd_rn(y[j], __ldg(p.residual + m * p.N + n + j));
        lo = fminf(lo, y[j]);
        hi = fmaxf(hi, y[j]);
      }
      float *dst = reinterpret_cast<float *>(p.Y) + m * p.N + n;
      if (y16)
        *reinterpret_cast<float4 *>(dst) = make_float4(y[0], y[1], y[2], y[3]);
      else
        for (int j = 0; j < 4; ++j)
          dst[j] = y[j];
    } else { // OMCUDA_EPI_REQUANT
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        w |= epi_requant(p, sc, v[j], n + j) << (8 * j);
      uint8_t *dst = reinterpret_cast<uint8_t *>(p.Y) + m * p.N + n;
      if ((((uintptr_t)dst) & 3u) == 0)
        *reinterpret_cast<uint32_t *>(dst) = w;
      else
        for (int j = 0; j < 4; ++j)
          dst[j] = (uint8_t)(w >> (8 * j));
    }
  }
  if (p.out_range && p.kind == OMCUDA_EPI_DEQUANT)
    epi_range_commit(p.out_range, lo, hi);
}

// The arguments of the pass that produces the raw partial sums.
omcudaGemmArgs split_pass_args(const omcudaGemmArgs &a, const SplitPlan &plan) {
  omcudaGemmArgs r = a;
  r.epilogue = OMCUDA_EPI_I32;
  r.a_zp = nullptr;
  r.a_zp_len = 0;
  r.b_zp = nullptr;
  r.b_zp_len = 0;
  r.a_rowsum = nullptr;
  r.residual = nullptr;
  r.out_minmax = nullptr;
  r.Y = plan.ws;
  return r;
}

template <int BN, int EPI, int EW>
int launch_bn_epi_ew(const omcudaGemmArgs &a, cudaStream_t st, const SplitPlan &plan = SplitPlan()) {
  using Cfg = TcConfig<BN, EW>;
  static PerDeviceInt attr_set;
  if (!attr_set.get()) {
    OMCUDA_CHECK(cudaFuncSetAttribute(gemm_i8_tc_kernel<BN, EPI, EW>,
        cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set.set(1);
  }
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, a.A, a.M, a.K, a.K, kBM);
  if (rc != OMCUDA_OK)
    return rc;
  rc = make_map(&map_b, a.B.bt, a.N, a.B.kp, a.B.kp, BN);
  if (rc != OMCUDA_OK)
    return rc;
  EpiParams p = make_epi_params(a);
  p.line_store = y_takes_line_stores<EPI>(a);
  p.l2_hints = l2_hints_wanted();
  p.split_k = plan.split;
  p.ws_rows = plan.ws_rows;
  int *status = tc_status_word();
  if (!status)
    return fail(OMCUDA_ENOMEM, "GemmI8: cannot allocate the status word");
  CUtensorMap map_y, map_y2;
  omcudaGemmArgs ya = a; // the matrix the stores see: all slices of the workspace
  if (plan.split > 1)
    ya.M = plan.split * plan.ws_rows;
  rc = make_y_maps<EPI>(ya, epi_cols_per_warp(BN, EW), p.line_store != 0, &map_y, &map_y2);
  if (rc != OMCUDA_OK)
    return rc;
  int64_t tiles = ceil_div(a.M, kBM) * ceil_div(a.N, BN) * plan.split;
  int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  uint32_t idesc = make_idesc(a.a_signed, a.B.b_signed, BN);
  gemm_i8_tc_kernel<BN, EPI, EW><<<grid, tc_threads(EW), Cfg::kSmemBytes, st>>>(
      map_a, map_b, map_y, map_y2, p, idesc, status, tc_wait_limit_ns());
  OMCUDA_CHECK_LAUNCH("gemm_i8_tc_kernel");
  return OMCUDA_OK;
}

// A long K loop hides the epilogue behind the MMAs and wants pipeline depth;
// a short one is bounded by the epilogue and wants more warps on it.
// (OMCUDA_GEMM_EW=8|16 overrides the choice, for experiments.)
inline bool want_wide_epilogue(const omcudaGemmArgs &a) {
  static const int forced = [] {
    const char *s = getenv("OMCUDA_GEMM_EW");
    return s ? atoi(s) : 0;
  }();
  if (forced == 8 || forced == 16)
    return forced == 16;
  return a.K < 2048;
}

template <int BN, int EPI>
int launch_bn_epi(const omcudaGemmArgs &a, cudaStream_t st) {
  return want_wide_epilogue(a) ? launch_bn_epi_ew<BN, EPI, 16>(a, st)
                               : launch_bn_epi_ew<BN, EPI, 8>(a, st);
}

template <int BN>
int launch_bn(const omcudaGemmArgs &a, cudaStream_t st) {
  switch (a.epilogue) {
  case OMCUDA_EPI_I32:
    return launch_bn_epi<BN, OMCUDA_EPI_I32>(a, st);
  case OMCUDA_EPI_DEQUANT:
    return launch_bn_epi<BN, OMCUDA_EPI_DEQUANT>(a, st);
  case OMCUDA_EPI_REQUANT:
    return launch_bn_epi<BN, OMCUDA_EPI_REQUANT>(a, st);
  case OMCUDA_EPI_DEQUANT_SPLIT:
    return launch_bn_epi<BN, OMCUDA_EPI_DEQUANT_SPLIT>(a, st);
  case OMCUDA_EPI_DEQUANT_RANGE:
    return launch_bn_epi<BN, OMCUDA_EPI_DEQUANT_RANGE>(a, st);
  case OMCUDA_EPI_DEQUANT_QUANT:
    return launch_bn_epi<BN, OMCUDA_EPI_DEQUANT_QUANT>(a, st);
  default:
    return fail(OMCUDA_EINVAL, "GemmI8: unknown epilogue %d", a.epilogue);
  }
}


// OMCUDA_GEMM_HALF_TILES=0 keeps every unit a whole tile, for experiments.
inline bool pair_half_tiles_wanted() {
  static const bool on = [] {
    const char *s = getenv("OMCUDA_GEMM_HALF_TILES");
    return !(s && atoi(s) == 0);
  }();
  return on;
}

// The 2-CTA kernel: 256 x 256 tiles on clusters of two CTAs.
template <int EPI, int EW>
int launch_pair_epi_ew(const omcudaGemmArgs &a, cudaStream_t st, const SplitPlan &plan = SplitPlan()) {
  constexpr int kThreads = tc_threads(EW);
  constexpr int kPairSmemBytes =
      tc_stages(kBM * kBK + 128 * kBK, EW) * (kBM * kBK + 128 * kBK) +
      EW * 32 * 128 + 1024;
  static PerDeviceInt max_clusters_dev;
  int max_clusters = max_clusters_dev.get();
  if (max_clusters == 0) {
    OMCUDA_CHECK(cudaFuncSetAttribute(gemm_i8_tc2_kernel<EPI, EW>,
        cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes));
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3((unsigned)sm_count() & ~1u, 1, 1);
    q.blockDim = dim3(kThreads, 1, 1);
    q.dynamicSmemBytes = kPairSmemBytes;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    q.attrs = qa;
    q.numAttrs = 1;
    int n = 0;
    OMCUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, gemm_i8_tc2_kernel<EPI, EW>, &q));
    max_clusters = n > 0 ? n : 1;
    max_clusters_dev.set(max_clusters);
  }
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, a.A, a.M, a.K, a.K, kBM);
  if (rc != OMCUDA_OK)
    return rc;
  rc = make_map(&map_b, a.B.bt, a.N, a.B.kp, a.B.kp, 128);
  if (rc != OMCUDA_OK)
    return rc;
  CUtensorMap map_b_half; // 64 B columns per CTA: the 256 x 128 units
  rc = make_map(&map_b_half, a.B.bt, a.N, a.B.kp, a.B.kp, 64);
  if (rc != OMCUDA_OK)
    return rc;
  EpiParams p = make_epi_params(a);
  p.line_store = y_takes_line_stores<EPI>(a);
  p.l2_hints = l2_hints_wanted();
  p.split_k = plan.split;
  p.ws_rows = plan.ws_rows;
  int *status = tc_status_word();
  if (!status)
    return fail(OMCUDA_ENOMEM, "GemmI8: cannot allocate the status word");
  int64_t tiles = ceil_div(a.M, 2 * kBM) * ceil_div(a.N, 256) * plan.split;
  // Units: whole tiles for the complete rounds; a last round that would keep
  // at most half of the clusters busy runs as twice as many half tiles
  // (never in a split-K pass, whose units are K slices of whole tiles).
  const int64_t rounds_full = (tiles / max_clusters) * max_clusters;
  const int64_t rest = tiles - rounds_full;
  const bool split_rest = plan.split == 1 && rest > 0 && 2 * rest <= max_clusters &&
                          pair_half_tiles_wanted();
  const int64_t full_units = split_rest ? rounds_full : tiles;
  const int64_t num_units = split_rest ? rounds_full + 2 * rest : tiles;
  int clusters = (int)(num_units < max_clusters ? num_units : max_clusters);
  // M = 256 across the pair (field holds M / 16), N = 256 or 128.
  uint32_t idesc = make_idesc(a.a_signed, a.B.b_signed, 256);
  idesc = (idesc & ~(0x1fu << 24)) | ((uint32_t)(256 >> 4) << 24);
  uint32_t idesc_half = make_idesc(a.a_signed, a.B.b_signed, 128);
  idesc_half = (idesc_half & ~(0x1fu << 24)) | ((uint32_t)(256 >> 4) << 24);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUtensorMap map_y, map_y2;
  omcudaGemmArgs ya = a; // the matrix the stores see: all slices of the workspace
  if (plan.split > 1)
    ya.M = plan.split * plan.ws_rows;
  rc = make_y_maps<EPI>(ya, epi_cols_per_warp(256, EW), p.line_store != 0, &map_y, &map_y2);
  if (rc != OMCUDA_OK)
    return rc;
  OMCUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_i8_tc2_kernel<EPI, EW>, map_a, map_b,
      map_b_half, map_y, map_y2, p, idesc, idesc_half, full_units, num_units, status,
      tc_wait_limit_ns()));
  count_launch();
  return OMCUDA_OK;
}

template <int EPI>
int launch_pair_epi(const omcudaGemmArgs &a, cudaStream_t st) {
  return want_wide_epilogue(a) ? launch_pair_epi_ew<EPI, 16>(a, st)
                               : launch_pair_epi_ew<EPI, 8>(a, st);
}

int launch_pair(const omcudaGemmArgs &a, cudaStream_t st) {
  switch (a.epilogue) {
  case OMCUDA_EPI_I32:
    return launch_pair_epi<OMCUDA_EPI_I32>(a, st);
  case OMCUDA_EPI_DEQUANT:
    return launch_pair_epi<OMCUDA_EPI_DEQUANT>(a, st);
  case OMCUDA_EPI_REQUANT:
    return launch_pair_epi<OMCUDA_EPI_REQUANT>(a, st);
  case OMCUDA_EPI_DEQUANT_SPLIT:
    return launch_pair_epi<OMCUDA_EPI_DEQUANT_SPLIT>(a, st);
  case OMCUDA_EPI_DEQUANT_RANGE:
    return launch_pair_epi<OMCUDA_EPI_DEQUANT_RANGE>(a, st);
  case OMCUDA_EPI_DEQUANT_QUANT:
    return launch_pair_epi<OMCUDA_EPI_DEQUANT_QUANT>(a, st);
  default:
    return fail(OMCUDA_EINVAL, "GemmI8: unknown epilogue %d", a.epilogue);
  }
}

// OMCUDA_GEMM_SPLIT_K=0 switches split-K off, N > 1 forces N slices wherever
// the shape allows it (experiments).
inline int split_k_forced() {
  static const int v = [] {
    const char *s = getenv("OMCUDA_GEMM_SPLIT_K");
    return s ? atoi(s) : -1;
  }();
  return v;
}

// How many K slices a GEMM of up to 512 rows should run as (1: none).  The
// partial pass uses 128 x 256 tiles on single CTAs up to 128 rows and 256 x
// 256 tiles on CTA pairs above.  The second launch and the round trip of the
// partial sums through L2 cost about 6 us, so it pays only when those tiles
// would occupy at most half of the machine and the K loop is long (measured
// with 32..512 rows: K = 14336, N = 4096 29-36 us against 43-45 us unsplit;
// K = 4096 20-37 us against 19-27 us, so K below 8192 stays unsplit).
int split_k_for(const omcudaGemmArgs &a, cudaStream_t st) {
  if (split_k_forced() == 0 || a.M > 512 || a.N < 256 || (a.N & 3) != 0)
    return 1;
  if (a.epilogue != OMCUDA_EPI_I32 && a.epilogue != OMCUDA_EPI_DEQUANT &&
      a.epilogue != OMCUDA_EPI_REQUANT)
    return 1;
  const int64_t num_kb = ceil_div(a.K, kBK);
  if (num_kb < 64 && split_k_forced() <= 1)
    return 1;
  const bool pair = a.M > kBM;
  const int64_t units = (pair ? ceil_div(a.M, 2 * kBM) : 1) * ceil_div(a.N, 256);
  const int64_t slots = pair ? sm_count() / 2 : sm_count();
  int64_t split = slots / units;
  if (split_k_forced() > 1)
    split = split_k_forced();
  if (split > num_kb / 4)
    split = num_kb / 4;
  if (split > 16)
    split = 16;
  if (split < 2)
    return 1;
  // The workspace comes from the stream-ordered pool, whose bookkeeping
  // (an event per freed block) must not run inside a stream capture.
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return 1;
  }
  return (int)split;
}

int launch_split_k(const omcudaGemmArgs &a, cudaStream_t st, int split) {
  SplitPlan plan;
  plan.split = split;
  plan.ws_rows = (a.M + 31) & ~int64_t(31);
  const size_t ws_bytes = (size_t)split * (size_t)plan.ws_rows * (size_t)a.N * sizeof(int32_t);
  plan.ws = static_cast<int32_t *>(pool_alloc_on(ws_bytes, st));
  if (!plan.ws)
    return fail(OMCUDA_ENOMEM, "GemmI8: cannot allocate the split-K workspace");
  const omcudaGemmArgs part = split_pass_args(a, plan);
  int rc;
  if (a.M > kBM)
    rc = want_wide_epilogue(a) ? launch_pair_epi_ew<OMCUDA_EPI_I32, 16>(part, st, plan)
                               : launch_pair_epi_ew<OMCUDA_EPI_I32, 8>(part, st, plan);
  else
    rc = want_wide_epilogue(a) ? launch_bn_epi_ew<256, OMCUDA_EPI_I32, 16>(part, st, plan)
                               : launch_bn_epi_ew<256, OMCUDA_EPI_I32, 8>(part, st, plan);
  if (rc == OMCUDA_OK) {
    const EpiParams p = make_epi_params(a);
    const int64_t total = a.M * (a.N >> 2);
    const int64_t blocks = ceil_div(total, 256);
    const int64_t cap = (int64_t)sm_count() * 8;
    splitk_reduce_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(
        plan.ws, split, plan.ws_rows, p);
    cudaError_t ce = cudaGetLastError();
    if (ce != cudaSuccess)
      rc = fail(OMCUDA_ECUDA, "splitk_reduce_kernel: %s", cudaGetErrorString(ce));
    else
      count_launch();
  }
  pool_free_on(plan.ws, st);
  return rc;
}

} // namespace

bool gemm_tc_supported(const omcudaGemmArgs &a) {
  return (a.K % 16 == 0) && (((uintptr_t)a.A & 15u) == 0) &&
         (((uintptr_t)a.B.bt & 15u) == 0) && a.M < (int64_t(1) << 31) &&
         a.N < (int64_t(1) << 31);
}

int launch_gemm_tc(const omcudaGemmArgs &a, cudaStream_t st) {
  // Tile width: the widest tile that still gives every SM work
  // (OMCUDA_GEMM_BN=64|128|256 overrides the choice, 512 selects the 2-CTA
  // kernel, for experiments).
  static const int forced_bn = [] {
    const char *s = getenv("OMCUDA_GEMM_BN");
    return s ? atoi(s) : 0;
  }();
  if (forced_bn == 0 || split_k_forced() > 1) {
    const int split = split_k_for(a, st);
    if (split > 1)
      return launch_split_k(a, st, split);
  }
  if (forced_bn == 512)
    return launch_pair(a, st);
  if (forced_bn == 256)
    return launch_bn<256>(a, st);
  if (forced_bn == 128)
    return launch_bn<128>(a, st);
  if (forced_bn == 64)
    return launch_bn<64>(a, st);
  const int64_t tm = ceil_div(a.M, kBM);
  const int sms = sm_count();
  // Enough 256 x 256 tiles to occupy the pairs of SMs (three quarters of them
  // will do when both CTAs of a pair have rows to work on): the 2-CTA kernel.
  // (256 x 4096 x 14336: 56 tiles on 74 pairs run 32.6 us, the 224 tiles of
  // 128 x 128 in one and a half rounds 37.1 us; with 128 rows or fewer the
  // single-CTA tiles win, 26 against 31 us.)
  const int64_t pair_tiles = ceil_div(a.M, 2 * kBM) * ceil_div(a.N, 256);
  if (a.N > 128 && (pair_tiles >= sms / 2 || (a.M > kBM && pair_tiles * 4 >= (sms / 2) * 3)))
    return launch_pair(a, st);
  if (a.N > 128 && tm * ceil_div(a.N, 256) >= sms)
    return launch_bn<256>(a, st);
  if (a.N > 64 && tm * ceil_div(a.N, 128) >= sms / 2)
    return launch_bn<128>(a, st);
  return launch_bn<64>(a, st);
}

// Reads (and clears) the word the tensor-core kernels raise when a bounded
// wait gave up.  Synchronises the stream.
int gemm_tc_check_status(cudaStream_t st) {
  int *word = nullptr;
  {
    const int dev = current_device_index();
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    word = dev >= 0 ? g_status_words[dev] : nullptr;
  }
  if (!word)
    return OMCUDA_OK;
  int h = 0;
  OMCUDA_CHECK(cudaMemcpyAsync(&h, word, sizeof(int), cudaMemcpyDeviceToHost, st));
  OMCUDA_CHECK(cudaStreamSynchronize(st));
  if (h != 0) {
    cudaMemsetAsync(word, 0, sizeof(int), st);
    return fail(OMCUDA_ETIMEDOUT,
        "a device-side wait on the TMA/MMA pipeline of a tensor-core kernel timed out");
  }
  return OMCUDA_OK;
}

// ---- bounded-wait self test ---------------------------------------------------------
//
// One CTA that does what the GEMM kernels do around a wait -- allocate tensor
// memory, arm an mbarrier, wait on it with mbar_wait -- except that nobody ever
// signals the barrier.  The wait must give up after wait_ns by itself, the CTA
// must free its tensor memory, raise the status word and return.
__global__ void __launch_bounds__(64, 1)
    bounded_wait_selftest_kernel(int *status, uint64_t wait_ns, uint64_t *waited_ns) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1)
    tmem_alloc(smem_u32(&tmem_base_slot), 64);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  if (threadIdx.x == 0) {
    const uint64_t t0 = global_timer();
    (void)mbar_wait(smem_u32(&bar), 0, &abort_flag, wait_ns); // phase 0 never completes
    if (waited_ns)
      *waited_ns = global_timer() - t0;
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
  if (threadIdx.x == 0 && abort_flag)
    atomicExch(status, 1);
}

} // namespace omcuda

extern "C" void omcudaDevSetWaitLimitNs(int64_t ns) {
  omcuda::g_wait_limit_ns.store(
      ns > 0 ? (uint64_t)ns : omcuda::kWaitLimitNs, std::memory_order_relaxed);
}

extern "C" int omcudaDevSelfTestBoundedWait(uint64_t *waited_ns_dev, void *stream) {
  using namespace omcuda;
  if (ensure_init() != OMCUDA_OK)
    return omcudaGetLastError();
  int *status = tc_status_word();
  if (!status)
    return fail(OMCUDA_ENOMEM, "SelfTestBoundedWait: cannot allocate the status word");
  // Never wait longer than a second here, whatever the configured limit.
  uint64_t ns = tc_wait_limit_ns();
  if (ns > 1000000000ull)
    ns = 1000000000ull;
  bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, ns, waited_ns_dev);
  OMCUDA_CHECK_LAUNCH("bounded_wait_selftest_kernel");
  return OMCUDA_OK;
}
