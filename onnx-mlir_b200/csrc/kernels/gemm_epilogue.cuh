// Epilogue arithmetic shared by the tensor-core and SIMT int8 GEMM kernels.
//
// The raw accumulator is sum_k A[m,k]*B[k,n] over the widened 8-bit operands.
// onnx-mlir subtracts the zero points before multiplying
// (src/Conversion/ONNXToKrnl/Math/MatMulInteger.cpp:59-84); expanding the
// product gives, in wrapping 32-bit arithmetic (exactly what arith.muli/addi
// compute):
//   sum (A-az)(B-bz) = acc - az*colsum_B[n] - bz[n]*rowsum_A[m] + K*az*bz[n]
// so zero points cost one or two multiply-adds per output instead of a pass
// over the operands.
//
// The three tails:
//   I32      MatMulInteger result.
//   DEQUANT  Cast(i32->f32) -> Mul -> [Mul] -> [Add] [-> Gelu] [-> Add residual]
//            (src/Conversion/ONNXToKrnl/Math/Elementwise.cpp:477-486, 358-388);
//            each fp32 op is rounded on its own (no fma).
//   DEQUANT_SPLIT  the DEQUANT value x written as two bf16 planes,
//            hi = bf16(x) and lo = bf16(x - hi): the operand format of the
//            tensor-core attention kernel (tensor-core GEMM only).
//   DEQUANT_RANGE / DEQUANT_QUANT  the DEQUANT value folded into a running
//            range only, and the same value quantized as DynamicQuantizeLinear
//            would with the parameters that range gives (tensor-core GEMM
//            only): together "linear -> DynamicQuantizeLinear" without the f32
//            tensor ever reaching memory.
//   REQUANT  QLinearMatMul: f32(acc) * S[n], round half even, fptosi,
//            + y zero point, truncate to 8 bits
//            (src/Conversion/ONNXToKrnl/Math/QLinearMatMul.cpp:123-138).
#pragma once

#include "../common.cuh"

namespace omcuda {

struct EpiParams {
  int64_t M, N, K;
  const void *a_zp;
  int a_zp_len; // 0, 1, or M
  int a_signed;
  const void *b_zp;
  int b_zp_len; // 0, 1, or N
  int b_signed;
  const int32_t *colsum; // [N]
  const int32_t *rowsum; // [M], needed when b_zp_len != 0
  int kind;              // omcudaEpilogue
  void *Y;
  const float *sa;
  const float *sb;
  int sb_len;
  int form;
  const float *bias;
  int gelu;
  int32_t y_zp;
  const float *residual; // f32 [M,N] added after the DEQUANT tail, or nullptr
  int res_vec_ok;        // residual rows take 16-byte loads
  uint32_t *out_range; // ordered-uint {min,max} or nullptr
  const uint32_t *q_range; // DEQUANT_QUANT: range the quantize parameters come from
  float *q_params;         // DEQUANT_QUANT: {scale, zero point as float} out
  float *q_scale;          // optional y_scale out
  uint8_t *q_zp;           // optional y_zero_point out
  int vec_ok;    // per-column vectors are 16-byte aligned: 128-bit loads allowed
  int line_store; // set by the tensor-core launcher: Y takes 16-byte line stores
  // L2 eviction hints of the tensor-core kernels' TMA copies: bit 0 output
  // stores evict_first, bit 1 A loads evict_first, bit 2 B loads evict_last.
  int l2_hints;
  int quant_mode; // OMCUDA_MODE_* flags for the quantizing tail
  // Split-K pass of the tensor-core kernels: a work unit is one of split_k
  // slices of a tile's K loop and stores its raw sums (EPI_I32 without zero
  // points) into rows [slice * ws_rows, slice * ws_rows + M) of a workspace;
  // splitk_reduce_kernel adds the slices and runs the real tail.  1: off.
  int split_k;
  int64_t ws_rows;
};

// Host: flattens the public argument block (gemm_simt.cu).
EpiParams make_epi_params(const omcudaGemmArgs &a);

// The tails that start with the DEQUANT arithmetic.
__host__ __device__ constexpr bool epi_is_dequant(int kind) {
  return kind == OMCUDA_EPI_DEQUANT || kind == OMCUDA_EPI_DEQUANT_SPLIT ||
         kind == OMCUDA_EPI_DEQUANT_RANGE || kind == OMCUDA_EPI_DEQUANT_QUANT;
}

#ifdef __CUDACC__
__device__ __forceinline__ int32_t load_zp8(
    const void *p, int64_t i, int is_signed) {
  return is_signed ? (int32_t) reinterpret_cast<const int8_t *>(p)[i]
                   : (int32_t) reinterpret_cast<const uint8_t *>(p)[i];
}

// Values that are fixed for one output row.
struct EpiRow {
  int32_t az;
  int32_t rs;
};

__device__ __forceinline__ EpiRow epi_row(const EpiParams &p, int64_t m) {
  EpiRow r;
  r.az = 0;
  r.rs = 0;
  if (p.a_zp_len == 1)
    r.az = load_zp8(p.a_zp, 0, p.a_signed);
  else if (p.a_zp_len > 1)
    r.az = load_zp8(p.a_zp, m, p.a_signed);
  if (p.b_zp_len != 0)
    r.rs = __ldg(p.rowsum + m);
  return r;
}

// Values that are fixed for one thread (scalars of the fp32 tails).
struct EpiScalars {
  float sa;
  float s0;
};

__device__ __forceinline__ EpiScalars epi_scalars(const EpiParams &p) {
  EpiScalars s;
  s.sa = 1.0f;
  s.s0 = 1.0f;
  if (epi_is_dequant(p.kind)) {
    s.sa = __ldg(p.sa);
    if (p.sb_len == 1)
      s.s0 = __fmul_rn(s.sa, __ldg(p.sb)); // onnx.Mul of the two scalars
  } else if (p.kind == OMCUDA_EPI_REQUANT) {
    if (p.sb_len == 1)
      s.s0 = __ldg(p.sb);
  }
  return s;
}

__device__ __forceinline__ int32_t epi_int(
    const EpiParams &p, const EpiRow &r, int32_t acc, int64_t n) {
  uint32_t v = (uint32_t)acc;
  if (p.a_zp_len != 0)
    v -= (uint32_t)r.az * (uint32_t)__ldg(p.colsum + n);
  if (p.b_zp_len != 0) {
    int32_t bz = load_zp8(p.b_zp, p.b_zp_len == 1 ? 0 : n, p.b_signed);
    v -= (uint32_t)bz * (uint32_t)r.rs;
    v += (uint32_t)p.K * (uint32_t)r.az * (uint32_t)bz;
  }
  return (int32_t)v;
}

__device__ __forceinline__ float epi_dequant(const EpiParams &p,
    const EpiScalars &s, int32_t v, int64_t n) {
  float f = __int2float_rn(v); // arith.sitofp
  float y;
  if (p.form == 0) {
    float sc = (p.sb_len == 1) ? s.s0 : __fmul_rn(s.sa, __ldg(p.sb + n));
    y = __fmul_rn(f, sc);
  } else {
    float sb = (p.sb_len == 1) ? __ldg(p.sb) : __ldg(p.sb + n);
    y = __fmul_rn(__fmul_rn(f, s.sa), sb);
  }
  if (p.bias)
    y = __fadd_rn(y, __ldg(p.bias + n));
  if (p.gelu)
    y = gelu_erf(y);
  return y;
}

__device__ __forceinline__ uint32_t epi_requant(const EpiParams &p,
    const EpiScalars &s, int32_t v, int64_t n) {
  float f = __int2float_rn(v);
  float sc = (p.sb_len == 1) ? s.s0 : __ldg(p.sb + n);
  float r = round_even(__fmul_rn(f, sc));
  uint32_t t = (uint32_t)__float2int_rz(r) + (uint32_t)p.y_zp;
  return t & 0xffu; // arith.trunci to 8 bits: wraps, does not saturate
}

// Folds a thread's {min,max} of the fp32 outputs into the running range.
__device__ __forceinline__ void epi_range_commit(
    uint32_t *range, float lo, float hi) {
  range_commit_warp(range, lo, hi);
}

#endif // __CUDACC__

} // namespace omcuda
