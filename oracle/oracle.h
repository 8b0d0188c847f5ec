/*
 * CPU oracle for the quantized-linear path of onnx-mlir.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the arithmetic
 * that onnx-mlir's ONNX->Krnl lowering emits for DynamicQuantizeLinear,
 * QuantizeLinear, MatMulInteger, QLinearMatMul, DequantizeLinear, the
 * Cast/Mul/Add dequantization tail and the fp32 ops of a BERT-shaped encoder.
 * It exists to check the CUDA library and to time a CPU baseline; nothing in
 * the product links, imports or executes it.
 *
 * Parity pinning: the restatement is checked against the known-answer vectors
 * held by the reference's own lit tests (test/mlir/onnx/onnx_constprop.mlir,
 * MatMulInteger and Round cases) and against golden vectors produced by
 * interpreting the IR the reference's lowering tests expect
 * (test/mlir/conversion/onnx_to_krnl/{Quantization,Math}/..._with_canonicalize.mlir).
 * The ONNX backend node-test data the reference also uses is not shipped with
 * the reference tree, so those vectors are not covered.
 *
 * Every function names the reference file:line whose semantics it follows
 * (paths relative to the onnx-mlir source tree).
 */
#ifndef OMCUDA_ORACLE_H
#define OMCUDA_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar building blocks -------------------------------------------- */

/* src/Dialect/Mlir/DialectBuilder.cpp:291-335 (roundEvenEmulation). */
float orc_round_even(float x);

/* ---- DynamicQuantizeLinear / QuantizeLinear ------------------------------ */

/* src/Conversion/ONNXToKrnl/Math/Reduction.cpp:191-260,394-548: whole-tensor
 * min and max with minnum/maxnum combine and +inf/-inf identities. */
/* Non-default arithmetic modes of the reference (see oracle.c); 0 = default. */
#define ORC_MODE_NO_ZERO_POINT 1
#define ORC_MODE_FAST_MATH 2
void orc_set_quant_mode(int flags);
void orc_minmax_f32(const float *x, int64_t n, float *mn, float *mx);

/* src/Conversion/ONNXToKrnl/Quantization/DynamicQuantizeLinear.cpp:43-84. */
void orc_dql_params(float mn, float mx, float *scale, float *zp_f, uint8_t *zp);

/* src/Conversion/ONNXToKrnl/Quantization/QuantizeLinear.cpp:122-145, u8 output
 * (qmin 0, qmax 255). */
void orc_quantize_u8(
    const float *x, int64_t n, float scale, float zp_f, uint8_t *y);

/* Same loop with i8 output (qmin -128, qmax 127), QuantizeLinear.cpp:211-218. */
void orc_quantize_i8(
    const float *x, int64_t n, float scale, float zp_f, int8_t *y);

/* DynamicQuantizeLinear.cpp:101-158: the three steps above chained. */
void orc_dynamic_quantize_linear(
    const float *x, int64_t n, uint8_t *y, float *scale, uint8_t *zp);

/* ---- integer matmuls ----------------------------------------------------- */

/* src/Conversion/ONNXToKrnl/Math/MatMulInteger.cpp:59-90.
 * A is [M,K], B is [K,N], row-major.  a_signed / b_signed select sign- or
 * zero-extension of the 8-bit operands.  a_zp has a_zp_len elements
 * (0 = absent, 1 = scalar, M = per row); b_zp has b_zp_len (0, 1 or N).
 * Zero points share their operand's signedness.  Accumulation wraps in 32
 * bits. */
void orc_matmul_integer(const void *A, int a_signed, const void *B,
    int b_signed, int64_t M, int64_t N, int64_t K, const void *a_zp,
    int64_t a_zp_len, const void *b_zp, int64_t b_zp_len, int32_t *Y);

/* src/Conversion/ONNXToKrnl/Math/QLinearMatMul.cpp:89-138.  8-bit operands
 * (a_signed/b_signed/y_signed choose i8 or u8), fp32 scales; b_scale and b_zp
 * have b_q_len elements (1 or N).  The output wraps modulo 256 (the lowering
 * truncates i32 to i8), it does not saturate. */
void orc_qlinear_matmul(const void *A, int a_signed, float a_scale,
    int32_t a_zp, const void *B, int b_signed, const float *b_scale,
    const void *b_zp, int64_t b_q_len, float y_scale, int32_t y_zp,
    int y_signed, int64_t M, int64_t N, int64_t K, void *Y);

/* ---- dequantization ------------------------------------------------------ */

/* Cast(i32->f32), Mul, Add lowered by Math/Elementwise.cpp:477-486 (+ Mul/Add):
 * form 0: y = float(acc) * s0 + bias[n]            (s0 = x_scale*w_scale,
 *                                                   rounded by the caller)
 * form 1: y = (float(acc) * s0) * s1 + bias[n]
 * bias may be NULL.  Multiplies and adds round separately (no fma). */
void orc_dequant_tail(const int32_t *acc, int64_t M, int64_t N, float s0,
    float s1, int form, const float *bias, float *y);

/* Math/Elementwise.cpp:1438-1461: y = (float(x) - float(zp)) * scale.
 * dtype: 0 = u8, 1 = i8, 2 = i32. */
void orc_dequantize_linear(
    const void *x, int dtype, int64_t n, float scale, int32_t zp, float *y);

/* ---- fp32 ops of the encoder ---------------------------------------------- */

/* Math/Softmax.cpp:25-134, last axis: max, exp(x-max) and running sum, divide. */
void orc_softmax_lastdim(const float *x, int64_t rows, int64_t cols, float *y);

/* NN/Normalization.cpp:748-880: mean = sum(x)/n, var = sum(x*x)/n - mean*mean,
 * inv = 1/sqrt(var+eps), y = (x-mean)*inv*gamma + beta. */
void orc_layernorm(const float *x, int64_t rows, int64_t cols,
    const float *gamma, const float *beta, float eps, float *y);

/* Math/Elementwise.cpp:358-388: 0.5*x * (1 + erff(x * (1/sqrt(2)))). */
void orc_gelu(const float *x, int64_t n, float *y);

/* y = a + b, elementwise (Math/Elementwise.cpp Add). */
void orc_add(const float *a, const float *b, int64_t n, float *y);

/* Tensor/Transpose.cpp with perm (0,2,1,3): [B,S,H,D] -> [B,H,S,D]. */
void orc_transpose_0213(
    const float *x, int64_t B, int64_t S, int64_t H, int64_t D, float *y);

/* Math/MatMul.cpp:488-507 on fp32: batched C[b] = A[b] (MxK) * B[b] (KxN),
 * sequential accumulation over k, separate multiply and add. */
void orc_matmul_f32(const float *A, const float *B, int64_t batch, int64_t M,
    int64_t N, int64_t K, float *C);

/* Scaled-dot-product attention written as the op chain a BERT graph holds:
 * Q,K,V are [B,S,heads*dh]; per (b,h): scores = Q K^T, scores *= scale,
 * softmax over the last axis, ctx = P V; output [B,S,heads*dh]. */
void orc_attention(const float *Q, const float *K, const float *V, int64_t B,
    int64_t S, int64_t heads, int64_t dh, float scale, float *out);

/* One dynamic-quantized linear layer as config graphs spell it:
 * DynamicQuantizeLinear(X) -> MatMulInteger(Xq, W, x_zp, 0) -> Cast f32 ->
 * Mul(x_scale * w_scale) -> Add(bias).  W is i8 [K,N].  Optional outputs
 * (xq, acc) may be NULL. */
void orc_dyn_quant_linear(const float *X, int64_t M, int64_t K,
    const int8_t *W, int64_t N, float w_scale, const float *bias, float *Y,
    uint8_t *xq, float *x_scale, uint8_t *x_zp, int32_t *acc);

/* Post-LN BERT encoder layer built from the ops above.  Weights for one layer:
 * wq,wk,wv,wo: i8 [H,H]; w1: i8 [H,F]; w2: i8 [F,H]; scales sc[6]; biases
 * bq,bk,bv,bo [H], b1 [F], b2 [H]; ln1g,ln1b,ln2g,ln2b [H]. x,y: [B*S,H]. */
typedef struct {
  const int8_t *wq, *wk, *wv, *wo, *w1, *w2;
  float sc[6];
  const float *bq, *bk, *bv, *bo, *b1, *b2;
  const float *ln1g, *ln1b, *ln2g, *ln2b;
} orc_encoder_layer_weights;

void orc_encoder_layer(const float *x, int64_t B, int64_t S, int64_t H,
    int64_t heads, int64_t F, const orc_encoder_layer_weights *w, float eps,
    float *y);

/* ---- CPU baseline shaped like the reference's emitted loops ---------------- */

/* MatMulInteger the way -O3 lowers it (MatMulInteger.cpp:59-84 then
 * Math/MatMul.cpp:148-150,310-326 and KrnlToAffine/KrnlMatmul.cpp:534-611):
 * both operands widened into full i32 temporaries, zero point subtracted into
 * second temporaries, zero-initialised C, 4x8x8 register-tiled i32 matmul with
 * no cache blocking.  threads > 1 splits the outer row loop (--parallel). */
void orc_ref_shaped_matmul_integer(const uint8_t *A, const int8_t *B, int64_t M,
    int64_t N, int64_t K, int32_t a_zp, int32_t *Y, int threads);

int orc_max_threads(void);
/* Number of OpenMP threads later calls use (launchers such as torchrun export
 * OMP_NUM_THREADS=1; the timed CPU baseline sets the host's core count). */
void orc_set_threads(int n);

/* Exhaustive check that orc_round_even(x) == rintf(x) for every finite float
 * (signs of zero aside); returns the number of mismatches. */
int64_t orc_selftest_round_even_exhaustive(void);

#ifdef __cplusplus
}
#endif
#endif
