/*
 * libomcuda: B200 (sm_100a) implementation of onnx-mlir's quantized-linear
 * path behind the reference's own C calling conventions.
 *
 * Three groups of entry points, all plain C:
 *
 *  1. Accelerator runtime hooks, named and shaped like the in-tree NNPA
 *     accelerator's (src/Accelerators/NNPA/Runtime/OMRuntimeNNPA.c:36-250):
 *     OMIsInitAccelCUDA, OMInitAccelCUDA, OMInitCompatibleAccelCUDA,
 *     OMShutdownAccelCUDA.  The generated run_main_graph calls the
 *     "compatible" hook first (src/Conversion/KrnlToLLVM/KrnlEntryPoint.cpp:149-187).
 *
 *  2. krnl.call targets (omcuda<Op>): what the compiler plugin emits in place
 *     of the CPU loops.  Calling convention of krnl.call
 *     (src/Dialect/Krnl/Krnl.td:52-96, src/Conversion/KrnlToLLVM/KrnlCall.cpp:34-226):
 *     output tensors first, then inputs, each a non-owning `OMTensor *`
 *     (NULL for an absent optional input), then integer attributes as int64_t
 *     and float attributes as double in attribute-name order; return void;
 *     the callee neither allocates nor frees the tensors' buffers.  Buffers
 *     may live in host or device memory; host buffers are staged through HBM
 *     inside the call.  Errors are sticky per thread (see omcudaGetLastError)
 *     and set errno, the convention run_main_graph uses to report failure
 *     (src/Runtime/ExecutionSession.cpp:324-362).
 *
 *  3. Device-pointer entry points (omcudaDev<Op>): the same kernels for
 *     callers that already hold device buffers and a CUDA stream.
 *
 * There is no CPU fallback: every entry point fails with OMCUDA_ECUDA when no
 * usable GPU is present.
 */
#ifndef OMCUDA_H
#define OMCUDA_H

#include <stdint.h>

#include "omcuda_runtime_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------------- */
/* Status                                                                   */
/* ---------------------------------------------------------------------- */

typedef enum {
  OMCUDA_OK = 0,
  OMCUDA_EINVAL = 1,    /* bad argument: dtype, rank, shape, stride, NULL */
  OMCUDA_ENOMEM = 2,    /* device or host allocation failed */
  OMCUDA_ECUDA = 3,     /* CUDA runtime / driver error, or no GPU */
  OMCUDA_ETIMEDOUT = 4, /* a bounded device-side wait gave up */
  OMCUDA_ENOTSUP = 5    /* valid ONNX but outside what the kernels cover */
} omcudaStatus;

/* Sticky per-thread status of the krnl.call-level entry points: the first
 * failure is kept and later calls return without doing work until cleared.
 * Replaces nothing in the reference; run_main_graph would test it (or errno)
 * before building its output list. */
int omcudaGetLastError(void);
const char *omcudaGetLastErrorString(void);
void omcudaClearError(void);

/* ---------------------------------------------------------------------- */
/* Accelerator runtime hooks (OMRuntimeNNPA.c:36-118,156-250 pattern)       */
/* ---------------------------------------------------------------------- */

extern long OMIsInitAccelCUDA;
/* Thread-safe, idempotent: picks the device (OMCUDA_DEVICE, else LOCAL_RANK,
 * else 0), creates the library stream and the device-memory pool. */
void OMInitAccelCUDA(void);
/* Returns non-zero when the library can serve a model compiled against
 * version `versionNum` (0xMMmmpp); on failure sets errno = EPERM and returns
 * 0, as OMInitCompatibleAccelNNPA does (OMRuntimeNNPA.c:156-232). */
uint64_t OMInitCompatibleAccelCUDA(uint64_t versionNum);
void OMShutdownAccelCUDA(void);
#define OMCUDA_VERSION 0x000100u

/* ---------------------------------------------------------------------- */
/* Device-resident tensors and streams                                      */
/* ---------------------------------------------------------------------- */

/* A stock OMTensor whose buffer is device memory from the library pool.  The
 * wrapper is non-owning in the reference's sense (omTensorDestroy must not
 * free() a device pointer): release with omcudaTensorDestroy. */
OMTensor *omcudaTensorCreateOnDevice(
    const int64_t *shape, int64_t rank, OM_DATA_TYPE dtype);
/* Copies (host or device source) into a new device / owning host tensor. */
OMTensor *omcudaTensorToDevice(const OMTensor *src);
OMTensor *omcudaTensorToHost(const OMTensor *src);
/* Releases a tensor made by the three calls above (buffer and wrapper). */
void omcudaTensorDestroy(OMTensor *t);
/* 1 when the tensor's data pointer is device memory, 0 for host memory. */
int omcudaTensorIsOnDevice(const OMTensor *t);
/* Pinned host memory for fast staging of host tensors. */
void *omcudaHostAlloc(int64_t bytes);
void omcudaHostFree(void *p);
/* Raw device memory from the pool (stream-ordered reuse on the library
 * stream). */
void *omcudaDeviceAlloc(int64_t bytes);
void omcudaDeviceFree(void *p);
/* The stream krnl.call-level entry points launch on (a cudaStream_t).  A
 * caller may substitute its own for the calling thread; NULL restores the
 * library stream.  Several host threads may be inside the library at once,
 * each on the shared library stream or on a stream of its own (the
 * run_main_graph of one model may be called concurrently,
 * docs/mnist_example/README.md:117-150 of the reference): temporaries come
 * from a pool whose reuse is ordered by stream (a block freed by one stream
 * reaches another only behind an event), and a cached constant prepared on
 * one stream is waited for by the others.  One omcudaEncoder object serves
 * one run at a time. */
void *omcudaGetStream(void);
void omcudaSetStream(void *stream);
/* A new non-blocking stream on the library's device for a host thread that
 * wants its calls to run beside those of other threads (pass it to
 * omcudaSetStream), without that thread linking the CUDA runtime itself. */
void *omcudaStreamCreate(void);
void omcudaStreamDestroy(void *stream);
void omcudaSynchronize(void);
/* Declares that a tensor's buffer is a model constant (krnl.global): its
 * prepared form (K-major copy and column sums of a MatMulInteger /
 * QLinearMatMul B operand) is built once and cached until
 * omcudaForgetConstants.  Without this, B is prepared on every call. */
void omcudaRegisterConstant(const OMTensor *t);
void omcudaForgetConstants(void);
/* The reference's two non-default arithmetic modes.  They are compile-time
 * options there; the plugin passes the ones a model was compiled with once, at
 * model initialisation.  Process wide; 0 (the default) is the arithmetic
 * every other comment of this header describes.
 *   OMCUDA_MODE_NO_ZERO_POINT  --disable-quantization-zero-point:
 *       DynamicQuantizeLinear derives the scale as usual and reports zero
 *       point 0 (src/Conversion/ONNXToKrnl/Quantization/DynamicQuantizeLinear.cpp:72-83,142),
 *       QuantizeLinear and DequantizeLinear ignore a given zero point
 *       (QuantizeLinear.cpp:231-237, Math/Elementwise.cpp:1453).
 *   OMCUDA_MODE_FAST_MATH  convert-onnx-to-krnl=enable-fast-math: the
 *       quantize step multiplies by RN(1 / scale) instead of dividing by the
 *       scale (QuantizeLinear.cpp:43-44,117-131); results differ from the
 *       default in rare last-place cases, exactly as the reference's do. */
#define OMCUDA_MODE_NO_ZERO_POINT 1
#define OMCUDA_MODE_FAST_MATH 2
void omcudaSetQuantizationMode(int64_t flags);
int64_t omcudaGetQuantizationMode(void);
/* Number of kernels this library has launched in this process. */
int64_t omcudaLaunchCount(void);

/* ---------------------------------------------------------------------- */
/* Loading compiled models and their constants                              */
/* ---------------------------------------------------------------------- */

/* What onnx-mlir's ExecutionSession gives a host program
 * (src/Runtime/ExecutionSession.cpp:60-380), as a C API: open a compiled
 * model, query its entry points and signatures, run it.  The tag selects the
 * suffixed symbols a model is compiled with (run_main_graph_<tag>, ...):
 * NULL or "" means the file name without extension in lower case, "NONE" the
 * unsuffixed symbols.  OM_CONSTANT_PATH is set to the model's folder unless the
 * caller set it.  Tensors are passed through untouched, so a model compiled
 * with the CUDA accelerator can be given (and returns) device-resident
 * tensors and models can be chained without a trip through host memory.
 * omcudaSessionRun returns NULL with errno set when the model fails. */
typedef struct omcudaSession omcudaSession;
omcudaSession *omcudaSessionCreate(
    const char *sharedLibPath, const char *tag, int defaultEntryPoint);
const char *const *omcudaSessionQueryEntryPoints(
    omcudaSession *s, int64_t *numOfEntryPoints);
int omcudaSessionSetEntryPoint(omcudaSession *s, const char *entryPointName);
const char *omcudaSessionInputSignature(omcudaSession *s);
const char *omcudaSessionOutputSignature(omcudaSession *s);
OMTensorList *omcudaSessionRun(omcudaSession *s, OMTensorList *inputs);
void omcudaSessionDestroy(omcudaSession *s);

/* The external-constants loader a compiled model calls for its
 * <model>.constants.bin (replaces omLoadConstantData / omUnloadConstantData,
 * src/Runtime/OMExternalConstant.c:57-138,176-189): the file is looked up in
 * OM_CONSTANT_PATH and mapped read-only; constAddr[0] receives its address (a
 * second call is a no-op).  Returns an omcudaStatus. */
int omcudaLoadConstantData(
    void **constAddr, const char *fname, int64_t size, int64_t isLE);
int omcudaUnloadConstantData(void **constAddr, int64_t size);

/* ---------------------------------------------------------------------- */
/* krnl.call targets                                                        */
/* ---------------------------------------------------------------------- */

/* Replaces ONNXDynamicQuantizeLinearOpLowering
 * (src/Conversion/ONNXToKrnl/Quantization/DynamicQuantizeLinear.cpp:101-158).
 * x: f32 any rank; y: u8 same shape; yScale: f32 rank 0; yZp: u8 rank 0. */
void omcudaDynamicQuantizeLinear(
    OMTensor *y, OMTensor *yScale, OMTensor *yZp, const OMTensor *x);

/* Replaces ONNXQuantizeLinearOpLowering (QuantizeLinear.cpp:155-246):
 * per-tensor scale, u8 or i8 output chosen by y's dtype; zp may be NULL. */
void omcudaQuantizeLinear(OMTensor *y, const OMTensor *x,
    const OMTensor *scale, const OMTensor *zp);

/* Replaces ONNXMatMulIntegerOpLowering
 * (src/Conversion/ONNXToKrnl/Math/MatMulInteger.cpp:32-92) and the i32
 * onnx.MatMul it creates.  A: u8/i8 [..,M,K]; B: u8/i8 [K,N]; Y: i32
 * [..,M,N]; aZp: NULL, scalar, [1] or [M]; bZp: NULL, scalar, [1] or [N]. */
void omcudaMatMulInteger(OMTensor *Y, const OMTensor *A, const OMTensor *B,
    const OMTensor *aZp, const OMTensor *bZp);

/* Replaces ONNXQLinearMatMulOpLowering
 * (src/Conversion/ONNXToKrnl/Math/QLinearMatMul.cpp:32-142), including its
 * wrap-around (not saturating) conversion of the result to 8 bits. */
void omcudaQLinearMatMul(OMTensor *y, const OMTensor *a, const OMTensor *aScale,
    const OMTensor *aZp, const OMTensor *b, const OMTensor *bScale,
    const OMTensor *bZp, const OMTensor *yScale, const OMTensor *yZp);

/* Replaces the scalar body of ONNXDequantizeLinearOp
 * (src/Conversion/ONNXToKrnl/Math/Elementwise.cpp:1438-1461), per-tensor. */
void omcudaDequantizeLinear(OMTensor *y, const OMTensor *x,
    const OMTensor *scale, const OMTensor *zp);

/* The fused subgraph DynamicQuantizeLinear -> MatMulInteger -> Cast(f32) ->
 * Mul -> [Mul] -> [Add], i.e. the pattern the NNPA plugin matches in
 * src/Accelerators/NNPA/Conversion/ONNXToZHigh/ONNXToZHigh.cpp:895-1215,
 * replacing the four CPU lowerings it spans.  X: f32 [..,K]; Wq: i8/u8 [K,N];
 * wScale: f32 scalar or [N]; wZp: NULL or matching Wq; bias: NULL or f32 [N].
 * scaleForm 0: Y = f32(acc) * (x_scale * w_scale) + bias
 * scaleForm 1: Y = (f32(acc) * x_scale) * w_scale + bias */
void omcudaDynQuantLinear(OMTensor *Y, const OMTensor *X, const OMTensor *Wq,
    const OMTensor *wScale, const OMTensor *wZp, const OMTensor *bias,
    int64_t scaleForm);

/* fp32 ops a quantized encoder graph holds between its linears. */
/* src/Conversion/ONNXToKrnl/Math/Softmax.cpp:268-312 (axis = last). */
void omcudaSoftmax(OMTensor *y, const OMTensor *x, int64_t axis);
/* src/Conversion/ONNXToKrnl/NN/Normalization.cpp:342-406,748-880 (axis = last);
 * bias may be NULL. */
void omcudaLayerNormalization(OMTensor *y, const OMTensor *x,
    const OMTensor *scale, const OMTensor *bias, int64_t axis, double epsilon);
/* src/Conversion/ONNXToKrnl/Math/Elementwise.cpp:358-388 (approximate=none). */
void omcudaGelu(OMTensor *y, const OMTensor *x);
/* Elementwise Add with equal shapes (Math/Elementwise.cpp). */
void omcudaAdd(OMTensor *y, const OMTensor *a, const OMTensor *b);
/* src/Conversion/ONNXToKrnl/Tensor/Transpose.cpp, perm (0,2,1,3) on rank 4. */
void omcudaTranspose0213(OMTensor *y, const OMTensor *x);
/* Batched fp32 onnx.MatMul, equal batch dims
 * (src/Conversion/ONNXToKrnl/Math/MatMul.cpp:488-507). */
void omcudaMatMulF32(OMTensor *y, const OMTensor *a, const OMTensor *b);
/* The attention subgraph of the encoder configs as one call: q,k,v,y are f32
 * [B,S,heads*dh]; scores = QK^T * scale, softmax over keys, times V. */
void omcudaAttention(OMTensor *y, const OMTensor *q, const OMTensor *k,
    const OMTensor *v, int64_t heads, double scale);

/* ---------------------------------------------------------------------- */
/* Device-pointer entry points                                              */
/* ---------------------------------------------------------------------- */

/* Bytes of scratch omcudaDevDynamicQuantizeLinear needs for n elements. */
int64_t omcudaDevDqlScratchBytes(int64_t n);
/* DynamicQuantizeLinear on device buffers.  scratch: device memory of at
 * least omcudaDevDqlScratchBytes(n) whose first 64 bytes are zero before the
 * first use (the kernel leaves them zeroed); calls that overlap on the GPU
 * need a scratch block each. */
int omcudaDevDynamicQuantizeLinear(const float *x, int64_t n, uint8_t *y,
    float *y_scale, uint8_t *y_zp, void *scratch, void *stream);
/* DynamicQuantizeLinear for callers that cannot allocate device memory (a
 * host whose HBM is entirely owned by its own arena, a loop that cannot
 * afford the synchronisation cudaMalloc implies, a process whose allocation
 * calls are refused).  Has no counterpart in the reference.  Same results as
 * omcudaDevDynamicQuantizeLinear, but the reduction's scratch is a fixed
 * 32 KiB array inside the library image (held on every GPU that loads the
 * library until the process exits), and the call performs no cudaMalloc,
 * cudaFree or other allocating call.  Limits and rules:
 *  - n may not exceed OMCUDA_DQL_NOALLOC_MAX_ELEMS; larger inputs are rejected
 *    with OMCUDA_EINVAL and nothing is launched.
 *  - The first call on each device looks up the array's device address
 *    (with that device current); make that first call before any stream
 *    capture begins.
 *  - All calls on a device share the one array, which keeps the previous
 *    call's contents; the entry point re-zeroes the part that must start at
 *    zero.  Two calls whose kernels overlap on the GPU (different streams,
 *    no ordering between them) race on it: order them. */
#define OMCUDA_DQL_NOALLOC_MAX_ELEMS ((int64_t)1 << 31)
int omcudaDevDynamicQuantizeLinearNoAlloc(const float *x, int64_t n, uint8_t *y,
    float *y_scale, uint8_t *y_zp, void *stream);
/* Quantize with given device scalars (scale f32; zp as 8-bit of y's type or
 * NULL). */
int omcudaDevQuantizeLinear(const float *x, int64_t n, void *y, int y_signed,
    const float *scale, const void *zp, void *stream);

/* A B operand prepared for the tensor-core GEMM: K-major copy Bt[N][Kp] and
 * column sums of B as i32. */
typedef struct {
  void *bt;        /* device, N * kp bytes */
  int32_t *colsum; /* device, N entries: sum over k of B[k][n] (widened) */
  int64_t K, N, kp;
  int b_signed;
} omcudaPreparedB;
int64_t omcudaDevPreparedBBytes(int64_t K, int64_t N, int64_t *kp);
int omcudaDevPrepareB(const void *B, int b_signed, int64_t K, int64_t N,
    omcudaPreparedB *out /* bt, colsum preallocated */, void *stream);

typedef enum {
  OMCUDA_EPI_I32 = 0,     /* MatMulInteger: i32 out */
  OMCUDA_EPI_DEQUANT = 1, /* Cast f32, Mul scale(s), Add bias [, Gelu] */
  OMCUDA_EPI_REQUANT = 2, /* QLinearMatMul: scale, round, +zp, wrap to 8 bit */
  /* The DEQUANT value x (without Gelu) stored as two bf16 planes instead of
   * f32: Y holds hi = bf16(x) as [M,N] bf16, followed by lo = bf16(x - hi) as
   * [M,N] bf16 (2*M*N*2 bytes in all): the operand format of
   * omcudaDevAttentionBf16.  Tensor-core kernel only. */
  OMCUDA_EPI_DEQUANT_SPLIT = 3,
  /* The two halves of "linear tail -> DynamicQuantizeLinear" without the f32
   * tensor in between (tensor-core kernel only).  DEQUANT_RANGE computes the
   * DEQUANT values, folds them into out_minmax and stores nothing (Y may be
   * NULL).  DEQUANT_QUANT computes the same values again and stores them as
   * uint8 [M,N], quantized with the scale and zero point that
   * DynamicQuantizeLinear derives from the range in q_range
   * (DynamicQuantizeLinear.cpp:43-84, QuantizeLinear.cpp:122-145); it leaves
   * those scalars where q_params / q_scale / q_zp point. */
  OMCUDA_EPI_DEQUANT_RANGE = 4,
  OMCUDA_EPI_DEQUANT_QUANT = 5
} omcudaEpilogue;

typedef struct {
  int64_t M, N, K;
  const void *A; /* device [M,K] row-major 8-bit */
  int a_signed;
  omcudaPreparedB B;
  /* Zero points, device pointers to 8-bit values of the operand's type. */
  const void *a_zp;
  int64_t a_zp_len; /* 0, 1 or M */
  const void *b_zp;
  int64_t b_zp_len; /* 0, 1 or N */
  /* Row sums of A (i32 [M]); required only when b_zp_len != 0. */
  const int32_t *a_rowsum;
  int epilogue; /* omcudaEpilogue */
  void *Y;      /* i32 / f32 / 8-bit [M,N] */
  /* DEQUANT: sa = device scalar (x_scale), sb = device w_scale (len 1 or N),
   * form as in omcudaDynQuantLinear; bias device [N] or NULL; gelu flag.
   * REQUANT: sb = device S[n] (len 1 or N) = (a_scale*b_scale[n])/y_scale,
   * y_zp as int in the output type's domain, y_signed. */
  const float *sa;
  const float *sb;
  int64_t sb_len;
  int scale_form;
  const float *bias;
  int gelu;
  int32_t y_zp;
  int y_signed;
  /* Optional running range (omcudaDevRangeInit) of the f32 outputs, for a
   * following DynamicQuantizeLinear. May be NULL. */
  void *out_minmax;
  /* 0 = choose (GEMV-shaped kernels up to 16 rows; tcgen05 above, with a
   * split-K pass through a pool workspace for up to 512 rows, K >= 8192 and
   * few tiles -- not inside a stream capture; the SIMT kernels when K is not
   * a multiple of 16 or A is not 16-byte aligned); 1 = force the tcgen05
   * kernels; 2 = force the SIMT (dp4a / mma.sync) kernels.  Every choice
   * gives the same bytes. */
  int kernel_choice;
  /* DEQUANT only: optional f32 [M,N] added last (y = tail(acc) + residual),
   * the onnx.Add of a residual connection around the linear
   * (Math/Elementwise.cpp, one more separately rounded fp32 add). May be
   * NULL. */
  const float *residual;
  /* DEQUANT_QUANT only: q_range = running range (omcudaDevRangeInit layout)
   * of the values about to be quantized; q_params (2 floats: scale, zero
   * point as float) is required, q_scale (y_scale) and q_zp (y_zero_point as
   * uint8) may be NULL.  All device pointers. */
  const void *q_range;
  float *q_params;
  float *q_scale;
  uint8_t *q_zp;
} omcudaGemmArgs;

int omcudaDevGemmI8(const omcudaGemmArgs *args, void *stream);

/* Bounded device-side waits.  Every wait of the tensor-core kernels (int8
 * GEMM, bf16 attention) on an mbarrier gives up after a limit -- two seconds
 * without progress of that wait unless changed here (ns <= 0 restores the
 * default) -- after which the CTA frees its tensor memory, raises a per-device
 * status word and returns; nothing traps or spins without a limit.  The word
 * is read (and cleared) by omcudaSynchronize, by every krnl.call-level entry
 * point that returns host results, by omcudaTensorToHost and by
 * omcudaEncoderWait, which then report OMCUDA_ETIMEDOUT (errno ETIMEDOUT).  A
 * caller of the omcudaDev* entry points that synchronises its own stream must
 * call omcudaSynchronize (on a thread whose stream it set with omcudaSetStream)
 * to learn of a timeout.  Has no counterpart in the reference, whose CPU loops
 * cannot wait on anything. */
void omcudaDevSetWaitLimitNs(int64_t ns);
/* Self test of that path: launches one CTA that allocates tensor memory and
 * waits, with the configured limit (capped at one second), on a barrier that
 * nothing signals.  The kernel returns by itself; afterwards the status word
 * is raised, so the next omcudaSynchronize reports OMCUDA_ETIMEDOUT, and
 * tensor memory is free again.  waited_ns (device pointer, may be NULL)
 * receives how long the wait lasted. */
int omcudaDevSelfTestBoundedWait(uint64_t *waited_ns, void *stream);

/* S[n] = (a_scale * b_scale[n]) / y_scale on device
 * (QLinearMatMul.cpp:127). */
int omcudaDevRequantScale(const float *a_scale, const float *b_scale,
    int64_t len, const float *y_scale, float *S, void *stream);
/* Row sums of an 8-bit [M,K] matrix as i32. */
int omcudaDevRowSum(const void *A, int a_signed, int64_t M, int64_t K,
    int32_t *rowsum, void *stream);

int omcudaDevDequantizeLinear(const void *x, int dtype /*0 u8,1 i8,2 i32*/,
    int64_t n, const float *scale, const void *zp, float *y, void *stream);
int omcudaDevSoftmax(
    const float *x, int64_t rows, int64_t cols, float *y, void *stream);
/* y = LayerNorm(x [+ residual]); out_minmax: optional running range of y. */
int omcudaDevLayerNorm(const float *x, const float *residual, int64_t rows,
    int64_t cols, const float *gamma, const float *beta, float eps, float *y,
    void *out_minmax, void *stream);
int omcudaDevGelu(const float *x, int64_t n, float *y, void *stream);
int omcudaDevAdd(
    const float *a, const float *b, int64_t n, float *y, void *stream);
int omcudaDevTranspose0213(const float *x, int64_t B, int64_t S, int64_t H,
    int64_t D, float *y, void *stream);
int omcudaDevMatMulF32(const float *A, const float *B, int64_t batch,
    int64_t M, int64_t N, int64_t K, float *C, void *stream);
int omcudaDevAttention(const float *Q, const float *K, const float *V,
    int64_t B, int64_t S, int64_t heads, int64_t dh, float scale, float *out,
    void *stream);
/* Same with explicit row pitches (in floats) of Q/K/V and of out, so that a
 * fused [T,3H] QKV buffer can be read in place, and an optional running range
 * of the outputs (see omcudaDevRangeInit). */
int omcudaDevAttentionEx(const float *Q, const float *K, const float *V,
    int64_t B, int64_t S, int64_t heads, int64_t dh, float scale, float *out,
    int64_t ld_in, int64_t ld_out, void *out_range, void *stream);

/* The same attention on the tcgen05 tensor cores, for head size 64 and a
 * sequence length that is a multiple of 128, over operands already split into
 * two bf16 planes: hi = bf16(a), lo = bf16(a - hi), each [B*S, ld_planes]
 * row-major; head h of Q / K / V owns columns [q_col + 64 h, ...), [k_col + 64 h,
 * ...), [v_col + 64 h, ...) of its row.  omcudaDevSplitBf16 makes the planes
 * from an fp32 matrix (columns [col0, col0 + cols) of the planes); the QKV
 * projection's GEMM can write them directly (OMCUDA_EPI_DEQUANT_SPLIT).
 * These are the two fp32 MatMuls, the Mul and the Softmax of the graph
 * (Math/MatMul.cpp:488-507, Math/Softmax.cpp:25-134) in one kernel. */
int omcudaDevSplitBf16(const float *x, int64_t rows, int64_t cols, int64_t ld_x,
    void *hi, void *lo, int64_t ld_planes, int64_t col0, void *stream);
int omcudaDevAttentionBf16Supported(int64_t B, int64_t S, int64_t heads,
    int64_t dh, int64_t ld_planes, int64_t ld_out);
int omcudaDevAttentionBf16(const void *hi, const void *lo, int64_t ld_planes,
    int64_t q_col, int64_t k_col, int64_t v_col, int64_t B, int64_t S,
    int64_t heads, int64_t dh, float scale, float *out, int64_t ld_out,
    void *out_range, void *stream);

/* Running {min,max} ranges: 8 bytes each, kept by producer kernels (GEMM
 * dequant epilogue, LayerNorm, attention) with integer atomics so that the
 * DynamicQuantizeLinear that follows does not need its own reduction pass.
 * omcudaDevRangeInit arms `count` ranges; omcudaDevQuantizeFromRange derives
 * scale / zero point from one (exactly as DynamicQuantizeLinear.cpp:43-84
 * does from the reduced min/max), writes them to params / y_scale / y_zp and
 * quantizes x, in one launch.  The range is left as it is: arm it again
 * before its producer runs a second time. */
int omcudaDevRangeInit(void *ranges, int64_t count, void *stream);
/* Folds the min / max of x into an armed range (for a tensor that no kernel of
 * the library produced). */
int omcudaDevRangeFold(const float *x, int64_t n, void *range, void *stream);
int omcudaDevQuantizeFromRange(const float *x, int64_t n, void *range,
    uint8_t *y, float *params /* 2 floats */, float *y_scale, uint8_t *y_zp,
    void *stream);

/* ---------------------------------------------------------------------- */
/* Encoder model harness                                                    */
/* ---------------------------------------------------------------------- */

/* Plays the part of the run_main_graph a compiled dynamic-quantized encoder
 * model would export (src/Conversion/KrnlToLLVM/KrnlEntryPoint.cpp:236-338):
 * unpack the input list, run the graph's ops in order through this library
 * with every intermediate resident in HBM, pack the output list.  The graph is
 * the post-LayerNorm BERT-shaped layer of the benchmark configurations:
 *   q,k,v = DynQuantLinear(x);  ctx = softmax(q k^T / sqrt(dh)) v
 *   h1 = LayerNorm(x + DynQuantLinear(ctx))
 *   y  = LayerNorm(h1 + DynQuantLinear(Gelu(DynQuantLinear(h1))))
 * where DynQuantLinear = DynamicQuantizeLinear -> MatMulInteger -> Cast ->
 * Mul(x_scale * w_scale) -> Add(bias), weights int8 [in,out], per-tensor
 * symmetric. */
typedef struct omcudaEncoder omcudaEncoder;
typedef struct {
  int64_t layers, hidden, heads, ffn;
  double epsilon;
} omcudaEncoderConfig;
typedef struct {
  const OMTensor *wq, *wk, *wv, *wo, *w1, *w2; /* int8 [in,out] */
  float w_scale[6];                            /* same order */
  const OMTensor *bq, *bk, *bv, *bo, *b1, *b2; /* f32 biases */
  const OMTensor *ln1_gamma, *ln1_beta, *ln2_gamma, *ln2_beta;
} omcudaEncoderLayerWeights;

omcudaEncoder *omcudaEncoderCreate(const omcudaEncoderConfig *cfg);
/* Uploads one layer's constants (host or device tensors) and prepares the
 * GEMM operands; the model-initialisation step of a compiled model. */
int omcudaEncoderSetLayer(
    omcudaEncoder *enc, int64_t layer, const omcudaEncoderLayerWeights *w);
/* run_main_graph: one f32 input [batch, seq, hidden] (host or device), one f32
 * output of the same shape and on the same side.  Returns NULL and sets errno
 * on failure. */
OMTensorList *omcudaEncoderRun(omcudaEncoder *enc, OMTensorList *inputs);
/* The same with the output tensor supplied by the caller, as a krnl.call
 * callee receives it (outputs first, preallocated; src/Dialect/Krnl/Krnl.td:52-96):
 * x and y are f32 [batch, seq, hidden], each in host or device memory.  Host
 * tensors are staged through HBM buffers the encoder keeps; give pinned host
 * memory (omcudaHostAlloc) for full-speed copies.  Returns when y is complete
 * (host y) or with the work queued on the calling thread's stream (device y). */
int omcudaEncoderRunInto(omcudaEncoder *enc, OMTensor *y, const OMTensor *x);
/* The same for host tensors as a pipeline: Submit queues "copy x in, run, copy
 * y out" and returns; the copy-in of a call overlaps the run of the call
 * before it and its copy-out the run of the call after it (separate copy
 * streams, two sets of staging buffers).  At most two calls are in flight: a
 * third Submit first waits for the oldest.  x must stay unchanged and y is
 * complete only after omcudaEncoderWait, which waits for every submitted
 * call and reports any error.  Give pinned host memory (omcudaHostAlloc);
 * pageable memory makes the copies synchronous.  Every call computes exactly
 * what omcudaEncoderRunInto computes. */
int omcudaEncoderSubmit(omcudaEncoder *enc, OMTensor *y, const OMTensor *x);
int omcudaEncoderWait(omcudaEncoder *enc);
/* Device-pointer form: x, y are device f32 [batch*seq, hidden].  An encoder
 * object owns one workspace: its runs are ordered by the caller (one host
 * thread at a time, runs on different streams ordered against each other);
 * use one encoder per concurrent stream.  From the third run with the same
 * (x, y, batch, seq, stream) on, the run is one CUDA-graph launch of the
 * sequence captured on the second (OMCUDA_ENCODER_GRAPH=0 switches that off;
 * a run on a stream that is itself being captured joins that capture). */
int omcudaEncoderRunDev(omcudaEncoder *enc, const float *x, int64_t batch,
    int64_t seq, float *y, void *stream);
/* Optional: bracket every int8 GEMM launch of later runs with CUDA events on
 * the run's stream; omcudaEncoderGemmStats returns their summed duration, the
 * 2*M*N*K they cover and their count since profiling was switched on. */
void omcudaEncoderSetProfiling(omcudaEncoder *enc, int on);
int omcudaEncoderGemmStats(
    omcudaEncoder *enc, double *ms_total, double *ops_total, int64_t *launches);
/* Global quantization ranges for a batch that is sharded over several GPUs.
 * DynamicQuantizeLinear is per tensor: its scale and zero point depend on every
 * row of the activation (DynamicQuantizeLinear.cpp:136-145 reduces over the
 * flattened tensor).  By default each rank quantizes with the range of its own
 * rows, so a rank's result equals the reference's on that rank's rows.  With a
 * hook set, the harness calls it once per DynamicQuantizeLinear of the graph
 * (4 per layer + 1), after the range of the local rows is complete and before
 * it is used: `range` is device memory holding two uint32, order-preserving
 * encodings (larger encoding = larger float) of the running minimum and
 * maximum; the callee must replace them, in `stream` order, by the minimum of
 * [0] and the maximum of [1] over all ranks (a 2-word all-reduce).  The
 * sharded run then equals the reference's run on the whole batch bit for bit.
 * No counterpart in the reference, which has no multi-device support. */
typedef void (*omcudaRangeSyncFn)(void *ctx, void *range, void *stream);
int omcudaEncoderSetRangeSync(omcudaEncoder *enc, omcudaRangeSyncFn fn, void *ctx);

/* Parity-test tap (no counterpart in the reference, which is inspected with
 * its own instrumentation passes instead): while a tap buffer is set, every
 * run also copies each layer's intermediates into it, so that a test can feed
 * the library's own input of every op to a checker and compare op by op
 * instead of through the free-running chain.  Per layer l, at byte offset
 * l * layer_stride + field: x (the layer input, f32 [T,H]) and xq_x (its
 * uint8 quantization), ctx / xq_ctx (attention output), h1 / xq_h1 (first
 * LayerNorm), f / xq_f (Gelu output, f32 / uint8 [T,F]) and y (the layer
 * output); after the last layer, at `params`, 4 floats per quantize site
 * (4 per layer in the order x, ctx, h1, f): scale, zero point as float, scale
 * again as the op's y_scale output, and the zero point as uint8 in the first
 * byte of the fourth word.  The buffer is device memory of at least `total`
 * bytes for the batch and sequence length of the run; NULL switches the tap
 * off.  The copies are ordered on the run's stream. */
typedef struct {
  int64_t x, xq_x, ctx, xq_ctx, h1, xq_h1, f, xq_f, y;
  int64_t layer_stride, params, total;
} omcudaEncoderTapLayout;
int omcudaEncoderGetTapLayout(const omcudaEncoder *enc, int64_t batch,
    int64_t seq, omcudaEncoderTapLayout *out);
int omcudaEncoderSetTap(omcudaEncoder *enc, void *dev_buf, int64_t bytes);
void omcudaEncoderDestroy(omcudaEncoder *enc);

#ifdef __cplusplus
}
#endif
#endif
