/*
 * Source of a compiled model for the CUDA accelerator, specialised by the
 * macros the model builder (omcuda/model_builder.py) puts in front of it.
 *
 * It is what onnx-mlir emits for a graph whose ops all became krnl.call into
 * libomcuda, written as C instead of LLVM IR (the compiler itself cannot be
 * built without LLVM/MLIR): the same exported symbols -- run_main_graph,
 * omQueryEntryPoints, omInputSignature, omOutputSignature, each also with the
 * model's tag as suffix (src/Conversion/KrnlToLLVM/KrnlEntryPoint.cpp:236-338,
 * include/onnx-mlir/Runtime/OMEntryPoint.h, OMSignature.h) --, the same
 * checks on the inputs (element type, rank, static dimensions,
 * KrnlEntryPoint.cpp:430-545), the accelerator initialisation call
 * (KrnlEntryPoint.cpp:149-187), constants in an external <name>.constants.bin
 * that is loaded when the library is loaded and released when it is unloaded
 * (src/Runtime/OMExternalConstant.c:57-189), and NULL + errno on failure.
 *
 * Macros:
 *   OM_TAG               model tag (symbol suffix), e.g. model
 *   OM_KIND              1 dynamic-quantized linear (one omcudaDynQuantLinear),
 *                        2 QLinearMatMul, 3 BERT-shaped encoder
 *   OM_CONST_FILE        "<name>.constants.bin", OM_CONST_BYTES its size
 *   OM_IN_SIG, OM_OUT_SIG  signatures, JSON as onnx-mlir prints them
 *   kind 1: OM_K, OM_N, OM_W_OFF, OM_WSCALE_OFF, OM_BIAS_OFF (-1: none), OM_SCALE_FORM
 *   kind 2: OM_K, OM_N and offsets OM_B_OFF, OM_BSCALE_OFF, OM_BZP_OFF, OM_BQ_LEN,
 *           scalars OM_A_SCALE, OM_A_ZP, OM_Y_SCALE, OM_Y_ZP
 *   kind 3: OM_LAYERS, OM_HIDDEN, OM_HEADS, OM_FFN, OM_EPS and OM_LAYER_STRIDE,
 *           per-layer offsets relative to the layer's block (see the builder)
 */
#include <errno.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "omcuda.h"

#define OM_CAT_(a, b) a##_##b
#define OM_CAT(a, b) OM_CAT_(a, b)
#define OM_TAGGED(name) OM_CAT(name, OM_TAG)
#define OM_STR_(x) #x
#define OM_STR(x) OM_STR_(x)

static void *g_constants = NULL; /* the mapped constants file */
static pthread_once_t g_once = PTHREAD_ONCE_INIT;
static int g_init_status = -1;

static const uint8_t *cptr(int64_t off) { return (const uint8_t *)g_constants + off; }

/* The constants file is loaded by the library's constructor and unloaded by
 * its destructor, like the reference's compiled models. */
__attribute__((constructor)) static void om_load_constants(void) {
  if (omcudaLoadConstantData(&g_constants, OM_CONST_FILE, OM_CONST_BYTES, 1) != OMCUDA_OK) {
    fprintf(stderr, "model %s: %s\n", OM_STR(OM_TAG), omcudaGetLastErrorString());
    omcudaClearError();
  }
}

/* ---- entry points and signatures ---------------------------------------- */

static const char *const g_entry_points[] = {"run_main_graph_" OM_STR(OM_TAG), NULL};

const char *const *OM_TAGGED(omQueryEntryPoints)(int64_t *n) {
  if (n)
    *n = 1;
  return g_entry_points;
}
const char *const *omQueryEntryPoints(int64_t *n) { return OM_TAGGED(omQueryEntryPoints)(n); }

static int known_entry(const char *name) {
  return name && (strcmp(name, "run_main_graph_" OM_STR(OM_TAG)) == 0 ||
                     strcmp(name, "run_main_graph") == 0);
}
const char *OM_TAGGED(omInputSignature)(const char *entry) {
  return known_entry(entry) ? OM_IN_SIG : NULL;
}
const char *OM_TAGGED(omOutputSignature)(const char *entry) {
  return known_entry(entry) ? OM_OUT_SIG : NULL;
}
const char *omInputSignature(const char *entry) { return OM_TAGGED(omInputSignature)(entry); }
const char *omOutputSignature(const char *entry) { return OM_TAGGED(omOutputSignature)(entry); }

/* ---- the graph ------------------------------------------------------------ */

static OMTensor *dev_const(int64_t off, const int64_t *shape, int64_t rank, OM_DATA_TYPE dt) {
  /* krnl.global: a view of the constants file, uploaded to HBM once. */
  OMTensor *host = omTensorCreate((void *)cptr(off), shape, rank, dt);
  if (!host)
    return NULL;
  OMTensor *dev = omcudaTensorToDevice(host);
  omTensorDestroy(host);
  return dev;
}

static OMTensor *make_output(const OMTensor *like, const int64_t *shape, int64_t rank,
    OM_DATA_TYPE dt) {
  /* Results live where the inputs live: device tensors in, device tensors
   * out; host tensors get an owning host result, as a CPU model returns. */
  if (omcudaTensorIsOnDevice(like))
    return omcudaTensorCreateOnDevice(shape, rank, dt);
  return omTensorCreateEmpty(shape, rank, dt);
}

static void free_output(OMTensor *t) {
  if (!t)
    return;
  if (omcudaTensorIsOnDevice(t))
    omcudaTensorDestroy(t);
  else
    omTensorDestroy(t);
}

static int bad_input(const char *what) {
  fprintf(stderr, "model %s: wrong input: %s\n", OM_STR(OM_TAG), what);
  errno = EINVAL;
  return 1;
}

#if OM_KIND == 1
static OMTensor *g_w, *g_wscale, *g_bias;
static void om_init(void) {
  if (!g_constants)
    return;
  const int64_t wshape[2] = {OM_K, OM_N}, bshape[1] = {OM_N};
  g_w = dev_const(OM_W_OFF, wshape, 2, ONNX_TYPE_INT8);
  g_wscale = dev_const(OM_WSCALE_OFF, NULL, 0, ONNX_TYPE_FLOAT);
  g_bias = OM_BIAS_OFF >= 0 ? dev_const(OM_BIAS_OFF, bshape, 1, ONNX_TYPE_FLOAT) : NULL;
  if (!g_w || !g_wscale || (OM_BIAS_OFF >= 0 && !g_bias))
    return;
  /* the weight's K-major copy and column sums are built once and cached */
  omcudaRegisterConstant(g_w);
  g_init_status = 0;
}
static OMTensorList *om_graph(OMTensorList *inputs) {
  if (omTensorListGetSize(inputs) != 1 && bad_input("expected 1 tensor"))
    return NULL;
  const OMTensor *x = omTensorListGetOmtByIndex(inputs, 0);
  int64_t rank = omTensorGetRank(x);
  if ((omTensorGetDataType(x) != ONNX_TYPE_FLOAT || rank < 1 || rank > 8 ||
          omTensorGetShape(x)[rank - 1] != OM_K) &&
      bad_input("X must be f32 [.., " OM_STR(OM_K) "]"))
    return NULL;
  int64_t yshape[8];
  for (int64_t i = 0; i + 1 < rank; ++i)
    yshape[i] = omTensorGetShape(x)[i];
  yshape[rank - 1] = OM_N;
  OMTensor *y = make_output(x, yshape, rank, ONNX_TYPE_FLOAT);
  if (!y)
    return NULL;
  omcudaDynQuantLinear(y, x, g_w, g_wscale, NULL, g_bias, OM_SCALE_FORM);
  if (omcudaTensorIsOnDevice(y))
    omcudaSynchronize();
  if (omcudaGetLastError() != OMCUDA_OK) {
    free_output(y);
    return NULL;
  }
  OMTensor *arr[1] = {y};
  return omTensorListCreate(arr, 1);
}
#elif OM_KIND == 2
static OMTensor *g_b, *g_bscale, *g_bzp, *g_ascale, *g_azp, *g_yscale, *g_yzp;
static OMTensor *scalar_f32(float v) {
  OMTensor *t = omTensorCreateEmpty(NULL, 0, ONNX_TYPE_FLOAT);
  if (t)
    *(float *)omTensorGetDataPtr(t) = v;
  return t;
}
static OMTensor *scalar_u8(uint8_t v) {
  OMTensor *t = omTensorCreateEmpty(NULL, 0, ONNX_TYPE_UINT8);
  if (t)
    *(uint8_t *)omTensorGetDataPtr(t) = v;
  return t;
}
static void om_init(void) {
  if (!g_constants)
    return;
  const int64_t bshape[2] = {OM_K, OM_N}, qshape[1] = {OM_BQ_LEN};
  g_b = dev_const(OM_B_OFF, bshape, 2, ONNX_TYPE_INT8);
  g_bscale = dev_const(OM_BSCALE_OFF, qshape, 1, ONNX_TYPE_FLOAT);
  g_bzp = dev_const(OM_BZP_OFF, qshape, 1, ONNX_TYPE_INT8);
  g_ascale = scalar_f32(OM_A_SCALE);
  g_yscale = scalar_f32(OM_Y_SCALE);
  g_azp = scalar_u8(OM_A_ZP);
  g_yzp = scalar_u8(OM_Y_ZP);
  if (!g_b || !g_bscale || !g_bzp || !g_ascale || !g_yscale || !g_azp || !g_yzp)
    return;
  omcudaRegisterConstant(g_b);
  g_init_status = 0;
}
static OMTensorList *om_graph(OMTensorList *inputs) {
  if (omTensorListGetSize(inputs) != 1 && bad_input("expected 1 tensor"))
    return NULL;
  const OMTensor *a = omTensorListGetOmtByIndex(inputs, 0);
  int64_t rank = omTensorGetRank(a);
  if ((omTensorGetDataType(a) != ONNX_TYPE_UINT8 || rank < 2 || rank > 8 ||
          omTensorGetShape(a)[rank - 1] != OM_K) &&
      bad_input("A must be ui8 [.., " OM_STR(OM_K) "]"))
    return NULL;
  int64_t yshape[8];
  for (int64_t i = 0; i + 1 < rank; ++i)
    yshape[i] = omTensorGetShape(a)[i];
  yshape[rank - 1] = OM_N;
  OMTensor *y = make_output(a, yshape, rank, ONNX_TYPE_UINT8);
  if (!y)
    return NULL;
  omcudaQLinearMatMul(y, a, g_ascale, g_azp, g_b, g_bscale, g_bzp, g_yscale, g_yzp);
  if (omcudaTensorIsOnDevice(y))
    omcudaSynchronize();
  if (omcudaGetLastError() != OMCUDA_OK) {
    free_output(y);
    return NULL;
  }
  OMTensor *arr[1] = {y};
  return omTensorListCreate(arr, 1);
}
#elif OM_KIND == 3
static omcudaEncoder *g_enc;
static const OMTensor *cview(int64_t off, int64_t d0, int64_t d1, OM_DATA_TYPE dt) {
  int64_t shape[2] = {d0, d1};
  return omTensorCreate((void *)cptr(off), shape, d1 > 0 ? 2 : 1, dt);
}
static void om_init(void) {
  if (!g_constants)
    return;
  omcudaEncoderConfig cfg = {OM_LAYERS, OM_HIDDEN, OM_HEADS, OM_FFN, OM_EPS};
  g_enc = omcudaEncoderCreate(&cfg);
  if (!g_enc)
    return;
  const int64_t H = OM_HIDDEN, F = OM_FFN;
  for (int64_t l = 0; l < OM_LAYERS; ++l) {
    /* layer block: wq wk wv wo [H,H] i8, w1 [H,F], w2 [F,H], 6 f32 scales,
     * bq bk bv bo [H], b1 [F], b2 [H], ln1g ln1b ln2g ln2b [H] (all f32) */
    int64_t o = l * OM_LAYER_STRIDE;
    omcudaEncoderLayerWeights w;
    memset(&w, 0, sizeof(w));
    const OMTensor **mats[6] = {&w.wq, &w.wk, &w.wv, &w.wo, &w.w1, &w.w2};
    const int64_t rows[6] = {H, H, H, H, H, F}, cols[6] = {H, H, H, H, F, H};
    for (int i = 0; i < 6; ++i) {
      *mats[i] = cview(o, rows[i], cols[i], ONNX_TYPE_INT8);
      o += rows[i] * cols[i];
    }
    o = (o + 3) & ~(int64_t)3;
    memcpy(w.w_scale, cptr(o), 6 * sizeof(float));
    o += 6 * sizeof(float);
    const OMTensor **vecs[10] = {&w.bq, &w.bk, &w.bv, &w.bo, &w.b1, &w.b2, &w.ln1_gamma,
        &w.ln1_beta, &w.ln2_gamma, &w.ln2_beta};
    const int64_t lens[10] = {H, H, H, H, F, H, H, H, H, H};
    for (int i = 0; i < 10; ++i) {
      *vecs[i] = cview(o, lens[i], 0, ONNX_TYPE_FLOAT);
      o += lens[i] * 4;
    }
    int rc = omcudaEncoderSetLayer(g_enc, l, &w);
    for (int i = 0; i < 6; ++i)
      omTensorDestroy((OMTensor *)*mats[i]);
    for (int i = 0; i < 10; ++i)
      omTensorDestroy((OMTensor *)*vecs[i]);
    if (rc != OMCUDA_OK)
      return;
  }
  g_init_status = 0;
}
static OMTensorList *om_graph(OMTensorList *inputs) {
  /* input checks and the NULL + errno convention are the harness's */
  return omcudaEncoderRun(g_enc, inputs);
}
#else
#error "unknown OM_KIND"
#endif

OMTensorList *OM_TAGGED(run_main_graph)(OMTensorList *inputs) {
  /* Accelerator initialisation, as the generated entry point does it:
   * version check, EPERM and NULL when the library cannot serve the model. */
  if (!OMInitCompatibleAccelCUDA(OMCUDA_VERSION))
    return NULL;
  if (!g_constants) {
    errno = ENOENT;
    return NULL;
  }
  pthread_once(&g_once, om_init);
  if (g_init_status != 0) {
    if (errno == 0)
      errno = EIO;
    return NULL;
  }
  if (!inputs) {
    errno = EINVAL;
    return NULL;
  }
  OMTensorList *out = om_graph(inputs);
  if (!out) {
    /* errno carries the reason to the caller; the library's sticky status is
     * cleared so that the next request starts clean. */
    int e = errno ? errno : EIO;
    if (omcudaGetLastError() != OMCUDA_OK) {
      fprintf(stderr, "model %s: %s\n", OM_STR(OM_TAG), omcudaGetLastErrorString());
      omcudaClearError();
    }
    errno = e;
  }
  return out;
}
OMTensorList *run_main_graph(OMTensorList *inputs) { return OM_TAGGED(run_main_graph)(inputs); }

__attribute__((destructor)) static void om_unload(void) {
#if OM_KIND == 3
  if (g_enc && OMIsInitAccelCUDA)
    omcudaEncoderDestroy(g_enc);
#endif
  if (g_constants)
    omcudaUnloadConstantData(&g_constants, OM_CONST_BYTES);
}
