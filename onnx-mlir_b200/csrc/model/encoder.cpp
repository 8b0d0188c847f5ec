// Encoder model harness: the role of a compiled model's run_main_graph for the
// dynamic-quantized BERT-shaped encoder configurations.
//
// The generated entry point of onnx-mlir unpacks an OMTensorList, calls the
// graph function and packs the results
// (src/Conversion/KrnlToLLVM/KrnlEntryPoint.cpp:236-338).  This harness does
// the same around a fixed schedule of omcudaDev* launches, one per op of the
// graph, with every intermediate kept in HBM:
//
//   per layer (T = batch*seq tokens, H hidden, F ffn):
//     xq        = quantize(x)                 range of x from its producer
//     qkv[T,3H] = GEMM(xq, [Wq|Wk|Wv]) dequant + bias   (one launch: the three
//                 linears share xq; columns are independent, so the result
//                 is bit-identical to three launches)
//     ctx[T,H]  = attention(qkv)              keeps the range of ctx
//     a[T,H]    = x + GEMM(quantize(ctx), Wo) dequant + bias   (the residual
//                 add rides in the GEMM's tail for activations beyond L2
//                 size, inside LayerNorm otherwise)
//     h1        = LayerNorm(a)                keeps the range of h1
//     f[T,F]    = GEMM(quantize(h1), W1) dequant + bias + Gelu, keeps range
//     o[T,H]    = h1 + GEMM(quantize(f), W2) dequant + bias
//     y         = LayerNorm(o)                keeps the range of y (next x)
//
// DynamicQuantizeLinear needs the min/max of its whole input before it can
// write a byte.  Instead of a separate reduction pass, each producer folds the
// min/max of what it writes into an 8-byte running range with integer
// atomics; min/max is order-independent, so scale and zero point come out
// bit-identical to the reference's reduction
// (src/Conversion/ONNXToKrnl/Quantization/DynamicQuantizeLinear.cpp:29-84).
// Only the very first activation needs the standalone min/max kernel.
#include <cuda_runtime.h>

#include <cerrno>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../common.cuh"
#include "../runtime/internal.h"

using namespace omcuda;

namespace {

struct DevBuf {
  void *p = nullptr;
  size_t bytes = 0;
  // st: the stream the buffer is (and was) used on, for the pool's
  // stream-ordered reuse.
  void ensure(size_t n, cudaStream_t st = current_stream()) {
    if (n <= bytes)
      return;
    if (p)
      pool_free_on(p, st);
    p = pool_alloc_on(n, st);
    bytes = p ? n : 0;
  }
  void release() {
    if (p)
      pool_free(p);
    p = nullptr;
    bytes = 0;
  }
};

struct LayerState {
  bool set = false;
  omcudaPreparedB wqkv{}, wo{}, w1{}, w2{};
  DevBuf wqkv_bt, wqkv_cs, wo_bt, wo_cs, w1_bt, w1_cs, w2_bt, w2_cs;
  DevBuf qkv_scale; // f32 [3H]: w_scale of q | k | v per column
  DevBuf scal;      // f32 [3]: w_scale of wo, w1, w2
  DevBuf bqkv, bo, b1, b2, ln1g, ln1b, ln2g, ln2b;
  bool has_ln1b = false, has_ln2b = false;
};

} // namespace

struct omcudaEncoder {
  omcudaEncoderConfig cfg{};
  std::vector<LayerState> layers;
  // workspace, sized for the largest (batch*seq) seen
  int64_t tokens = 0;
  DevBuf xq, qkv, ctx, a, h1, f, o, ybuf[2];
  DevBuf stage_in, stage_out; // HBM staging of host tensors (omcudaEncoderRunInto)
  // Pipelined host-tensor runs (omcudaEncoderSubmit): two slots, so that the
  // copies of one call overlap the encoder run of its neighbours.
  struct Slot {
    DevBuf in, out;
    cudaEvent_t in_done = nullptr, run_done = nullptr, out_done = nullptr;
    bool used = false;
  } slot[2];
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  uint64_t submitted = 0;
  DevBuf ranges;  // 4 running ranges per layer + 1
  DevBuf params;  // 16 bytes per quantize site
  DevBuf dql_scratch;
  // optional timing of the GEMM launches (omcudaEncoderSetProfiling)
  bool profiling = false;
  std::vector<cudaEvent_t> ev;   // start/end pairs, recorded on the run stream
  size_t ev_used = 0;
  double gemm_ops = 0.0;         // 2*M*N*K summed over the recorded launches
  // optional copy of every layer's intermediates (omcudaEncoderSetTap)
  uint8_t *tap = nullptr;
  int64_t tap_bytes = 0;
  // optional all-reduce of every quantization range over the ranks that share
  // a batch (omcudaEncoderSetRangeSync)
  omcudaRangeSyncFn range_sync = nullptr;
  void *range_sync_ctx = nullptr;
  // Captured runs (CUDA graphs): a run is a fixed sequence of 11 launches per
  // layer whose arguments depend only on (x, y, batch, seq, stream) and two
  // process-wide settings (quantization mode, wait limit), so the
  // second run with the same key is captured and later ones are one graph
  // launch.  Dropped whenever a buffer a graph points into may have moved.
  struct Captured {
    const float *x;
    float *y;
    int64_t batch, seq;
    cudaStream_t st;
    // process-wide settings that end up in kernel arguments
    int quant_mode;
    uint64_t wait_ns;
    int seen;             // uncaptured runs so far with this key
    cudaGraphExec_t exec; // null until captured (or when capture failed)
    bool failed;
    int64_t launches;     // kernels in the graph, for the launch counter
  };
  std::vector<Captured> captured;
};

namespace {

void drop_graphs(omcudaEncoder *e);

int upload(DevBuf &dst, const OMTensor *t, size_t bytes, cudaStream_t st) {
  dst.ensure(bytes);
  if (!dst.p)
    return OMCUDA_ENOMEM;
  return check_cuda(cudaMemcpyAsync(dst.p, omTensorGetDataPtr(t), bytes,
                        cudaMemcpyDefault, st),
      "encoder: upload");
}

bool is_i8_matrix(const OMTensor *t, int64_t k, int64_t n) {
  return t && omTensorGetDataType(t) == ONNX_TYPE_INT8 &&
         omTensorGetRank(t) == 2 && omTensorGetShape(t)[0] == k &&
         omTensorGetShape(t)[1] == n;
}

bool is_f32_vec(const OMTensor *t, int64_t n) {
  return t && omTensorGetDataType(t) == ONNX_TYPE_FLOAT &&
         omTensorGetNumElems(t) == n;
}

int prepare(const void *w_dev, int64_t K, int64_t N, DevBuf &bt, DevBuf &cs,
    omcudaPreparedB *pb, cudaStream_t st) {
  int64_t kp;
  int64_t bytes = omcudaDevPreparedBBytes(K, N, &kp);
  bt.ensure((size_t)bytes);
  cs.ensure((size_t)N * sizeof(int32_t));
  if (!bt.p || !cs.p)
    return OMCUDA_ENOMEM;
  memset(pb, 0, sizeof(*pb));
  pb->bt = bt.p;
  pb->colsum = (int32_t *)cs.p;
  return omcudaDevPrepareB(w_dev, 1, K, N, pb, st);
}

// out[K][3H] = [a | b | c], each [K][H]
__global__ void concat_cols_kernel(const int8_t *a, const int8_t *b,
    const int8_t *c, int64_t K, int64_t H, int8_t *out) {
  int64_t total = K * 3 * H;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t k = i / (3 * H), n = i % (3 * H);
    const int8_t *src = n < H ? a : (n < 2 * H ? b : c);
    out[i] = src[k * H + (n % H)];
  }
}

__global__ void fill_kernel(float *dst, int64_t n, float v) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n)
    dst[i] = v;
}

int gemm(omcudaEncoder *e, const uint8_t *A, const uint8_t *a_zp,
    const float *a_scale, const omcudaPreparedB &B, int64_t M,
    const float *w_scale, int64_t ws_len, const float *bias, int gelu, void *Y,
    void *out_range, cudaStream_t st, int epilogue = OMCUDA_EPI_DEQUANT,
    const float *residual = nullptr, const void *q_range = nullptr,
    float *q_slot = nullptr) {
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (e->profiling) {
    while (e->ev.size() < e->ev_used + 2) {
      cudaEvent_t ne;
      if (cudaEventCreate(&ne) != cudaSuccess)
        break;
      e->ev.push_back(ne);
    }
    if (e->ev.size() >= e->ev_used + 2) {
      e0 = e->ev[e->ev_used];
      e1 = e->ev[e->ev_used + 1];
      e->ev_used += 2;
      e->gemm_ops += 2.0 * (double)M * (double)B.N * (double)B.K;
      cudaEventRecord(e0, st);
    }
  }
  omcudaGemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = M;
  g.N = B.N;
  g.K = B.K;
  g.A = A;
  g.a_signed = 0;
  g.B = B;
  g.a_zp = a_zp;
  g.a_zp_len = 1;
  g.epilogue = epilogue;
  g.Y = Y;
  g.sa = a_scale;
  g.sb = w_scale;
  g.sb_len = ws_len;
  g.scale_form = 0;
  g.bias = bias;
  g.gelu = gelu;
  g.out_minmax = out_range;
  g.residual = residual;
  if (q_slot) { // a quantize site's slot: scale, zero point, y_scale, y_zero_point
    g.q_range = q_range;
    g.q_params = q_slot;
    g.q_scale = q_slot + 2;
    g.q_zp = (uint8_t *)(q_slot + 3);
  }
  int rc = omcudaDevGemmI8(&g, st);
  if (e1)
    cudaEventRecord(e1, st);
  return rc;
}

int64_t up16(int64_t v) { return (v + 15) & ~int64_t(15); }

void tap_layout(const omcudaEncoderConfig &c, int64_t T, omcudaEncoderTapLayout *o) {
  const int64_t th4 = up16(T * c.hidden * 4), th1 = up16(T * c.hidden);
  const int64_t tf4 = up16(T * c.ffn * 4), tf1 = up16(T * c.ffn);
  int64_t at = 0;
  o->x = at, at += th4;
  o->xq_x = at, at += th1;
  o->ctx = at, at += th4;
  o->xq_ctx = at, at += th1;
  o->h1 = at, at += th4;
  o->xq_h1 = at, at += th1;
  o->f = at, at += tf4;
  o->xq_f = at, at += tf1;
  o->y = at, at += th4;
  o->layer_stride = at;
  o->params = at * c.layers;
  o->total = o->params + up16((4 * c.layers + 1) * 16);
}

int tap_copy(omcudaEncoder *e, int64_t off, const void *src, int64_t bytes,
    cudaStream_t st) {
  if (!e->tap)
    return OMCUDA_OK;
  return check_cuda(cudaMemcpyAsync(e->tap + off, src, (size_t)bytes,
                        cudaMemcpyDeviceToDevice, st),
      "encoder: tap copy");
}

// Off unless OMCUDA_FFN_TWO_PASS=1: on B200 the two passes over the product
// measured slower than one pass that writes f32 plus the quantize pass (the
// Gelu tail is bound by instruction issue, not by the f32 traffic it saves).
bool ffn_two_pass_wanted() {
  static const bool on = [] {
    const char *s = getenv("OMCUDA_FFN_TWO_PASS");
    return s && atoi(s) == 1;
  }();
  return on;
}

int ensure_workspace(omcudaEncoder *e, int64_t T, cudaStream_t st) {
  const int64_t H = e->cfg.hidden, F = e->cfg.ffn;
  const int64_t maxk = H > F ? H : F;
  if (T > e->tokens) {
    e->xq.ensure((size_t)(T * maxk), st);
    e->qkv.ensure((size_t)(T * 3 * H) * 4, st);
    e->ctx.ensure((size_t)(T * H) * 4, st);
    e->a.ensure((size_t)(T * H) * 4, st);
    e->h1.ensure((size_t)(T * H) * 4, st);
    e->f.ensure((size_t)(T * F) * 4, st);
    e->o.ensure((size_t)(T * H) * 4, st);
    e->ybuf[0].ensure((size_t)(T * H) * 4, st);
    e->ybuf[1].ensure((size_t)(T * H) * 4, st);
    if (!e->xq.p || !e->qkv.p || !e->ctx.p || !e->a.p || !e->h1.p || !e->f.p ||
        !e->o.p || !e->ybuf[0].p || !e->ybuf[1].p)
      return OMCUDA_ENOMEM;
    e->tokens = T;
  }
  if (!e->ranges.p) {
    size_t nr = (size_t)(4 * e->cfg.layers + 1);
    e->ranges.ensure(nr * 8, st);
    e->params.ensure(nr * 16, st);
    e->dql_scratch.ensure((size_t)omcudaDevDqlScratchBytes(0), st);
    if (!e->ranges.p || !e->params.p || !e->dql_scratch.p)
      return OMCUDA_ENOMEM;
    int rc = check_cuda(cudaMemsetAsync(e->dql_scratch.p, 0, e->dql_scratch.bytes, st),
        "encoder: scratch");
    if (rc != OMCUDA_OK)
      return rc;
  }
  return OMCUDA_OK;
}

} // namespace

extern "C" omcudaEncoder *omcudaEncoderCreate(const omcudaEncoderConfig *cfg) {
  if (ensure_init() != OMCUDA_OK)
    return nullptr;
  if (!cfg || cfg->layers <= 0 || cfg->hidden <= 0 || cfg->heads <= 0 ||
      cfg->ffn <= 0 || cfg->hidden % cfg->heads != 0) {
    fail(OMCUDA_EINVAL, "EncoderCreate: bad configuration");
    return nullptr;
  }
  int64_t dh = cfg->hidden / cfg->heads;
  if (dh != 32 && dh != 64 && dh != 128) {
    fail(OMCUDA_ENOTSUP, "EncoderCreate: head size must be 32, 64 or 128");
    return nullptr;
  }
  omcudaEncoder *e = new omcudaEncoder();
  e->cfg = *cfg;
  e->layers.resize((size_t)cfg->layers);
  return e;
}

extern "C" int omcudaEncoderSetLayer(
    omcudaEncoder *e, int64_t layer, const omcudaEncoderLayerWeights *w) {
  if (!e || !w || layer < 0 || layer >= e->cfg.layers)
    return fail(OMCUDA_EINVAL, "EncoderSetLayer: bad argument");
  const int64_t H = e->cfg.hidden, F = e->cfg.ffn;
  if (!is_i8_matrix(w->wq, H, H) || !is_i8_matrix(w->wk, H, H) ||
      !is_i8_matrix(w->wv, H, H) || !is_i8_matrix(w->wo, H, H) ||
      !is_i8_matrix(w->w1, H, F) || !is_i8_matrix(w->w2, F, H))
    return fail(OMCUDA_EINVAL, "EncoderSetLayer: weights must be int8 [in,out]");
  if (!is_f32_vec(w->bq, H) || !is_f32_vec(w->bk, H) || !is_f32_vec(w->bv, H) ||
      !is_f32_vec(w->bo, H) || !is_f32_vec(w->b1, F) || !is_f32_vec(w->b2, H) ||
      !is_f32_vec(w->ln1_gamma, H) || !is_f32_vec(w->ln2_gamma, H) ||
      (w->ln1_beta && !is_f32_vec(w->ln1_beta, H)) ||
      (w->ln2_beta && !is_f32_vec(w->ln2_beta, H)))
    return fail(OMCUDA_EINVAL, "EncoderSetLayer: bias / LayerNorm shapes");
  cudaStream_t st = current_stream();
  drop_graphs(e); // captured runs hold the old weights' addresses
  LayerState &L = e->layers[(size_t)layer];
  int rc = OMCUDA_OK;
  // [Wq | Wk | Wv] as one [H, 3H] operand
  DevBuf tq, tk, tv, cat, t1, t2, t3;
  if ((rc = upload(tq, w->wq, (size_t)(H * H), st)) != OMCUDA_OK ||
      (rc = upload(tk, w->wk, (size_t)(H * H), st)) != OMCUDA_OK ||
      (rc = upload(tv, w->wv, (size_t)(H * H), st)) != OMCUDA_OK)
    return rc;
  cat.ensure((size_t)(3 * H * H));
  if (!cat.p)
    return OMCUDA_ENOMEM;
  concat_cols_kernel<<<sm_count() * 4, 256, 0, st>>>((const int8_t *)tq.p,
      (const int8_t *)tk.p, (const int8_t *)tv.p, H, H, (int8_t *)cat.p);
  count_launch();
  if ((rc = check_cuda(cudaGetLastError(), "concat_cols_kernel")) != OMCUDA_OK)
    return rc;
  if ((rc = prepare(cat.p, H, 3 * H, L.wqkv_bt, L.wqkv_cs, &L.wqkv, st)) != OMCUDA_OK)
    return rc;
  if ((rc = upload(t1, w->wo, (size_t)(H * H), st)) != OMCUDA_OK ||
      (rc = prepare(t1.p, H, H, L.wo_bt, L.wo_cs, &L.wo, st)) != OMCUDA_OK)
    return rc;
  if ((rc = upload(t2, w->w1, (size_t)(H * F), st)) != OMCUDA_OK ||
      (rc = prepare(t2.p, H, F, L.w1_bt, L.w1_cs, &L.w1, st)) != OMCUDA_OK)
    return rc;
  if ((rc = upload(t3, w->w2, (size_t)(F * H), st)) != OMCUDA_OK ||
      (rc = prepare(t3.p, F, H, L.w2_bt, L.w2_cs, &L.w2, st)) != OMCUDA_OK)
    return rc;
  // scales
  L.qkv_scale.ensure((size_t)(3 * H) * sizeof(float));
  L.scal.ensure(4 * sizeof(float));
  if (!L.qkv_scale.p || !L.scal.p)
    return OMCUDA_ENOMEM;
  for (int i = 0; i < 3; ++i) {
    fill_kernel<<<(unsigned)ceil_div(H, 256), 256, 0, st>>>(
        (float *)L.qkv_scale.p + i * H, H, w->w_scale[i]);
    count_launch();
  }
  float hs[4] = {w->w_scale[3], w->w_scale[4], w->w_scale[5], 0.0f};
  if ((rc = check_cuda(cudaMemcpyAsync(L.scal.p, hs, sizeof(hs),
                           cudaMemcpyHostToDevice, st),
           "encoder: scales")) != OMCUDA_OK)
    return rc;
  // biases and LayerNorm parameters
  L.bqkv.ensure((size_t)(3 * H) * sizeof(float));
  if (!L.bqkv.p)
    return OMCUDA_ENOMEM;
  const OMTensor *bs[3] = {w->bq, w->bk, w->bv};
  for (int i = 0; i < 3; ++i)
    if ((rc = check_cuda(cudaMemcpyAsync((float *)L.bqkv.p + i * H,
                             omTensorGetDataPtr(bs[i]), (size_t)H * 4,
                             cudaMemcpyDefault, st),
             "encoder: bias")) != OMCUDA_OK)
      return rc;
  if ((rc = upload(L.bo, w->bo, (size_t)H * 4, st)) != OMCUDA_OK ||
      (rc = upload(L.b1, w->b1, (size_t)F * 4, st)) != OMCUDA_OK ||
      (rc = upload(L.b2, w->b2, (size_t)H * 4, st)) != OMCUDA_OK ||
      (rc = upload(L.ln1g, w->ln1_gamma, (size_t)H * 4, st)) != OMCUDA_OK ||
      (rc = upload(L.ln2g, w->ln2_gamma, (size_t)H * 4, st)) != OMCUDA_OK)
    return rc;
  L.has_ln1b = w->ln1_beta != nullptr;
  L.has_ln2b = w->ln2_beta != nullptr;
  if (L.has_ln1b &&
      (rc = upload(L.ln1b, w->ln1_beta, (size_t)H * 4, st)) != OMCUDA_OK)
    return rc;
  if (L.has_ln2b &&
      (rc = upload(L.ln2b, w->ln2_beta, (size_t)H * 4, st)) != OMCUDA_OK)
    return rc;
  // hs[] and the staging buffers go out of scope: finish the copies first.
  if ((rc = check_cuda(cudaStreamSynchronize(st), "encoder: sync")) != OMCUDA_OK)
    return rc;
  tq.release();
  tk.release();
  tv.release();
  cat.release();
  t1.release();
  t2.release();
  t3.release();
  L.set = true;
  return OMCUDA_OK;
}

namespace {

void drop_graphs(omcudaEncoder *e) {
  for (auto &c : e->captured)
    if (c.exec)
      cudaGraphExecDestroy(c.exec);
  e->captured.clear();
}

// OMCUDA_ENCODER_GRAPH=0 launches every run kernel by kernel.
bool graphs_wanted() {
  static const bool on = [] {
    const char *s = getenv("OMCUDA_ENCODER_GRAPH");
    return !(s && atoi(s) == 0);
  }();
  return on;
}

int run_launches(omcudaEncoder *e, const float *x, int64_t batch, int64_t seq, float *y,
    cudaStream_t st);

} // namespace

extern "C" int omcudaEncoderRunDev(omcudaEncoder *e, const float *x,
    int64_t batch, int64_t seq, float *y, void *stream) {
  if (!e || !x || !y || batch <= 0 || seq <= 0)
    return fail(OMCUDA_EINVAL, "EncoderRun: bad argument");
  for (auto &L : e->layers)
    if (!L.set)
      return fail(OMCUDA_EINVAL, "EncoderRun: a layer has no weights");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t tokens_before = e->tokens;
  int rc = ensure_workspace(e, batch * seq, st);
  if (rc != OMCUDA_OK)
    return rc;
  if (e->tokens != tokens_before)
    drop_graphs(e); // the workspace moved
  // Runs that call back to the host (range sync), copy intermediates out (tap)
  // or record events between launches (profiling) are not captured.
  if (!graphs_wanted() || e->tap || e->range_sync || e->profiling)
    return run_launches(e, x, batch, seq, y, st);
  omcudaEncoder::Captured *c = nullptr;
  const int mode = quant_mode();
  const uint64_t wait_ns = tc_wait_limit_ns();
  for (auto &k : e->captured)
    if (k.x == x && k.y == y && k.batch == batch && k.seq == seq && k.st == st &&
        k.quant_mode == mode && k.wait_ns == wait_ns)
      c = &k;
  if (!c) {
    if (e->captured.size() >= 8)
      drop_graphs(e);
    e->captured.push_back({x, y, batch, seq, st, mode, wait_ns, 0, nullptr, false, 0});
    c = &e->captured.back();
  }
  if (c->exec) {
    OMCUDA_CHECK(cudaGraphLaunch(c->exec, st));
    count_launch((int)c->launches);
    return OMCUDA_OK;
  }
  if (c->failed || c->seen < 1) {
    // The first run with a key goes kernel by kernel: it performs the one-time
    // set-up of the launchers (function attributes, the status word), which
    // must not happen inside a capture.
    ++c->seen;
    return run_launches(e, x, batch, seq, y, st);
  }
  cudaStreamCaptureStatus busy = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &busy) != cudaSuccess || busy != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return run_launches(e, x, batch, seq, y, st); // the caller is capturing: join its graph
  }
  const int64_t before = omcudaLaunchCount();
  if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    (void)cudaGetLastError();
    c->failed = true;
    return run_launches(e, x, batch, seq, y, st);
  }
  rc = run_launches(e, x, batch, seq, y, st);
  cudaGraph_t graph = nullptr;
  cudaError_t ce = cudaStreamEndCapture(st, &graph);
  const int64_t captured_launches = omcudaLaunchCount() - before;
  count_launch((int)-captured_launches); // nothing ran yet
  if (rc != OMCUDA_OK || ce != cudaSuccess || !graph) {
    (void)cudaGetLastError();
    if (graph)
      cudaGraphDestroy(graph);
    c->failed = true;
    if (rc != OMCUDA_OK)
      return rc;
    return run_launches(e, x, batch, seq, y, st);
  }
  ce = cudaGraphInstantiate(&c->exec, graph, 0);
  cudaGraphDestroy(graph);
  if (ce != cudaSuccess) {
    (void)cudaGetLastError();
    c->exec = nullptr;
    c->failed = true;
    return run_launches(e, x, batch, seq, y, st);
  }
  c->launches = captured_launches;
  OMCUDA_CHECK(cudaGraphLaunch(c->exec, st));
  count_launch((int)c->launches);
  return OMCUDA_OK;
}

namespace {

int run_launches(omcudaEncoder *e, const float *x, int64_t batch, int64_t seq, float *y,
    cudaStream_t st) {
  const int64_t H = e->cfg.hidden, F = e->cfg.ffn, heads = e->cfg.heads;
  const int64_t dh = H / heads, T = batch * seq;
  int rc = OMCUDA_OK;
  const float att_scale = 1.0f / sqrtf((float)dh);
  const float eps = (float)e->cfg.epsilon;
  const int64_t nranges = 4 * e->cfg.layers + 1;
  uint8_t *ranges = (uint8_t *)e->ranges.p;
  float *params = (float *)e->params.p;
  uint8_t *xq = (uint8_t *)e->xq.p;
  // Head size 64 and a sequence that is a multiple of 128 take the tcgen05
  // attention kernel, which reads Q, K, V as bf16 hi/lo planes.
  const bool use_tc_attention =
      omcudaDevAttentionBf16Supported(batch, seq, heads, dh, 3 * H, H) != 0;
  // (the f32 [T,3H] buffer holds the two bf16 [T,3H] planes instead)
  const bool fuse_residual = (size_t)(T * H) * 4 >= ((size_t)64 << 20);
  // Gelu(Linear(h1)) feeds nothing but a DynamicQuantizeLinear, so the f32
  // [T,F] tensor can be avoided by running the product twice: once to learn
  // the range of the activations, once to quantize them on the way out.
  // Same values, same bytes (an experiment switch, see ffn_two_pass_wanted).
  const bool ffn_two_pass = ffn_two_pass_wanted();
  omcudaEncoderTapLayout tl;
  tap_layout(e->cfg, T, &tl);
  if (e->range_sync && ffn_two_pass)
    return fail(OMCUDA_ENOTSUP, "EncoderRun: range sync and the two-pass FFN do not combine");
#define SYNC_RANGE(r)                                                          \
  do {                                                                         \
    if (e->range_sync)                                                         \
      e->range_sync(e->range_sync_ctx, (r), (void *)st);                       \
  } while (0)
  if (e->tap && (ffn_two_pass || e->tap_bytes < tl.total))
    return fail(OMCUDA_EINVAL,
        "EncoderRun: the tap buffer holds %lld bytes, this run needs %lld",
        (long long)e->tap_bytes, (long long)tl.total);
  uint8_t *fq = (uint8_t *)e->f.p; // uint8 [T,F] in the two-pass form
  void *planes_hi = e->qkv.p;
  void *planes_lo = (uint8_t *)e->qkv.p + (size_t)(T * 3 * H) * 2;
#define RUN(call)                                                              \
  do {                                                                         \
    rc = (call);                                                               \
    if (rc != OMCUDA_OK)                                                       \
      return rc;                                                               \
  } while (0)
  RUN(omcudaDevRangeInit(ranges, nranges, st));
  // Slot layout of a quantize site (4 floats): [0] scale, [1] zero point as
  // float (both read by the quantize pass), [2] scale as the op's y_scale
  // output, [3] first byte: zero point as uint8 (the GEMM's a_zero_point).
  // The model input has no producer here: it gets the standalone reduction.
  if (e->range_sync) {
    // global ranges: the input's range is folded like a producer's, reduced
    // over the ranks, and the quantize pass derives scale and zero point
    RUN(omcudaDevRangeFold(x, T * H, ranges, st));
    SYNC_RANGE(ranges);
    RUN(omcudaDevQuantizeFromRange(x, T * H, ranges, xq, params, params + 2,
        (uint8_t *)(params + 3), st));
  } else {
    RUN(omcudaDevDynamicQuantizeLinear(x, T * H, xq, params + 2,
        (uint8_t *)(params + 3), e->dql_scratch.p, st));
  }
  const float *cur = x;
  for (int64_t l = 0; l < e->cfg.layers; ++l) {
    LayerState &L = e->layers[(size_t)l];
    uint8_t *r_x = ranges + (size_t)(4 * l) * 8;
    uint8_t *r_ctx = ranges + (size_t)(4 * l + 1) * 8;
    uint8_t *r_h1 = ranges + (size_t)(4 * l + 2) * 8;
    uint8_t *r_f = ranges + (size_t)(4 * l + 3) * 8;
    uint8_t *r_y = ranges + (size_t)(4 * l + 4) * 8;
    float *p_x = params + (size_t)(4 * l) * 4;
    float *p_ctx = params + (size_t)(4 * l + 1) * 4;
    float *p_h1 = params + (size_t)(4 * l + 2) * 4;
    float *p_f = params + (size_t)(4 * l + 3) * 4;
    float *nxt = (l + 1 == e->cfg.layers) ? y : (float *)e->ybuf[l & 1].p;
    if (l > 0) {
      SYNC_RANGE(r_x);
      RUN(omcudaDevQuantizeFromRange(cur, T * H, r_x, xq, p_x, p_x + 2,
          (uint8_t *)(p_x + 3), st));
    }
    const int64_t tb = l * tl.layer_stride;
    RUN(tap_copy(e, tb + tl.x, cur, T * H * 4, st));
    RUN(tap_copy(e, tb + tl.xq_x, xq, T * H, st));
    if (use_tc_attention) {
      // The projection writes q | k | v straight into the bf16 hi/lo planes
      // the attention kernel reads; the f32 values never reach HBM.
      RUN(gemm(e, xq, (const uint8_t *)(p_x + 3), p_x + 2, L.wqkv, T,
          (const float *)L.qkv_scale.p, 3 * H, (const float *)L.bqkv.p, 0,
          planes_hi, nullptr, st, OMCUDA_EPI_DEQUANT_SPLIT));
      RUN(omcudaDevAttentionBf16(planes_hi, planes_lo, 3 * H, 0, H, 2 * H, batch,
          seq, heads, dh, att_scale, (float *)e->ctx.p, H, r_ctx, st));
    } else {
      RUN(gemm(e, xq, (const uint8_t *)(p_x + 3), p_x + 2, L.wqkv, T,
          (const float *)L.qkv_scale.p, 3 * H, (const float *)L.bqkv.p, 0,
          (float *)e->qkv.p, nullptr, st));
      const float *q = (const float *)e->qkv.p;
      RUN(omcudaDevAttentionEx(q, q + H, q + 2 * H, batch, seq, heads, dh,
          att_scale, (float *)e->ctx.p, 3 * H, H, r_ctx, st));
    }
    SYNC_RANGE(r_ctx);
    RUN(omcudaDevQuantizeFromRange((const float *)e->ctx.p, T * H, r_ctx, xq,
        p_ctx, p_ctx + 2, (uint8_t *)(p_ctx + 3), st));
    RUN(tap_copy(e, tb + tl.ctx, e->ctx.p, T * H * 4, st));
    RUN(tap_copy(e, tb + tl.xq_ctx, xq, T * H, st));
    // a = [x +] Linear(ctx): the residual add rides in the GEMM's tail when
    // the activations are too large for L2 (it saves LayerNorm one pass over
    // HBM); small ones are cheaper to add inside LayerNorm.  Same fp32 add
    // either way.
    RUN(gemm(e, xq, (const uint8_t *)(p_ctx + 3), p_ctx + 2, L.wo, T,
        (const float *)L.scal.p, 1, (const float *)L.bo.p, 0, (float *)e->a.p,
        nullptr, st, OMCUDA_EPI_DEQUANT, fuse_residual ? cur : nullptr));
    RUN(omcudaDevLayerNorm(fuse_residual ? (const float *)e->a.p : cur,
        fuse_residual ? nullptr : (const float *)e->a.p, T, H,
        (const float *)L.ln1g.p, L.has_ln1b ? (const float *)L.ln1b.p : nullptr,
        eps, (float *)e->h1.p, r_h1, st));
    SYNC_RANGE(r_h1);
    RUN(omcudaDevQuantizeFromRange((const float *)e->h1.p, T * H, r_h1, xq,
        p_h1, p_h1 + 2, (uint8_t *)(p_h1 + 3), st));
    RUN(tap_copy(e, tb + tl.h1, e->h1.p, T * H * 4, st));
    RUN(tap_copy(e, tb + tl.xq_h1, xq, T * H, st));
    if (ffn_two_pass) {
      RUN(gemm(e, xq, (const uint8_t *)(p_h1 + 3), p_h1 + 2, L.w1, T,
          (const float *)L.scal.p + 1, 1, (const float *)L.b1.p, 1, nullptr, r_f,
          st, OMCUDA_EPI_DEQUANT_RANGE));
      RUN(gemm(e, xq, (const uint8_t *)(p_h1 + 3), p_h1 + 2, L.w1, T,
          (const float *)L.scal.p + 1, 1, (const float *)L.b1.p, 1, fq, nullptr,
          st, OMCUDA_EPI_DEQUANT_QUANT, nullptr, r_f, p_f));
    } else {
      RUN(gemm(e, xq, (const uint8_t *)(p_h1 + 3), p_h1 + 2, L.w1, T,
          (const float *)L.scal.p + 1, 1, (const float *)L.b1.p, 1,
          (float *)e->f.p, r_f, st));
      SYNC_RANGE(r_f);
      RUN(omcudaDevQuantizeFromRange((const float *)e->f.p, T * F, r_f, xq, p_f,
          p_f + 2, (uint8_t *)(p_f + 3), st));
      RUN(tap_copy(e, tb + tl.f, e->f.p, T * F * 4, st));
      RUN(tap_copy(e, tb + tl.xq_f, xq, T * F, st));
    }
    RUN(gemm(e, ffn_two_pass ? fq : xq, (const uint8_t *)(p_f + 3), p_f + 2, L.w2, T,
        (const float *)L.scal.p + 2, 1, (const float *)L.b2.p, 0,
        (float *)e->o.p, nullptr, st, OMCUDA_EPI_DEQUANT,
        fuse_residual ? (const float *)e->h1.p : nullptr));
    RUN(omcudaDevLayerNorm(fuse_residual ? (const float *)e->o.p : (const float *)e->h1.p,
        fuse_residual ? nullptr : (const float *)e->o.p, T, H,
        (const float *)L.ln2g.p, L.has_ln2b ? (const float *)L.ln2b.p : nullptr,
        eps, nxt, r_y, st));
    RUN(tap_copy(e, tb + tl.y, nxt, T * H * 4, st));
    cur = nxt;
  }
  RUN(tap_copy(e, tl.params, params, (4 * e->cfg.layers + 1) * 16, st));
#undef RUN
#undef SYNC_RANGE
  return OMCUDA_OK;
}

} // namespace

extern "C" OMTensorList *omcudaEncoderRun(omcudaEncoder *e, OMTensorList *inputs) {
  if (sticky_error() || ensure_init() != OMCUDA_OK)
    return nullptr;
  if (!e || !inputs || omTensorListGetSize(inputs) != 1) {
    fail(OMCUDA_EINVAL, "EncoderRun: expected one input tensor");
    return nullptr;
  }
  const OMTensor *x = omTensorListGetOmtByIndex(inputs, 0);
  // The checks a generated entry point makes on its inputs
  // (KrnlEntryPoint.cpp:430-545): element type, rank, static dimensions.
  if (!x || omTensorGetDataType(x) != ONNX_TYPE_FLOAT || omTensorGetRank(x) != 3 ||
      omTensorGetShape(x)[2] != e->cfg.hidden) {
    fail(OMCUDA_EINVAL, "EncoderRun: input must be f32 [batch, seq, %lld]",
        (long long)e->cfg.hidden);
    return nullptr;
  }
  const int64_t B = omTensorGetShape(x)[0], S = omTensorGetShape(x)[1];
  const int64_t n = B * S * e->cfg.hidden;
  cudaStream_t st = current_stream();
  const bool on_dev = omcudaTensorIsOnDevice(x) != 0;
  OMTensor *out = nullptr;
  if (on_dev) {
    out = omcudaTensorCreateOnDevice(omTensorGetShape(x), 3, ONNX_TYPE_FLOAT);
    if (!out)
      return nullptr;
    if (omcudaEncoderRunDev(e, (const float *)omTensorGetDataPtr(x), B, S,
            (float *)omTensorGetDataPtr(out), st) != OMCUDA_OK) {
      omcudaTensorDestroy(out);
      return nullptr;
    }
  } else {
    DevBuf dx, dy;
    dx.ensure((size_t)n * 4);
    dy.ensure((size_t)n * 4);
    out = omTensorCreateEmpty(omTensorGetShape(x), 3, ONNX_TYPE_FLOAT);
    bool ok = dx.p && dy.p && out;
    ok = ok && check_cuda(cudaMemcpyAsync(dx.p, omTensorGetDataPtr(x),
                              (size_t)n * 4, cudaMemcpyHostToDevice, st),
                   "encoder: H2D") == OMCUDA_OK;
    ok = ok && omcudaEncoderRunDev(e, (const float *)dx.p, B, S, (float *)dy.p,
                   st) == OMCUDA_OK;
    ok = ok && check_cuda(cudaMemcpyAsync(omTensorGetDataPtr(out), dy.p,
                              (size_t)n * 4, cudaMemcpyDeviceToHost, st),
                   "encoder: D2H") == OMCUDA_OK;
    if (ok) {
      omcudaSynchronize();
      ok = !sticky_error();
    }
    dx.release();
    dy.release();
    if (!ok) {
      if (out)
        omTensorDestroy(out);
      if (!sticky_error())
        fail(OMCUDA_ENOMEM, "EncoderRun: allocation failed");
      return nullptr;
    }
  }
  OMTensor *arr[1] = {out};
  OMTensorList *res = omTensorListCreate(arr, 1);
  if (!res) {
    fail(OMCUDA_ENOMEM, "EncoderRun: cannot build the output list");
    return nullptr;
  }
  return res;
}

extern "C" int omcudaEncoderRunInto(
    omcudaEncoder *e, OMTensor *y, const OMTensor *x) {
  if (sticky_error())
    return omcudaGetLastError();
  int rc = ensure_init();
  if (rc != OMCUDA_OK)
    return rc;
  if (!e || !x || !y || omTensorGetDataType(x) != ONNX_TYPE_FLOAT ||
      omTensorGetDataType(y) != ONNX_TYPE_FLOAT || omTensorGetRank(x) != 3 ||
      omTensorGetRank(y) != 3 || omTensorGetShape(x)[2] != e->cfg.hidden)
    return fail(OMCUDA_EINVAL, "EncoderRunInto: x and y must be f32 [batch, seq, %lld]",
        (long long)e->cfg.hidden);
  for (int i = 0; i < 3; ++i)
    if (omTensorGetShape(x)[i] != omTensorGetShape(y)[i])
      return fail(OMCUDA_EINVAL, "EncoderRunInto: y must have the shape of x");
  const int64_t B = omTensorGetShape(x)[0], S = omTensorGetShape(x)[1];
  const size_t bytes = (size_t)(B * S * e->cfg.hidden) * 4;
  cudaStream_t st = current_stream();
  const bool x_dev = omcudaTensorIsOnDevice(x) != 0;
  const bool y_dev = omcudaTensorIsOnDevice(y) != 0;
  const float *dx = (const float *)omTensorGetDataPtr(x);
  float *dy = (float *)omTensorGetDataPtr(y);
  if (!x_dev) {
    e->stage_in.ensure(bytes);
    if (!e->stage_in.p)
      return OMCUDA_ENOMEM;
    OMCUDA_CHECK(cudaMemcpyAsync(e->stage_in.p, omTensorGetDataPtr(x), bytes,
        cudaMemcpyHostToDevice, st));
    dx = (const float *)e->stage_in.p;
  }
  if (!y_dev) {
    e->stage_out.ensure(bytes);
    if (!e->stage_out.p)
      return OMCUDA_ENOMEM;
    dy = (float *)e->stage_out.p;
  }
  rc = omcudaEncoderRunDev(e, dx, B, S, dy, st);
  if (rc != OMCUDA_OK)
    return rc;
  if (!y_dev) {
    OMCUDA_CHECK(cudaMemcpyAsync(omTensorGetDataPtr(y), dy, bytes,
        cudaMemcpyDeviceToHost, st));
    omcudaSynchronize(); // the host buffer is complete when the call returns
    if (sticky_error())
      return omcudaGetLastError();
  }
  return OMCUDA_OK;
}

// One call of the pipeline: H2D on the encoder's inbound copy stream, the run
// on the calling thread's stream, D2H on the outbound copy stream, chained by
// events.  Slot k & 1 is reused by call k + 2: its input buffer once run k is
// done (a stream wait), its output buffer once copy-out k is done (a host
// wait, which also bounds the queue to two calls).
extern "C" int omcudaEncoderSubmit(
    omcudaEncoder *e, OMTensor *y, const OMTensor *x) {
  if (sticky_error())
    return omcudaGetLastError();
  int rc = ensure_init();
  if (rc != OMCUDA_OK)
    return rc;
  if (!e || !x || !y || omTensorGetDataType(x) != ONNX_TYPE_FLOAT ||
      omTensorGetDataType(y) != ONNX_TYPE_FLOAT || omTensorGetRank(x) != 3 ||
      omTensorGetRank(y) != 3 || omTensorGetShape(x)[2] != e->cfg.hidden)
    return fail(OMCUDA_EINVAL, "EncoderSubmit: x and y must be f32 [batch, seq, %lld]",
        (long long)e->cfg.hidden);
  for (int i = 0; i < 3; ++i)
    if (omTensorGetShape(x)[i] != omTensorGetShape(y)[i])
      return fail(OMCUDA_EINVAL, "EncoderSubmit: y must have the shape of x");
  if (omcudaTensorIsOnDevice(x) || omcudaTensorIsOnDevice(y))
    return fail(OMCUDA_EINVAL,
        "EncoderSubmit: host tensors only (device tensors: omcudaEncoderRunInto)");
  const int64_t B = omTensorGetShape(x)[0], S = omTensorGetShape(x)[1];
  const size_t bytes = (size_t)(B * S * e->cfg.hidden) * 4;
  cudaStream_t st = current_stream();
  if (!e->copy_in) {
    OMCUDA_CHECK(cudaStreamCreateWithFlags(&e->copy_in, cudaStreamNonBlocking));
    OMCUDA_CHECK(cudaStreamCreateWithFlags(&e->copy_out, cudaStreamNonBlocking));
  }
  omcudaEncoder::Slot &sl = e->slot[e->submitted & 1];
  if (!sl.in_done) {
    OMCUDA_CHECK(cudaEventCreateWithFlags(&sl.in_done, cudaEventDisableTiming));
    OMCUDA_CHECK(cudaEventCreateWithFlags(&sl.run_done, cudaEventDisableTiming));
    OMCUDA_CHECK(cudaEventCreateWithFlags(&sl.out_done, cudaEventDisableTiming));
  }
  if (sl.used) {
    OMCUDA_CHECK(cudaEventSynchronize(sl.out_done));
    OMCUDA_CHECK(cudaStreamWaitEvent(e->copy_in, sl.run_done, 0));
  }
  if (bytes > sl.in.bytes || bytes > sl.out.bytes) {
    // growing a buffer frees the old one: nothing may still be using it
    OMCUDA_CHECK(cudaStreamSynchronize(st));
    sl.in.ensure(bytes);
    sl.out.ensure(bytes);
    if (!sl.in.p || !sl.out.p)
      return OMCUDA_ENOMEM;
  }
  OMCUDA_CHECK(cudaMemcpyAsync(sl.in.p, omTensorGetDataPtr(x), bytes,
      cudaMemcpyHostToDevice, e->copy_in));
  OMCUDA_CHECK(cudaEventRecord(sl.in_done, e->copy_in));
  OMCUDA_CHECK(cudaStreamWaitEvent(st, sl.in_done, 0));
  rc = omcudaEncoderRunDev(e, (const float *)sl.in.p, B, S, (float *)sl.out.p, st);
  if (rc != OMCUDA_OK)
    return rc;
  OMCUDA_CHECK(cudaEventRecord(sl.run_done, st));
  OMCUDA_CHECK(cudaStreamWaitEvent(e->copy_out, sl.run_done, 0));
  OMCUDA_CHECK(cudaMemcpyAsync(omTensorGetDataPtr(y), sl.out.p, bytes,
      cudaMemcpyDeviceToHost, e->copy_out));
  OMCUDA_CHECK(cudaEventRecord(sl.out_done, e->copy_out));
  sl.used = true;
  ++e->submitted;
  return OMCUDA_OK;
}

extern "C" int omcudaEncoderWait(omcudaEncoder *e) {
  if (!e)
    return fail(OMCUDA_EINVAL, "EncoderWait: null encoder");
  if (e->copy_out) {
    for (auto &sl : e->slot)
      if (sl.used)
        OMCUDA_CHECK(cudaEventSynchronize(sl.out_done));
  }
  omcudaSynchronize(); // surfaces a bounded-wait timeout of the kernels
  return sticky_error() ? omcudaGetLastError() : OMCUDA_OK;
}

extern "C" int omcudaEncoderSetRangeSync(
    omcudaEncoder *e, omcudaRangeSyncFn fn, void *ctx) {
  if (!e)
    return fail(OMCUDA_EINVAL, "EncoderSetRangeSync: null encoder");
  e->range_sync = fn;
  e->range_sync_ctx = ctx;
  return OMCUDA_OK;
}

extern "C" int omcudaEncoderGetTapLayout(const omcudaEncoder *e, int64_t batch,
    int64_t seq, omcudaEncoderTapLayout *out) {
  if (!e || !out || batch <= 0 || seq <= 0)
    return fail(OMCUDA_EINVAL, "EncoderGetTapLayout: bad argument");
  tap_layout(e->cfg, batch * seq, out);
  return OMCUDA_OK;
}

extern "C" int omcudaEncoderSetTap(omcudaEncoder *e, void *dev_buf, int64_t bytes) {
  if (!e || (dev_buf && bytes <= 0))
    return fail(OMCUDA_EINVAL, "EncoderSetTap: bad argument");
  e->tap = (uint8_t *)dev_buf;
  e->tap_bytes = dev_buf ? bytes : 0;
  return OMCUDA_OK;
}

extern "C" void omcudaEncoderSetProfiling(omcudaEncoder *e, int on) {
  if (!e)
    return;
  e->profiling = on != 0;
  e->ev_used = 0;
  e->gemm_ops = 0.0;
}

extern "C" int omcudaEncoderGemmStats(
    omcudaEncoder *e, double *ms_total, double *ops_total, int64_t *launches) {
  if (!e || !ms_total || !ops_total || !launches)
    return fail(OMCUDA_EINVAL, "EncoderGemmStats: bad argument");
  double ms = 0.0;
  for (size_t i = 0; i + 1 < e->ev_used; i += 2) {
    OMCUDA_CHECK(cudaEventSynchronize(e->ev[i + 1]));
    float t = 0.0f;
    OMCUDA_CHECK(cudaEventElapsedTime(&t, e->ev[i], e->ev[i + 1]));
    ms += t;
  }
  *ms_total = ms;
  *ops_total = e->gemm_ops;
  *launches = (int64_t)(e->ev_used / 2);
  return OMCUDA_OK;
}

extern "C" void omcudaEncoderDestroy(omcudaEncoder *e) {
  if (!e)
    return;
  if (OMIsInitAccelCUDA)
    cudaStreamSynchronize(current_stream());
  drop_graphs(e);
  for (cudaEvent_t ev : e->ev)
    cudaEventDestroy(ev);
  for (auto &sl : e->slot) {
    if (sl.out_done)
      cudaEventSynchronize(sl.out_done);
    for (cudaEvent_t ev : {sl.in_done, sl.run_done, sl.out_done})
      if (ev)
        cudaEventDestroy(ev);
    sl.in.release();
    sl.out.release();
  }
  if (e->copy_in)
    cudaStreamDestroy(e->copy_in);
  if (e->copy_out)
    cudaStreamDestroy(e->copy_out);
  for (auto &L : e->layers) {
    DevBuf *all[] = {&L.wqkv_bt, &L.wqkv_cs, &L.wo_bt, &L.wo_cs, &L.w1_bt,
        &L.w1_cs, &L.w2_bt, &L.w2_cs, &L.qkv_scale, &L.scal, &L.bqkv, &L.bo,
        &L.b1, &L.b2, &L.ln1g, &L.ln1b, &L.ln2g, &L.ln2b};
    for (DevBuf *b : all)
      b->release();
  }
  DevBuf *ws[] = {&e->stage_in, &e->stage_out, &e->xq, &e->qkv, &e->ctx, &e->a, &e->h1, &e->f, &e->o,
      &e->ybuf[0], &e->ybuf[1], &e->ranges, &e->params, &e->dql_scratch};
  for (DevBuf *b : ws)
    b->release();
  delete e;
}
