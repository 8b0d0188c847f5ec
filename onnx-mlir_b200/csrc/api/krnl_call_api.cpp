// krnl.call-level entry points: the functions a model compiled with the CUDA
// accelerator plugin calls in place of the CPU loops.  Arguments arrive as
// non-owning OMTensor wrappers (src/Conversion/KrnlToLLVM/KrnlCall.cpp:34-226:
// outputs first, then inputs, NULL for absent optionals, integer attributes as
// int64_t, float attributes as double).  A buffer may be host or device
// memory; host buffers are staged through HBM inside the call and the call
// returns after the results are back, device buffers are used in place and the
// call returns with the work queued on the library stream.
//
// Error convention: the first failure sticks to the calling thread and sets
// errno; later calls return without doing anything, so a generated
// run_main_graph can test once before it builds its output list and return
// NULL, the way the reference reports failure
// (src/Runtime/ExecutionSession.cpp:324-362).
#include <cuda_runtime.h>

#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <tuple>
#include <vector>

#include "../common.cuh"
#include "../runtime/internal.h"

namespace omcuda {

int gemm_tc_check_status(cudaStream_t st);

namespace {

bool is_device_ptr(const void *p) {
  if (!p)
    return false;
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

int64_t dtype_bytes(OM_DATA_TYPE t) {
  switch (t) {
  case ONNX_TYPE_UINT8:
  case ONNX_TYPE_INT8:
    return 1;
  case ONNX_TYPE_UINT16: // raw bf16 planes of the attention operands
  case ONNX_TYPE_BFLOAT16:
    return 2;
  case ONNX_TYPE_FLOAT:
  case ONNX_TYPE_INT32:
    return 4;
  case ONNX_TYPE_INT64:
    return 8;
  default:
    return 0;
  }
}

// Dense row-major check: the memref a krnl.call receives normally is, but the
// callee has to verify (strides are in elements).
bool is_dense(const OMTensor *t) {
  int64_t rank = omTensorGetRank(t);
  const int64_t *shape = omTensorGetShape(t);
  const int64_t *strides = omTensorGetStrides(t);
  int64_t run = 1;
  for (int64_t i = rank - 1; i >= 0; --i) {
    if (shape[i] != 1 && strides[i] != run)
      return false;
    run *= shape[i];
  }
  return true;
}

bool same_shape(const OMTensor *a, const OMTensor *b) {
  if (omTensorGetRank(a) != omTensorGetRank(b))
    return false;
  for (int64_t i = 0; i < omTensorGetRank(a); ++i)
    if (omTensorGetShape(a)[i] != omTensorGetShape(b)[i])
      return false;
  return true;
}

// Per-call staging of host tensors and scratch.
class Stage {
public:
  explicit Stage(cudaStream_t st) : st_(st) {}
  // Temporaries go back to the pool stream-ordered: whoever takes them next
  // is queued behind the kernels of this call that still use them.
  ~Stage() {
    for (void *p : temps_)
      pool_free_on(p, st_);
  }
  // Hands a pool block to this call for release at its end.
  void adopt(void *p) {
    if (p)
      temps_.push_back(p);
  }

  bool ok() const { return rc_ == OMCUDA_OK; }
  int rc() const { return rc_; }
  void set(int rc) {
    if (rc_ == OMCUDA_OK)
      rc_ = rc;
  }

  void *scratch(size_t bytes) {
    void *p = pool_alloc_on(bytes ? bytes : 1, st_);
    if (!p) {
      set(OMCUDA_ENOMEM);
      return nullptr;
    }
    temps_.push_back(p);
    return p;
  }

  // Device pointer holding the tensor's data (copied in when it is on host).
  const void *in(const OMTensor *t) {
    if (!t)
      return nullptr;
    void *p = omTensorGetDataPtr(t);
    int64_t bytes = omTensorGetBufferSize(t);
    if (bytes == 0)
      return p;
    if (is_device_ptr(p))
      return p;
    void *d = scratch((size_t)bytes);
    if (!d)
      return nullptr;
    set(check_cuda(cudaMemcpyAsync(d, p, (size_t)bytes, cudaMemcpyHostToDevice, st_),
        "H2D copy"));
    h2d_ += bytes;
    return d;
  }

  // Device pointer the kernel writes; copied back by finish() when on host.
  void *out(OMTensor *t) {
    void *p = omTensorGetDataPtr(t);
    int64_t bytes = omTensorGetBufferSize(t);
    if (bytes == 0 || is_device_ptr(p))
      return p;
    void *d = scratch((size_t)bytes);
    if (!d)
      return nullptr;
    outs_.push_back({p, d, (size_t)bytes});
    return d;
  }

  int finish(bool check_gemm) {
    if (!ok())
      return rc_;
    for (auto &o : outs_)
      set(check_cuda(cudaMemcpyAsync(o.host, o.dev, o.bytes,
                         cudaMemcpyDeviceToHost, st_),
          "D2H copy"));
    if (!outs_.empty()) {
      if (check_gemm)
        set(gemm_tc_check_status(st_)); // synchronises
      else
        set(check_cuda(cudaStreamSynchronize(st_), "cudaStreamSynchronize"));
    }
    return rc_;
  }

private:
  struct Out {
    void *host;
    void *dev;
    size_t bytes;
  };
  cudaStream_t st_;
  int rc_ = OMCUDA_OK;
  std::vector<void *> temps_;
  std::vector<Out> outs_;
  int64_t h2d_ = 0;
};

// ---- DynamicQuantizeLinear scratch ------------------------------------------------------
//
// One block per call (not per stream): two host threads may interleave their
// launches on the shared library stream, and the reduction leaves the scale
// and zero point in its scratch for the quantize pass that follows.

void *dql_scratch_for(Stage &sg, cudaStream_t st) {
  void *p = sg.scratch((size_t)omcudaDevDqlScratchBytes(0));
  if (!p)
    return nullptr;
  // Only the ticket line has to start at zero.
  if (check_cuda(cudaMemsetAsync(p, 0, 64, st), "cudaMemsetAsync(dql scratch)") != OMCUDA_OK)
    return nullptr;
  return p;
}

// ---- constants: prepared B operands cached by buffer ----------------------------------

struct PreparedEntry {
  omcudaPreparedB pb;
  cudaStream_t stream; // where the prepare kernels ran
  cudaEvent_t ready;   // recorded behind them
};
std::mutex g_const_mutex;
std::set<const void *> g_const_ptrs;
std::map<std::tuple<const void *, int64_t, int64_t, int>, PreparedEntry> g_prepared;

bool is_registered_constant(const void *p) {
  std::lock_guard<std::mutex> lock(g_const_mutex);
  return g_const_ptrs.count(p) != 0;
}

// Returns a prepared form of B ([K,N], 8-bit).  `key_ptr` is the tensor's own
// pointer (the cache key); `b_dev` the staged device copy.  A cache hit from a
// stream other than the one that prepared the entry first waits for that
// prepare to finish.
int prepared_b(Stage &sg, const void *key_ptr, const void *b_dev, int b_signed,
    int64_t K, int64_t N, cudaStream_t st, omcudaPreparedB *out) {
  bool cacheable = is_registered_constant(key_ptr);
  auto key = std::make_tuple(key_ptr, K, N, b_signed);
  if (cacheable) {
    std::lock_guard<std::mutex> lock(g_const_mutex);
    auto it = g_prepared.find(key);
    if (it != g_prepared.end()) {
      if (it->second.stream != st && it->second.ready)
        OMCUDA_CHECK(cudaStreamWaitEvent(st, it->second.ready, 0));
      *out = it->second.pb;
      return OMCUDA_OK;
    }
  }
  int64_t kp;
  int64_t bytes = omcudaDevPreparedBBytes(K, N, &kp);
  omcudaPreparedB pb;
  memset(&pb, 0, sizeof(pb));
  if (cacheable) {
    pb.bt = pool_alloc_on((size_t)bytes, st);
    pb.colsum = (int32_t *)pool_alloc_on((size_t)N * sizeof(int32_t), st);
  } else {
    pb.bt = sg.scratch((size_t)bytes);
    pb.colsum = (int32_t *)sg.scratch((size_t)N * sizeof(int32_t));
  }
  if (!pb.bt || !pb.colsum) {
    if (cacheable) {
      sg.adopt(pb.bt);
      sg.adopt(pb.colsum);
    }
    return OMCUDA_ENOMEM;
  }
  int rc = omcudaDevPrepareB(b_dev, b_signed, K, N, &pb, st);
  if (rc != OMCUDA_OK) {
    if (cacheable) {
      sg.adopt(pb.bt);
      sg.adopt(pb.colsum);
    }
    return rc;
  }
  if (cacheable) {
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventRecord(ev, st) != cudaSuccess) {
      (void)cudaGetLastError();
      if (ev)
        cudaEventDestroy(ev);
      ev = nullptr;
      // no event to order other streams behind: finish the prepare now
      OMCUDA_CHECK(cudaStreamSynchronize(st));
    }
    std::lock_guard<std::mutex> lock(g_const_mutex);
    if (g_prepared.count(key)) {
      // Another thread prepared the same constant meanwhile: use ours for this
      // call only and give it back at the end of the call.
      sg.adopt(pb.bt);
      sg.adopt(pb.colsum);
      if (ev)
        cudaEventDestroy(ev);
    } else {
      g_prepared[key] = PreparedEntry{pb, st, ev};
    }
  }
  *out = pb;
  return OMCUDA_OK;
}

bool begin_call() { return !sticky_error() && ensure_init() == OMCUDA_OK; }

// numpy-style matmul shapes (src/Dialect/ONNX/ONNXOps/Math/MatMul.cpp:46-166):
// a 1-D A is a row vector, a 1-D B a column vector, and the leading (batch)
// dimensions of A [.., M, K] and B [.., K, N] broadcast against each other.
// The result is a list of 2-D products: product i reads A at element offset
// a_off[i], B at b_off[i] and writes Y at i * M * N.  An unbatched B folds all
// of A's leading dimensions into M (one product).
struct MatDims {
  int64_t batch, M, K, N;
  bool b_batched;
  std::vector<int64_t> a_off, b_off;
};

int matmul_dims(const OMTensor *A, const OMTensor *B, MatDims *d) {
  int64_t ra = omTensorGetRank(A), rb = omTensorGetRank(B);
  const int64_t *sa = omTensorGetShape(A), *sb = omTensorGetShape(B);
  if (ra < 1 || rb < 1)
    return fail(OMCUDA_EINVAL, "matmul: rank-0 operand");
  d->K = sa[ra - 1];
  int64_t kb = (rb == 1) ? sb[0] : sb[rb - 2];
  d->N = (rb == 1) ? 1 : sb[rb - 1];
  if (kb != d->K)
    return fail(OMCUDA_EINVAL, "matmul: inner dimensions differ (%lld vs %lld)",
        (long long)d->K, (long long)kb);
  d->a_off.assign(1, 0);
  d->b_off.assign(1, 0);
  if (rb <= 2) {
    int64_t rows = 1;
    for (int64_t i = 0; i + 1 < ra; ++i)
      rows *= sa[i];
    d->batch = 1;
    d->M = rows;
    d->b_batched = false;
    return OMCUDA_OK;
  }
  // Batch dimensions, right-aligned: A's are sa[0 .. ra-2) (none for a vector),
  // B's are sb[0 .. rb-2).
  const int64_t na = ra >= 2 ? ra - 2 : 0, nb = rb - 2;
  const int64_t nd = na > nb ? na : nb;
  d->M = ra >= 2 ? sa[ra - 2] : 1;
  std::vector<int64_t> dims((size_t)nd), astr((size_t)nd), bstr((size_t)nd);
  int64_t arun = d->M * d->K, brun = d->K * d->N, batch = 1;
  for (int64_t i = nd - 1; i >= 0; --i) {
    const int64_t ia = i - (nd - na), ib = i - (nd - nb);
    const int64_t da = ia >= 0 ? sa[ia] : 1, db = ib >= 0 ? sb[ib] : 1;
    if (da != db && da != 1 && db != 1)
      return fail(OMCUDA_EINVAL, "matmul: batch dimensions %lld and %lld do not broadcast",
          (long long)da, (long long)db);
    dims[(size_t)i] = da == 1 ? db : da;
    astr[(size_t)i] = da == 1 ? 0 : arun; // a broadcast dimension does not advance
    bstr[(size_t)i] = db == 1 ? 0 : brun;
    arun *= da;
    brun *= db;
    batch *= dims[(size_t)i];
  }
  d->batch = batch;
  d->b_batched = true;
  d->a_off.assign((size_t)batch, 0);
  d->b_off.assign((size_t)batch, 0);
  for (int64_t i = 0; i < batch; ++i) {
    int64_t rem = i, ao = 0, bo = 0;
    for (int64_t k = nd - 1; k >= 0; --k) {
      const int64_t idx = rem % dims[(size_t)k];
      rem /= dims[(size_t)k];
      ao += idx * astr[(size_t)k];
      bo += idx * bstr[(size_t)k];
    }
    d->a_off[(size_t)i] = ao;
    d->b_off[(size_t)i] = bo;
  }
  return OMCUDA_OK;
}

bool is_8bit(OM_DATA_TYPE t) { return t == ONNX_TYPE_UINT8 || t == ONNX_TYPE_INT8; }

} // namespace

} // namespace omcuda

using namespace omcuda;

extern "C" {

// ---- device tensors --------------------------------------------------------------------

OMTensor *omcudaTensorCreateOnDevice(
    const int64_t *shape, int64_t rank, OM_DATA_TYPE dtype) {
  if (ensure_init() != OMCUDA_OK)
    return nullptr;
  int64_t esz = dtype_bytes(dtype);
  if (esz == 0 || rank < 0 || (rank > 0 && !shape)) {
    fail(OMCUDA_EINVAL, "omcudaTensorCreateOnDevice: unsupported dtype or shape");
    return nullptr;
  }
  int64_t n = 1;
  for (int64_t i = 0; i < rank; ++i)
    n *= shape[i];
  void *d = pool_alloc((size_t)(n * esz));
  if (!d)
    return nullptr;
  OMTensor *t = omTensorCreate(d, shape, rank, dtype);
  if (!t)
    pool_free(d);
  return t;
}

OMTensor *omcudaTensorToDevice(const OMTensor *src) {
  if (!src)
    return nullptr;
  OMTensor *t = omcudaTensorCreateOnDevice(
      omTensorGetShape(src), omTensorGetRank(src), omTensorGetDataType(src));
  if (!t)
    return nullptr;
  int64_t bytes = omTensorGetBufferSize(src);
  if (bytes > 0 &&
      check_cuda(cudaMemcpyAsync(omTensorGetDataPtr(t), omTensorGetDataPtr(src),
                     (size_t)bytes, cudaMemcpyDefault, current_stream()),
          "copy to device") != OMCUDA_OK) {
    omcudaTensorDestroy(t);
    return nullptr;
  }
  return t;
}

OMTensor *omcudaTensorToHost(const OMTensor *src) {
  if (!src || ensure_init() != OMCUDA_OK)
    return nullptr;
  OMTensor *t = omTensorCreateEmpty(
      omTensorGetShape(src), omTensorGetRank(src), omTensorGetDataType(src));
  if (!t) {
    fail(OMCUDA_ENOMEM, "omcudaTensorToHost: host allocation failed");
    return nullptr;
  }
  int64_t bytes = omTensorGetBufferSize(src);
  cudaStream_t st = current_stream();
  if (bytes > 0 &&
      (check_cuda(cudaMemcpyAsync(omTensorGetDataPtr(t), omTensorGetDataPtr(src),
                      (size_t)bytes, cudaMemcpyDefault, st),
           "copy to host") != OMCUDA_OK ||
          gemm_tc_check_status(st) != OMCUDA_OK)) {
    omTensorDestroy(t);
    return nullptr;
  }
  return t;
}

void omcudaTensorDestroy(OMTensor *t) {
  if (!t)
    return;
  void *p = omTensorGetAllocatedPtr(t);
  if (pool_owns(p)) {
    pool_free(p);
    omTensorSetOwning(t, 0);
  }
  omTensorDestroy(t);
}

int omcudaTensorIsOnDevice(const OMTensor *t) {
  return t && is_device_ptr(omTensorGetDataPtr(t)) ? 1 : 0;
}

void omcudaRegisterConstant(const OMTensor *t) {
  if (!t)
    return;
  std::lock_guard<std::mutex> lock(g_const_mutex);
  g_const_ptrs.insert(omTensorGetDataPtr(t));
}

void omcudaForgetConstants(void) {
  std::lock_guard<std::mutex> lock(g_const_mutex);
  for (auto &kv : g_prepared) {
    if (kv.second.ready) {
      cudaEventSynchronize(kv.second.ready);
      cudaEventDestroy(kv.second.ready);
    }
    pool_free(kv.second.pb.bt);
    pool_free(kv.second.pb.colsum);
  }
  g_prepared.clear();
  g_const_ptrs.clear();
}

// ---- DynamicQuantizeLinear / QuantizeLinear / DequantizeLinear -------------------------------

void omcudaDynamicQuantizeLinear(
    OMTensor *y, OMTensor *yScale, OMTensor *yZp, const OMTensor *x) {
  if (!begin_call())
    return;
  if (!y || !yScale || !yZp || !x) {
    fail(OMCUDA_EINVAL, "DynamicQuantizeLinear: NULL tensor");
    return;
  }
  if (omTensorGetDataType(x) != ONNX_TYPE_FLOAT ||
      omTensorGetDataType(y) != ONNX_TYPE_UINT8 ||
      omTensorGetDataType(yScale) != ONNX_TYPE_FLOAT ||
      omTensorGetDataType(yZp) != ONNX_TYPE_UINT8) {
    fail(OMCUDA_EINVAL, "DynamicQuantizeLinear: expected f32 -> (u8, f32, u8)");
    return;
  }
  if (!same_shape(x, y) || omTensorGetNumElems(yScale) != 1 ||
      omTensorGetNumElems(yZp) != 1) {
    fail(OMCUDA_EINVAL, "DynamicQuantizeLinear: shape mismatch");
    return;
  }
  if (!is_dense(x) || !is_dense(y)) {
    fail(OMCUDA_ENOTSUP, "DynamicQuantizeLinear: non-contiguous tensor");
    return;
  }
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *dx = (const float *)sg.in(x);
  uint8_t *dy = (uint8_t *)sg.out(y);
  float *ds = (float *)sg.out(yScale);
  uint8_t *dz = (uint8_t *)sg.out(yZp);
  void *scr = dql_scratch_for(sg, st);
  if (!sg.ok() || !scr)
    return;
  sg.set(omcudaDevDynamicQuantizeLinear(
      dx, omTensorGetNumElems(x), dy, ds, dz, scr, st));
  sg.finish(false);
}

void omcudaQuantizeLinear(OMTensor *y, const OMTensor *x, const OMTensor *scale,
    const OMTensor *zp) {
  if (!begin_call())
    return;
  if (!y || !x || !scale) {
    fail(OMCUDA_EINVAL, "QuantizeLinear: NULL tensor");
    return;
  }
  OM_DATA_TYPE yt = omTensorGetDataType(y);
  if (omTensorGetDataType(x) != ONNX_TYPE_FLOAT || !is_8bit(yt) ||
      omTensorGetDataType(scale) != ONNX_TYPE_FLOAT ||
      (zp && omTensorGetDataType(zp) != yt)) {
    fail(OMCUDA_EINVAL, "QuantizeLinear: expected f32 -> u8/i8 with f32 scale");
    return;
  }
  // Per-axis quantization is rejected by the reference's lowering as well
  // (QuantizeLinear.cpp:192-193).
  if (omTensorGetNumElems(scale) != 1 || (zp && omTensorGetNumElems(zp) != 1)) {
    fail(OMCUDA_ENOTSUP, "QuantizeLinear: per-axis scale is not supported");
    return;
  }
  if (!same_shape(x, y) || !is_dense(x) || !is_dense(y)) {
    fail(OMCUDA_EINVAL, "QuantizeLinear: shape mismatch or non-contiguous");
    return;
  }
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *dx = (const float *)sg.in(x);
  const float *dsc = (const float *)sg.in(scale);
  const void *dzp = sg.in(zp);
  void *dy = sg.out(y);
  if (!sg.ok())
    return;
  sg.set(omcudaDevQuantizeLinear(dx, omTensorGetNumElems(x), dy,
      yt == ONNX_TYPE_INT8, dsc, dzp, st));
  sg.finish(false);
}

void omcudaDequantizeLinear(OMTensor *y, const OMTensor *x,
    const OMTensor *scale, const OMTensor *zp) {
  if (!begin_call())
    return;
  if (!y || !x || !scale) {
    fail(OMCUDA_EINVAL, "DequantizeLinear: NULL tensor");
    return;
  }
  OM_DATA_TYPE xt = omTensorGetDataType(x);
  int code = xt == ONNX_TYPE_UINT8 ? 0 : xt == ONNX_TYPE_INT8 ? 1
             : xt == ONNX_TYPE_INT32 ? 2 : -1;
  if (code < 0 || omTensorGetDataType(y) != ONNX_TYPE_FLOAT ||
      omTensorGetDataType(scale) != ONNX_TYPE_FLOAT ||
      (zp && omTensorGetDataType(zp) != xt)) {
    fail(OMCUDA_EINVAL, "DequantizeLinear: expected u8/i8/i32 -> f32");
    return;
  }
  if (omTensorGetNumElems(scale) != 1 || (zp && omTensorGetNumElems(zp) != 1)) {
    fail(OMCUDA_ENOTSUP, "DequantizeLinear: per-axis scale is not supported");
    return;
  }
  if (!same_shape(x, y) || !is_dense(x) || !is_dense(y)) {
    fail(OMCUDA_EINVAL, "DequantizeLinear: shape mismatch or non-contiguous");
    return;
  }
  cudaStream_t st = current_stream();
  Stage sg(st);
  const void *dx = sg.in(x);
  const float *dsc = (const float *)sg.in(scale);
  const void *dzp = sg.in(zp);
  float *dy = (float *)sg.out(y);
  if (!sg.ok())
    return;
  sg.set(omcudaDevDequantizeLinear(
      dx, code, omTensorGetNumElems(x), dsc, dzp, dy, st));
  sg.finish(false);
}

// ---- MatMulInteger ----------------------------------------------------------------------------

void omcudaMatMulInteger(OMTensor *Y, const OMTensor *A, const OMTensor *B,
    const OMTensor *aZp, const OMTensor *bZp) {
  if (!begin_call())
    return;
  if (!Y || !A || !B) {
    fail(OMCUDA_EINVAL, "MatMulInteger: NULL tensor");
    return;
  }
  OM_DATA_TYPE at = omTensorGetDataType(A), bt = omTensorGetDataType(B);
  if (!is_8bit(at) || !is_8bit(bt) || omTensorGetDataType(Y) != ONNX_TYPE_INT32 ||
      (aZp && omTensorGetDataType(aZp) != at) ||
      (bZp && omTensorGetDataType(bZp) != bt)) {
    fail(OMCUDA_EINVAL, "MatMulInteger: expected 8-bit operands and i32 result");
    return;
  }
  if (!is_dense(A) || !is_dense(B) || !is_dense(Y)) {
    fail(OMCUDA_ENOTSUP, "MatMulInteger: non-contiguous tensor");
    return;
  }
  MatDims d;
  if (matmul_dims(A, B, &d) != OMCUDA_OK)
    return;
  if (omTensorGetNumElems(Y) != d.batch * d.M * d.N) {
    fail(OMCUDA_EINVAL, "MatMulInteger: result has the wrong number of elements");
    return;
  }
  int64_t azn = aZp ? omTensorGetNumElems(aZp) : 0;
  int64_t bzn = bZp ? omTensorGetNumElems(bZp) : 0;
  // a_zero_point: scalar, [1], or one per row of a 2-D A (MatMulInteger.cpp:64-74).
  if (azn > 1 && !(d.batch == 1 && azn == d.M && omTensorGetRank(A) == 2)) {
    fail(OMCUDA_ENOTSUP, "MatMulInteger: a_zero_point must be scalar or [M]");
    return;
  }
  if (bzn > 1 && bzn != d.N) {
    fail(OMCUDA_EINVAL, "MatMulInteger: b_zero_point must be scalar or [N]");
    return;
  }
  if (omTensorGetNumElems(Y) == 0)
    return;
  cudaStream_t st = current_stream();
  Stage sg(st);
  const uint8_t *dA = (const uint8_t *)sg.in(A);
  const uint8_t *dB = (const uint8_t *)sg.in(B);
  const void *dAz = sg.in(aZp);
  const void *dBz = sg.in(bZp);
  int32_t *dY = (int32_t *)sg.out(Y);
  if (!sg.ok())
    return;
  // A B slice that several products share (a broadcast batch dimension) is
  // prepared once.
  std::map<int64_t, omcudaPreparedB> prepared;
  for (int64_t b = 0; b < d.batch && sg.ok(); ++b) {
    omcudaGemmArgs g;
    memset(&g, 0, sizeof(g));
    g.M = d.M;
    g.N = d.N;
    g.K = d.K;
    g.A = dA + d.a_off[(size_t)b];
    g.a_signed = at == ONNX_TYPE_INT8;
    const int64_t bo = d.b_off[(size_t)b];
    auto hit = prepared.find(bo);
    if (hit != prepared.end()) {
      g.B = hit->second;
    } else {
      const void *key = (const uint8_t *)omTensorGetDataPtr(B) + bo;
      sg.set(prepared_b(sg, key, dB + bo, bt == ONNX_TYPE_INT8, d.K, d.N, st, &g.B));
      if (!sg.ok())
        break;
      prepared[bo] = g.B;
    }
    g.a_zp = dAz;
    g.a_zp_len = azn;
    g.b_zp = dBz;
    g.b_zp_len = bzn;
    if (bzn) {
      int32_t *rs = (int32_t *)sg.scratch((size_t)d.M * sizeof(int32_t));
      if (!rs)
        break;
      sg.set(omcudaDevRowSum(g.A, g.a_signed, d.M, d.K, rs, st));
      g.a_rowsum = rs;
    }
    g.epilogue = OMCUDA_EPI_I32;
    g.Y = dY + b * d.M * d.N;
    sg.set(omcudaDevGemmI8(&g, st));
  }
  sg.finish(true);
}

// ---- QLinearMatMul ----------------------------------------------------------------------------------

void omcudaQLinearMatMul(OMTensor *y, const OMTensor *a, const OMTensor *aScale,
    const OMTensor *aZp, const OMTensor *b, const OMTensor *bScale,
    const OMTensor *bZp, const OMTensor *yScale, const OMTensor *yZp) {
  if (!begin_call())
    return;
  if (!y || !a || !aScale || !aZp || !b || !bScale || !bZp || !yScale || !yZp) {
    fail(OMCUDA_EINVAL, "QLinearMatMul: NULL tensor");
    return;
  }
  OM_DATA_TYPE at = omTensorGetDataType(a), bt = omTensorGetDataType(b),
               yt = omTensorGetDataType(y);
  // The reference's pattern only fires for 8-bit tensors and f32 scales
  // (QLinearMatMul.cpp:53-68).
  if (!is_8bit(at) || !is_8bit(bt) || !is_8bit(yt) ||
      omTensorGetDataType(aZp) != at || omTensorGetDataType(bZp) != bt ||
      omTensorGetDataType(yZp) != yt ||
      omTensorGetDataType(aScale) != ONNX_TYPE_FLOAT ||
      omTensorGetDataType(bScale) != ONNX_TYPE_FLOAT ||
      omTensorGetDataType(yScale) != ONNX_TYPE_FLOAT) {
    fail(OMCUDA_EINVAL, "QLinearMatMul: expected 8-bit tensors and f32 scales");
    return;
  }
  if (!is_dense(a) || !is_dense(b) || !is_dense(y)) {
    fail(OMCUDA_ENOTSUP, "QLinearMatMul: non-contiguous tensor");
    return;
  }
  MatDims d;
  if (matmul_dims(a, b, &d) != OMCUDA_OK)
    return;
  if (d.b_batched) {
    fail(OMCUDA_ENOTSUP, "QLinearMatMul: batched B is not supported");
    return;
  }
  if (omTensorGetNumElems(y) != d.M * d.N) {
    fail(OMCUDA_EINVAL, "QLinearMatMul: result has the wrong number of elements");
    return;
  }
  int64_t bsn = omTensorGetNumElems(bScale), bzn = omTensorGetNumElems(bZp);
  if (omTensorGetNumElems(aScale) != 1 || omTensorGetNumElems(aZp) != 1 ||
      omTensorGetNumElems(yScale) != 1 || omTensorGetNumElems(yZp) != 1 ||
      (bsn != 1 && bsn != d.N) || (bzn != 1 && bzn != d.N)) {
    fail(OMCUDA_ENOTSUP,
        "QLinearMatMul: a/y quantization must be per-tensor, b per-tensor or "
        "per-column");
    return;
  }
  if (omTensorGetNumElems(y) == 0)
    return;
  cudaStream_t st = current_stream();
  Stage sg(st);
  const uint8_t *dA = (const uint8_t *)sg.in(a);
  const uint8_t *dB = (const uint8_t *)sg.in(b);
  const float *dAs = (const float *)sg.in(aScale);
  const float *dBs = (const float *)sg.in(bScale);
  const float *dYs = (const float *)sg.in(yScale);
  const void *dAz = sg.in(aZp);
  const void *dBz = sg.in(bZp);
  void *dY = sg.out(y);
  // The output zero point enters the epilogue as an immediate.
  int32_t yzp = 0;
  {
    uint8_t raw = 0;
    const void *p = omTensorGetDataPtr(yZp);
    if (is_device_ptr(p))
      sg.set(check_cuda(cudaMemcpyAsync(&raw, p, 1, cudaMemcpyDeviceToHost, st),
          "read y_zero_point")),
          sg.set(check_cuda(cudaStreamSynchronize(st), "sync"));
    else
      raw = *(const uint8_t *)p;
    yzp = (yt == ONNX_TYPE_INT8) ? (int32_t)(int8_t)raw : (int32_t)raw;
  }
  if (!sg.ok())
    return;
  omcudaGemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = d.M;
  g.N = d.N;
  g.K = d.K;
  g.A = dA;
  g.a_signed = at == ONNX_TYPE_INT8;
  sg.set(prepared_b(sg, omTensorGetDataPtr(b), dB, bt == ONNX_TYPE_INT8, d.K, d.N,
      st, &g.B));
  float *S = (float *)sg.scratch((size_t)bsn * sizeof(float));
  if (!sg.ok() || !S)
    return;
  sg.set(omcudaDevRequantScale(dAs, dBs, bsn, dYs, S, st));
  g.a_zp = dAz;
  g.a_zp_len = 1;
  g.b_zp = dBz;
  g.b_zp_len = bzn;
  int32_t *rs = (int32_t *)sg.scratch((size_t)d.M * sizeof(int32_t));
  if (!rs)
    return;
  sg.set(omcudaDevRowSum(dA, g.a_signed, d.M, d.K, rs, st));
  g.a_rowsum = rs;
  g.epilogue = OMCUDA_EPI_REQUANT;
  g.Y = dY;
  g.sb = S;
  g.sb_len = bsn;
  g.y_zp = yzp;
  g.y_signed = yt == ONNX_TYPE_INT8;
  if (sg.ok())
    sg.set(omcudaDevGemmI8(&g, st));
  sg.finish(true);
}

// ---- fused dynamic-quantized linear ---------------------------------------------------------------------

void omcudaDynQuantLinear(OMTensor *Y, const OMTensor *X, const OMTensor *Wq,
    const OMTensor *wScale, const OMTensor *wZp, const OMTensor *bias,
    int64_t scaleForm) {
  if (!begin_call())
    return;
  if (!Y || !X || !Wq || !wScale) {
    fail(OMCUDA_EINVAL, "DynQuantLinear: NULL tensor");
    return;
  }
  OM_DATA_TYPE wt = omTensorGetDataType(Wq);
  if (omTensorGetDataType(X) != ONNX_TYPE_FLOAT ||
      omTensorGetDataType(Y) != ONNX_TYPE_FLOAT || !is_8bit(wt) ||
      omTensorGetDataType(wScale) != ONNX_TYPE_FLOAT ||
      (wZp && omTensorGetDataType(wZp) != wt) ||
      (bias && omTensorGetDataType(bias) != ONNX_TYPE_FLOAT) ||
      (scaleForm != 0 && scaleForm != 1)) {
    fail(OMCUDA_EINVAL, "DynQuantLinear: dtype or attribute mismatch");
    return;
  }
  if (omTensorGetRank(Wq) != 2 || omTensorGetRank(X) < 1 || !is_dense(X) ||
      !is_dense(Wq) || !is_dense(Y)) {
    fail(OMCUDA_ENOTSUP, "DynQuantLinear: need dense X [..,K] and W [K,N]");
    return;
  }
  MatDims d;
  if (matmul_dims(X, Wq, &d) != OMCUDA_OK)
    return;
  int64_t wsn = omTensorGetNumElems(wScale);
  int64_t wzn = wZp ? omTensorGetNumElems(wZp) : 0;
  if (omTensorGetNumElems(Y) != d.M * d.N || (wsn != 1 && wsn != d.N) ||
      (wzn > 1 && wzn != d.N) || (bias && omTensorGetNumElems(bias) != d.N)) {
    fail(OMCUDA_EINVAL, "DynQuantLinear: shape mismatch");
    return;
  }
  if (omTensorGetNumElems(Y) == 0)
    return;
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *dX = (const float *)sg.in(X);
  const uint8_t *dW = (const uint8_t *)sg.in(Wq);
  const float *dWs = (const float *)sg.in(wScale);
  const void *dWz = sg.in(wZp);
  const float *dBias = (const float *)sg.in(bias);
  float *dY = (float *)sg.out(Y);
  uint8_t *xq = (uint8_t *)sg.scratch((size_t)(d.M * d.K));
  float *xs = (float *)sg.scratch(16);
  void *scr = dql_scratch_for(sg, st);
  if (!sg.ok() || !scr)
    return;
  uint8_t *xz = (uint8_t *)(xs + 1);
  sg.set(omcudaDevDynamicQuantizeLinear(dX, d.M * d.K, xq, xs, xz, scr, st));
  omcudaGemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = d.M;
  g.N = d.N;
  g.K = d.K;
  g.A = xq;
  g.a_signed = 0;
  if (sg.ok())
    sg.set(prepared_b(sg, omTensorGetDataPtr(Wq), dW, wt == ONNX_TYPE_INT8, d.K,
        d.N, st, &g.B));
  g.a_zp = xz;
  g.a_zp_len = 1;
  if (wzn) {
    g.b_zp = dWz;
    g.b_zp_len = wzn;
    int32_t *rs = (int32_t *)sg.scratch((size_t)d.M * sizeof(int32_t));
    if (!rs)
      return;
    if (sg.ok())
      sg.set(omcudaDevRowSum(xq, 0, d.M, d.K, rs, st));
    g.a_rowsum = rs;
  }
  g.epilogue = OMCUDA_EPI_DEQUANT;
  g.Y = dY;
  g.sa = xs;
  g.sb = dWs;
  g.sb_len = wsn;
  g.scale_form = (int)scaleForm;
  g.bias = dBias;
  if (sg.ok())
    sg.set(omcudaDevGemmI8(&g, st));
  sg.finish(true);
}

// ---- fp32 encoder ops ----------------------------------------------------------------------------------------

static bool f32_dense(const OMTensor *t) {
  return t && omTensorGetDataType(t) == ONNX_TYPE_FLOAT && is_dense(t);
}

void omcudaSoftmax(OMTensor *y, const OMTensor *x, int64_t axis) {
  if (!begin_call())
    return;
  if (!f32_dense(x) || !f32_dense(y) || !same_shape(x, y) ||
      omTensorGetRank(x) < 1) {
    fail(OMCUDA_EINVAL, "Softmax: expected dense f32 tensors of equal shape");
    return;
  }
  int64_t rank = omTensorGetRank(x);
  if (axis < 0)
    axis += rank;
  if (axis != rank - 1) {
    fail(OMCUDA_ENOTSUP, "Softmax: only the last axis is supported");
    return;
  }
  int64_t cols = omTensorGetShape(x)[rank - 1];
  int64_t rows = cols ? omTensorGetNumElems(x) / cols : 0;
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *dx = (const float *)sg.in(x);
  float *dy = (float *)sg.out(y);
  if (!sg.ok())
    return;
  if (rows > 0)
    sg.set(omcudaDevSoftmax(dx, rows, cols, dy, st));
  sg.finish(false);
}

void omcudaLayerNormalization(OMTensor *y, const OMTensor *x,
    const OMTensor *scale, const OMTensor *bias, int64_t axis, double epsilon) {
  if (!begin_call())
    return;
  if (!f32_dense(x) || !f32_dense(y) || !f32_dense(scale) ||
      (bias && !f32_dense(bias)) || !same_shape(x, y) || omTensorGetRank(x) < 1) {
    fail(OMCUDA_EINVAL, "LayerNormalization: expected dense f32 tensors");
    return;
  }
  int64_t rank = omTensorGetRank(x);
  if (axis < 0)
    axis += rank;
  int64_t cols = omTensorGetShape(x)[rank - 1];
  if (axis != rank - 1 || omTensorGetNumElems(scale) != cols ||
      (bias && omTensorGetNumElems(bias) != cols)) {
    fail(OMCUDA_ENOTSUP, "LayerNormalization: only the last axis with [C] params");
    return;
  }
  int64_t rows = cols ? omTensorGetNumElems(x) / cols : 0;
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *dx = (const float *)sg.in(x);
  const float *dg = (const float *)sg.in(scale);
  const float *db = (const float *)sg.in(bias);
  float *dy = (float *)sg.out(y);
  if (!sg.ok())
    return;
  if (rows > 0)
    sg.set(omcudaDevLayerNorm(
        dx, nullptr, rows, cols, dg, db, (float)epsilon, dy, nullptr, st));
  sg.finish(false);
}

void omcudaGelu(OMTensor *y, const OMTensor *x) {
  if (!begin_call())
    return;
  if (!f32_dense(x) || !f32_dense(y) || !same_shape(x, y)) {
    fail(OMCUDA_EINVAL, "Gelu: expected dense f32 tensors of equal shape");
    return;
  }
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *dx = (const float *)sg.in(x);
  float *dy = (float *)sg.out(y);
  if (!sg.ok())
    return;
  sg.set(omcudaDevGelu(dx, omTensorGetNumElems(x), dy, st));
  sg.finish(false);
}

void omcudaAdd(OMTensor *y, const OMTensor *a, const OMTensor *b) {
  if (!begin_call())
    return;
  if (!f32_dense(a) || !f32_dense(b) || !f32_dense(y) || !same_shape(a, b) ||
      !same_shape(a, y)) {
    fail(OMCUDA_EINVAL, "Add: expected dense f32 tensors of equal shape");
    return;
  }
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *da = (const float *)sg.in(a);
  const float *db = (const float *)sg.in(b);
  float *dy = (float *)sg.out(y);
  if (!sg.ok())
    return;
  sg.set(omcudaDevAdd(da, db, omTensorGetNumElems(a), dy, st));
  sg.finish(false);
}

void omcudaTranspose0213(OMTensor *y, const OMTensor *x) {
  if (!begin_call())
    return;
  if (!f32_dense(x) || !f32_dense(y) || omTensorGetRank(x) != 4 ||
      omTensorGetRank(y) != 4) {
    fail(OMCUDA_EINVAL, "Transpose: expected dense rank-4 f32 tensors");
    return;
  }
  const int64_t *s = omTensorGetShape(x), *o = omTensorGetShape(y);
  if (o[0] != s[0] || o[1] != s[2] || o[2] != s[1] || o[3] != s[3]) {
    fail(OMCUDA_EINVAL, "Transpose: output shape is not the (0,2,1,3) permutation");
    return;
  }
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *dx = (const float *)sg.in(x);
  float *dy = (float *)sg.out(y);
  if (!sg.ok())
    return;
  sg.set(omcudaDevTranspose0213(dx, s[0], s[1], s[2], s[3], dy, st));
  sg.finish(false);
}

void omcudaMatMulF32(OMTensor *y, const OMTensor *a, const OMTensor *b) {
  if (!begin_call())
    return;
  if (!f32_dense(a) || !f32_dense(b) || !f32_dense(y)) {
    fail(OMCUDA_EINVAL, "MatMul: expected dense f32 tensors");
    return;
  }
  MatDims d;
  if (matmul_dims(a, b, &d) != OMCUDA_OK)
    return;
  if (omTensorGetNumElems(y) != d.batch * d.M * d.N) {
    fail(OMCUDA_EINVAL, "MatMul: result has the wrong number of elements");
    return;
  }
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *da = (const float *)sg.in(a);
  const float *db = (const float *)sg.in(b);
  float *dy = (float *)sg.out(y);
  if (!sg.ok())
    return;
  bool uniform = true; // equal batch dimensions on both sides: one launch
  for (int64_t b = 0; b < d.batch; ++b)
    uniform = uniform && d.a_off[(size_t)b] == b * d.M * d.K &&
              d.b_off[(size_t)b] == b * d.K * d.N;
  if (uniform) {
    sg.set(omcudaDevMatMulF32(da, db, d.batch, d.M, d.N, d.K, dy, st));
  } else {
    for (int64_t b = 0; b < d.batch && sg.ok(); ++b)
      sg.set(omcudaDevMatMulF32(da + d.a_off[(size_t)b], db + d.b_off[(size_t)b], 1,
          d.M, d.N, d.K, dy + b * d.M * d.N, st));
  }
  sg.finish(false);
}

void omcudaAttention(OMTensor *y, const OMTensor *q, const OMTensor *k,
    const OMTensor *v, int64_t heads, double scale) {
  if (!begin_call())
    return;
  if (!f32_dense(q) || !f32_dense(k) || !f32_dense(v) || !f32_dense(y) ||
      omTensorGetRank(q) != 3 || !same_shape(q, k) || !same_shape(q, v) ||
      !same_shape(q, y) || heads <= 0 || omTensorGetShape(q)[2] % heads != 0) {
    fail(OMCUDA_EINVAL, "Attention: expected dense f32 [B,S,heads*dh] tensors");
    return;
  }
  const int64_t *s = omTensorGetShape(q);
  cudaStream_t st = current_stream();
  Stage sg(st);
  const float *dq = (const float *)sg.in(q);
  const float *dk = (const float *)sg.in(k);
  const float *dv = (const float *)sg.in(v);
  float *dy = (float *)sg.out(y);
  if (!sg.ok())
    return;
  const int64_t B = s[0], S = s[1], H = s[2], dh = H / heads, T = B * S;
  // (the tensor-core kernel needs a positive finite scale; any other constant
  // of the graph's Mul goes to the fp32 kernels, which scale before the max)
  const bool tc_scale = scale > 0.0 && (float)scale < INFINITY;
  if (tc_scale && omcudaDevAttentionBf16Supported(B, S, heads, dh, 3 * H, H) &&
      ((((uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv | (uintptr_t)dy) & 15u) == 0)) {
    // Tensor-core path: split the operands into bf16 hi/lo planes [T, 3H]
    // (Q | K | V side by side, the layout the fused QKV projection writes).
    const size_t plane = (size_t)T * 3 * H * 2;
    uint8_t *planes = (uint8_t *)sg.scratch(2 * plane);
    if (planes) {
      void *hi = planes, *lo = planes + plane;
      int rc = omcudaDevSplitBf16(dq, T, H, H, hi, lo, 3 * H, 0, st);
      if (rc == OMCUDA_OK)
        rc = omcudaDevSplitBf16(dk, T, H, H, hi, lo, 3 * H, H, st);
      if (rc == OMCUDA_OK)
        rc = omcudaDevSplitBf16(dv, T, H, H, hi, lo, 3 * H, 2 * H, st);
      if (rc == OMCUDA_OK)
        rc = omcudaDevAttentionBf16(hi, lo, 3 * H, 0, H, 2 * H, B, S, heads, dh,
            (float)scale, dy, H, nullptr, st);
      sg.set(rc);
    }
  } else {
    sg.set(omcudaDevAttention(dq, dk, dv, B, S, heads, dh, (float)scale, dy, st));
  }
  sg.finish(true);
}

} // extern "C"
