// Process-wide state of libomcuda: accelerator init/shutdown hooks, sticky
// per-thread status, the library stream and a caching device-memory pool.
//
// The init/shutdown hooks follow the interface the in-tree NNPA accelerator
// documents (src/Accelerators/NNPA/Runtime/OMRuntimeNNPA.c:36-118): a global
// OMIsInitAccel<X> flag readable without a lock, an idempotent thread-safe
// OMInitAccel<X>, a version-gated OMInitCompatibleAccel<X> that reports EPERM
// (:156-232), and OMShutdownAccel<X>.
#include <cuda_runtime.h>

#include <atomic>
#include <cerrno>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "../common.cuh"
#include "internal.h"

extern "C" {
long OMIsInitAccelCUDA = 0;
}

namespace omcuda {

int gemm_tc_check_status(cudaStream_t st);

namespace {

struct ThreadStatus {
  int code = OMCUDA_OK;
  char msg[512] = {0};
  cudaStream_t stream_override = nullptr;
  bool has_override = false;
};
thread_local ThreadStatus t_status;

std::mutex g_init_mutex;
cudaStream_t g_stream = nullptr;
int g_device = -1;
int g_sm_count = 0;
std::atomic<int64_t> g_launches{0};

// Caching pool.  Blocks are reused only for requests of the same rounded
// size.  Reuse is stream-ordered: a freed block remembers the stream it was
// last used on and an event recorded there at the time of the free.  The same
// stream may take it again at once (its earlier work is ahead in the queue);
// another stream gets it only after the event has completed, or is made to
// wait for the event first.
struct FreeBlock {
  void *p;
  cudaStream_t stream;
  cudaEvent_t done; // may be null: nothing was in flight (or no stream known)
};
std::mutex g_pool_mutex;
std::multimap<size_t, FreeBlock> g_free_blocks;
std::unordered_map<void *, size_t> g_live_blocks;
std::vector<cudaEvent_t> g_spare_events;

cudaEvent_t take_event_locked() {
  if (!g_spare_events.empty()) {
    cudaEvent_t e = g_spare_events.back();
    g_spare_events.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return e;
}

size_t round_size(size_t b) {
  if (b < 512)
    return 512;
  if (b < (1u << 20))
    return (b + 511) & ~size_t(511);
  return (b + (size_t(2) << 20) - 1) & ~((size_t(2) << 20) - 1);
}

int errno_for(int code) {
  switch (code) {
  case OMCUDA_EINVAL:
    return EINVAL;
  case OMCUDA_ENOMEM:
    return ENOMEM;
  case OMCUDA_ETIMEDOUT:
    return ETIMEDOUT;
  case OMCUDA_ENOTSUP:
    return ENOTSUP;
  default:
    return EIO;
  }
}

} // namespace

void pool_release_all();

int fail(int code, const char *fmt, ...) {
  if (t_status.code == OMCUDA_OK) {
    t_status.code = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_status.msg, sizeof(t_status.msg), fmt, ap);
    va_end(ap);
    if (getenv("OMCUDA_VERBOSE"))
      fprintf(stderr, "[omcuda] error %d: %s\n", code, t_status.msg);
  }
  errno = errno_for(code);
  return code;
}

int check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess)
    return OMCUDA_OK;
  int code = (e == cudaErrorMemoryAllocation) ? OMCUDA_ENOMEM : OMCUDA_ECUDA;
  return fail(code, "%s: %s", what, cudaGetErrorString(e));
}

int current_device_index() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    return -1;
  }
  return dev;
}

namespace {
std::mutex g_per_device_mutex;
}

int PerDeviceInt::get() {
  const int dev = current_device_index();
  if (dev < 0)
    return 0;
  std::lock_guard<std::mutex> lock(g_per_device_mutex);
  return v[dev];
}

void PerDeviceInt::set(int x) {
  const int dev = current_device_index();
  if (dev < 0)
    return;
  std::lock_guard<std::mutex> lock(g_per_device_mutex);
  v[dev] = x;
}

namespace {
std::atomic<int> g_quant_mode{0};
}
int quant_mode() { return g_quant_mode.load(std::memory_order_relaxed); }

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() { return g_sm_count > 0 ? g_sm_count : 148; }

bool sticky_error() { return t_status.code != OMCUDA_OK; }

// Initialises on first use; returns OMCUDA_OK or records the failure.
int ensure_init() {
  if (OMIsInitAccelCUDA)
    return OMCUDA_OK;
  std::lock_guard<std::mutex> lock(g_init_mutex);
  if (OMIsInitAccelCUDA)
    return OMCUDA_OK;
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess || ndev == 0) {
    (void)cudaGetLastError();
    return fail(OMCUDA_ECUDA, "no CUDA device available (%s)",
        e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  }
  int dev = 0;
  if (const char *s = getenv("OMCUDA_DEVICE"))
    dev = atoi(s);
  else if (const char *r = getenv("LOCAL_RANK"))
    dev = atoi(r) % ndev;
  if (dev < 0 || dev >= ndev)
    return fail(OMCUDA_EINVAL, "device %d out of range (%d devices)", dev, ndev);
  OMCUDA_CHECK(cudaSetDevice(dev));
  cudaDeviceProp prop;
  OMCUDA_CHECK(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10)
    return fail(OMCUDA_ECUDA,
        "device %d is sm_%d%d; this library is built for sm_100a only", dev,
        prop.major, prop.minor);
  g_sm_count = prop.multiProcessorCount;
  OMCUDA_CHECK(cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking));
  g_device = dev;
  std::atomic_thread_fence(std::memory_order_release);
  OMIsInitAccelCUDA = 1;
  return OMCUDA_OK;
}

cudaStream_t current_stream() {
  if (t_status.has_override)
    return t_status.stream_override;
  return g_stream;
}

void *pool_alloc_on(size_t bytes, cudaStream_t st) {
  if (ensure_init() != OMCUDA_OK)
    return nullptr;
  size_t sz = round_size(bytes);
  {
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    auto range = g_free_blocks.equal_range(sz);
    auto pick = range.second;
    // First choice: a block this stream freed itself, or one that is idle.
    for (auto it = range.first; it != range.second; ++it) {
      const FreeBlock &fb = it->second;
      if (!fb.done || fb.stream == st || cudaEventQuery(fb.done) == cudaSuccess) {
        pick = it;
        break;
      }
    }
    (void)cudaGetLastError(); // cudaEventQuery's cudaErrorNotReady is not an error
    bool wait = false;
    if (pick == range.second && range.first != range.second) {
      pick = range.first; // busy on another stream: order this stream behind it
      wait = true;
    }
    if (pick != range.second) {
      FreeBlock fb = pick->second;
      g_free_blocks.erase(pick);
      if (wait && cudaStreamWaitEvent(st, fb.done, 0) != cudaSuccess) {
        (void)cudaGetLastError();
        cudaEventSynchronize(fb.done);
      }
      if (fb.done)
        g_spare_events.push_back(fb.done);
      g_live_blocks[fb.p] = sz;
      return fb.p;
    }
  }
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, sz);
  if (e != cudaSuccess) {
    // Give cached blocks back to the driver and try once more.
    (void)cudaGetLastError();
    pool_release_all();
    e = cudaMalloc(&p, sz);
    if (e != cudaSuccess) {
      check_cuda(e, "cudaMalloc");
      return nullptr;
    }
  }
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  g_live_blocks[p] = sz;
  return p;
}

void *pool_alloc(size_t bytes) { return pool_alloc_on(bytes, current_stream()); }

void pool_free_on(void *p, cudaStream_t st) {
  if (!p)
    return;
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  auto it = g_live_blocks.find(p);
  if (it == g_live_blocks.end())
    return; // not ours
  FreeBlock fb{p, st, take_event_locked()};
  if (fb.done && cudaEventRecord(fb.done, st) != cudaSuccess) {
    (void)cudaGetLastError();
    g_spare_events.push_back(fb.done);
    fb.done = nullptr;
  }
  if (!fb.done) {
    // No event to order a later user behind: make the block idle now.
    cudaStreamSynchronize(st);
  }
  g_free_blocks.emplace(it->second, fb);
  g_live_blocks.erase(it);
}

void pool_free(void *p) { pool_free_on(p, current_stream()); }

bool pool_owns(const void *p) {
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  return g_live_blocks.count(const_cast<void *>(p)) != 0;
}

void pool_release_all() {
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  for (auto &kv : g_free_blocks) {
    if (kv.second.done) {
      cudaEventSynchronize(kv.second.done);
      cudaEventDestroy(kv.second.done);
    }
    cudaFree(kv.second.p);
  }
  g_free_blocks.clear();
  for (cudaEvent_t e : g_spare_events)
    cudaEventDestroy(e);
  g_spare_events.clear();
}

} // namespace omcuda

using namespace omcuda;

extern "C" {

int omcudaGetLastError(void) { return t_status.code; }

const char *omcudaGetLastErrorString(void) {
  return t_status.code == OMCUDA_OK ? "" : t_status.msg;
}

void omcudaClearError(void) {
  t_status.code = OMCUDA_OK;
  t_status.msg[0] = 0;
}

void OMInitAccelCUDA(void) { (void)ensure_init(); }

uint64_t OMInitCompatibleAccelCUDA(uint64_t versionNum) {
  // A model built for a newer major.minor than this library cannot be served.
  if ((versionNum >> 8) > (uint64_t(OMCUDA_VERSION) >> 8)) {
    errno = EPERM;
    return 0;
  }
  if (ensure_init() != OMCUDA_OK) {
    errno = EPERM;
    return 0;
  }
  return 1;
}

void OMShutdownAccelCUDA(void) {
  std::lock_guard<std::mutex> lock(g_init_mutex);
  if (!OMIsInitAccelCUDA)
    return;
  cudaStreamSynchronize(g_stream);
  omcudaForgetConstants();
  pool_release_all();
  cudaStreamDestroy(g_stream);
  g_stream = nullptr;
  OMIsInitAccelCUDA = 0;
}

void *omcudaGetStream(void) {
  if (ensure_init() != OMCUDA_OK)
    return nullptr;
  return (void *)current_stream();
}

void omcudaSetStream(void *stream) {
  if (stream) {
    t_status.stream_override = (cudaStream_t)stream;
    t_status.has_override = true;
  } else {
    t_status.has_override = false;
  }
}

void *omcudaStreamCreate(void) {
  if (ensure_init() != OMCUDA_OK)
    return nullptr;
  cudaStream_t st = nullptr;
  if (check_cuda(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking),
          "cudaStreamCreate") != OMCUDA_OK)
    return nullptr;
  return (void *)st;
}

void omcudaStreamDestroy(void *stream) {
  if (!stream)
    return;
  if (t_status.has_override && t_status.stream_override == (cudaStream_t)stream)
    t_status.has_override = false;
  cudaStreamSynchronize((cudaStream_t)stream);
  cudaStreamDestroy((cudaStream_t)stream);
}

void omcudaSynchronize(void) {
  if (!OMIsInitAccelCUDA)
    return;
  // Also surfaces a bounded-wait timeout raised by a GEMM kernel.
  gemm_tc_check_status(current_stream());
  check_cuda(cudaStreamSynchronize(current_stream()), "cudaStreamSynchronize");
}

void *omcudaDeviceAlloc(int64_t bytes) {
  if (bytes < 0) {
    fail(OMCUDA_EINVAL, "omcudaDeviceAlloc: negative size");
    return nullptr;
  }
  return pool_alloc((size_t)bytes);
}

void omcudaDeviceFree(void *p) { pool_free(p); }

void *omcudaHostAlloc(int64_t bytes) {
  if (ensure_init() != OMCUDA_OK)
    return nullptr;
  void *p = nullptr;
  if (check_cuda(cudaMallocHost(&p, (size_t)(bytes > 0 ? bytes : 1)),
          "cudaMallocHost") != OMCUDA_OK)
    return nullptr;
  return p;
}

void omcudaHostFree(void *p) {
  if (p)
    cudaFreeHost(p);
}

int64_t omcudaLaunchCount(void) { return g_launches.load(); }

void omcudaSetQuantizationMode(int64_t flags) {
  g_quant_mode.store((int)(flags & (OMCUDA_MODE_NO_ZERO_POINT | OMCUDA_MODE_FAST_MATH)),
      std::memory_order_relaxed);
}

int64_t omcudaGetQuantizationMode(void) { return quant_mode(); }

} // extern "C"
