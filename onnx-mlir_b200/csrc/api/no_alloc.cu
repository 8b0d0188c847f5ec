// DynamicQuantizeLinear for callers that may not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: an inference
// server that handed every byte of HBM to its own arena at start-up and
// forbids plug-ins to touch the CUDA allocator, a latency-critical loop that
// cannot afford the device-wide synchronisation cudaMalloc/cudaFree imply, or
// a process whose allocation calls are intercepted and refused by a
// sandboxing layer.  The ordinary entry point
// omcudaDevDynamicQuantizeLinear makes such a caller bring its own scratch
// buffer; this variant needs none: its scratch (the per-block partial min/max
// table, the ticket counter and the two derived scalars of the single-pass
// grid reduction) lives in a fixed array that is part of the library image.
// Every GPU that loads the library therefore holds kScratchBytes (32 KiB) of
// device memory for it until the process exits.
//
// The function calls no cudaMalloc, cudaFree or allocating library routine.
// (Its first call on a device looks the array's address up with
// cudaGetSymbolAddress, which may make the CUDA runtime load the library's
// device code on that device; make that first call at start-up, before any
// stream capture.)  It has no counterpart in onnx-mlir.
#include <cuda_runtime.h>

#include <mutex>

#include "../common.cuh"

namespace {

constexpr size_t kScratchBytes = 32 * 1024;
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a handle for
// cudaGetSymbolAddress; it is not a device address and must never be handed
// to a kernel as one.
static __device__ __align__(256) unsigned char g_dql_scratch[kScratchBytes];

std::mutex g_setup_mutex;
void *g_scratch_addr[kMaxDevices] = {nullptr};

// Resolves the device address of g_dql_scratch for the current device, once
// per device.  The lookup runs with that device current, as the runtime
// requires for a per-device symbol.
int scratch_for_current_device(void **out) {
  int dev = -1;
  int rc = omcuda::check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (rc != OMCUDA_OK)
    return rc;
  if (dev < 0 || dev >= kMaxDevices)
    return omcuda::fail(OMCUDA_ENOTSUP,
        "DynamicQuantizeLinearNoAlloc: device index %d is beyond the %d this "
        "entry point keeps addresses for", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    void *ptr = nullptr;
    rc = omcuda::check_cuda(cudaGetSymbolAddress((void **)&ptr, g_dql_scratch),
        "cudaGetSymbolAddress(g_dql_scratch)");
    if (rc != OMCUDA_OK)
      return rc;
    if (!ptr)
      return omcuda::fail(OMCUDA_ECUDA,
          "DynamicQuantizeLinearNoAlloc: the scratch symbol has no address");
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return OMCUDA_OK;
}

} // namespace

extern "C" int omcudaDevDynamicQuantizeLinearNoAlloc(const float *x, int64_t n,
    uint8_t *y, float *y_scale, uint8_t *y_zp, void *stream) {
  if (n < 0 || (n > 0 && (!x || !y)))
    return omcuda::fail(OMCUDA_EINVAL,
        "DynamicQuantizeLinearNoAlloc: bad argument");
  if (n > OMCUDA_DQL_NOALLOC_MAX_ELEMS)
    return omcuda::fail(OMCUDA_EINVAL,
        "DynamicQuantizeLinearNoAlloc: %lld elements exceed the limit of %lld "
        "this allocation-free entry point accepts; use "
        "omcudaDevDynamicQuantizeLinear with caller-provided scratch",
        (long long)n, (long long)OMCUDA_DQL_NOALLOC_MAX_ELEMS);
  if ((size_t)omcudaDevDqlScratchBytes(n) > kScratchBytes)
    return omcuda::fail(OMCUDA_EINVAL,
        "DynamicQuantizeLinearNoAlloc: the reduction needs %lld bytes of "
        "scratch, the built-in array holds %lld",
        (long long)omcudaDevDqlScratchBytes(n), (long long)kScratchBytes);
  void *scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != OMCUDA_OK)
    return rc;
  // The array still holds whatever the previous call left.  The reduction only
  // requires its ticket counter (first 64-byte line) to start at zero.
  rc = omcuda::check_cuda(
      cudaMemsetAsync(scratch, 0, 64, (cudaStream_t)stream), "cudaMemsetAsync");
  if (rc != OMCUDA_OK)
    return rc;
  return omcudaDevDynamicQuantizeLinear(x, n, y, y_scale, y_zp, scratch, stream);
}
