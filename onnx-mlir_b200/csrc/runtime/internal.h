// Internal host-side interfaces shared by libomcuda's translation units.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "omcuda.h"

namespace omcuda {

int ensure_init();
bool sticky_error();
cudaStream_t current_stream();
// Device-memory pool with stream-ordered reuse.  The plain forms use the
// calling thread's stream (omcudaGetStream); the _on forms name the stream the
// block will be / was last used on.
void *pool_alloc(size_t bytes);
void pool_free(void *p);
void *pool_alloc_on(size_t bytes, cudaStream_t st);
void pool_free_on(void *p, cudaStream_t st);
bool pool_owns(const void *p);

// Index of the device current on the calling thread, or -1.
constexpr int kMaxDevices = 64;
int current_device_index();
// A value a kernel's launcher computes once per device (launch attributes
// set, cluster occupancy); 0 means "not yet".  Safe to use from several host
// threads and with several devices in one process.
struct PerDeviceInt {
  int v[kMaxDevices] = {0};
  int get();
  void set(int x);
};

// OMCUDA_MODE_* flags set with omcudaSetQuantizationMode (process wide).
int quant_mode();

// Wait limit the tensor-core kernels are launched with (gemm_tc.cu).
uint64_t tc_wait_limit_ns();

// dql.cu
int launch_quantize_with_params(const float *x, int64_t n, uint8_t *y,
    const float *params, cudaStream_t st);

// gemm_tc.cu / gemm_simt.cu
bool gemm_tc_supported(const omcudaGemmArgs &a);
int launch_gemm_tc(const omcudaGemmArgs &a, cudaStream_t st);
int launch_gemm_simt(const omcudaGemmArgs &a, cudaStream_t st);

// attention_mma.cu
bool attention_mma_supported(const float *Q, const float *K, const float *V,
    const float *out, int64_t dh, int64_t ld_in, int64_t ld_out);
int launch_attention_mma(const float *Q, const float *K, const float *V,
    int64_t B, int64_t S, int64_t heads, int64_t dh, float scale, float *out,
    int64_t ld_in, int64_t ld_out, void *out_range, cudaStream_t st);

// attention_tc.cu: tcgen05 attention over bf16 hi/lo planes [T, ld_planes]
// (head size 64, sequence a multiple of 128), and the fp32 -> planes split.
bool attention_tc_supported(int64_t B, int64_t S, int64_t heads, int64_t dh,
    int64_t ld_planes, int64_t ld_out, const void *hi, const void *lo,
    const float *out);
int launch_attention_tc(const void *hi, const void *lo, int64_t ld_planes,
    int64_t q_col, int64_t k_col, int64_t v_col, int64_t B, int64_t S,
    int64_t heads, float scale, float *out, int64_t ld_out, void *out_range,
    cudaStream_t st);
int launch_split_bf16(const float *x, int64_t rows, int64_t cols, int64_t ld_x,
    void *hi, void *lo, int64_t ld_p, int64_t col0, cudaStream_t st);

} // namespace omcuda
