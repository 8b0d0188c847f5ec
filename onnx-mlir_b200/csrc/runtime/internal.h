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
void *pool_alloc(size_t bytes);
void pool_free(void *p);
bool pool_owns(const void *p);

// dql.cu
int launch_quantize_with_params(const float *x, int64_t n, uint8_t *y,
    const float *params, cudaStream_t st);
int launch_params_from_range(uint32_t *range, float *params, float *y_scale,
    uint8_t *y_zp, cudaStream_t st);

// gemm_tc.cu / gemm_simt.cu
bool gemm_tc_supported(const omcudaGemmArgs &a);
int launch_gemm_tc(const omcudaGemmArgs &a, cudaStream_t st);
int launch_gemm_simt(const omcudaGemmArgs &a, cudaStream_t st);

} // namespace omcuda
