/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===---------- CUDAPasses.hpp - CUDA accelerator passes ------------------===//

#ifndef ONNX_MLIR_CUDA_PASSES_H
#define ONNX_MLIR_CUDA_PASSES_H

#include "mlir/Pass/Pass.h"

namespace onnx_mlir {

/// ONNX -> ONNX: DynamicQuantizeLinear -> MatMulInteger -> Cast -> Mul
/// [-> Mul] [-> Add] becomes onnx.Custom {function_name = "omcudaDynQuantLinear"}.
std::unique_ptr<mlir::Pass> createFuseDynQuantLinearForCUDAPass();

/// Verifies that every ONNX op left in the module has a libomcuda lowering;
/// emits an error per offending op and fails the pass otherwise.
std::unique_ptr<mlir::Pass> createRejectOpsWithoutCUDALoweringPass();

/// LLVM level: malloc / free of memrefs become omcudaDeviceAlloc /
/// omcudaDeviceFree (device-resident intermediates).
std::unique_ptr<mlir::Pass> createReplaceMallocByDeviceAllocPass();

} // namespace onnx_mlir
#endif
