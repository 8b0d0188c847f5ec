/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===------------------------- CUDACompilerUtils.hpp ----------------------===//

#ifndef ONNX_MLIR_CUDA_COMPILER_UTILS_H
#define ONNX_MLIR_CUDA_COMPILER_UTILS_H

#include "mlir/IR/BuiltinOps.h"
#include "mlir/IR/OwningOpRef.h"
#include "mlir/Pass/PassManager.h"

#include "include/onnx-mlir/Compiler/OMCompilerTypes.h"

namespace onnx_mlir {

/// The CUDA accelerator's pass pipeline (model: addPassesNNPA,
/// src/Accelerators/NNPA/Compiler/NNPACompilerUtils.cpp).
void addPassesCUDA(mlir::OwningOpRef<mlir::ModuleOp> &module,
    mlir::PassManager &pm, onnx_mlir::EmissionTargetType &emissionTarget,
    std::string outputNameNoExt);

void configurePassesCUDA();

} // namespace onnx_mlir
#endif
