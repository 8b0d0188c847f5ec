/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===------------------------- CUDACompilerUtils.cpp ----------------------===//
//
// Pipeline of --maccel=CUDA.  The stock pipeline is kept (ONNX passes ->
// convert-onnx-to-krnl -> krnl-to-llvm, src/Compiler/CompilerPasses.cpp:575-621);
// the accelerator adds, before the lowering, the subgraph fusion and the
// full-offload check, and after it the device-allocation rewrite.
//
//===----------------------------------------------------------------------===//

#include "mlir/Pass/PassManager.h"
#include "mlir/Transforms/Passes.h"

#include "src/Accelerators/CUDA/Compiler/CUDACompilerOptions.hpp"
#include "src/Accelerators/CUDA/Compiler/CUDACompilerUtils.hpp"
#include "src/Accelerators/CUDA/Pass/CUDAPasses.hpp"
#include "src/Compiler/CompilerOptions.hpp"
#include "src/Compiler/CompilerPasses.hpp"
#include "src/Pass/Passes.hpp"

namespace onnx_mlir {

void configurePassesCUDA() {
  // The fusion pattern needs DynamicQuantizeLinear, MatMulInteger and the
  // Cast/Mul/Add tail as they come from the model: nothing to switch off in
  // the shared passes.
}

void addPassesCUDA(mlir::OwningOpRef<mlir::ModuleOp> &module,
    mlir::PassManager &pm, onnx_mlir::EmissionTargetType &emissionTarget,
    std::string outputNameNoExt) {
  configurePassesCUDA();

  // ONNX-level passes of the stock pipeline (shape inference, constant
  // propagation, Recompose: LayerNormalization, Gelu and QLinearMatMul are
  // rebuilt from their primitive patterns there,
  // src/Dialect/ONNX/Transforms/Recompose.cpp:92-146,388-416,592-648).
  InputIRLevelType inputIRLevel = determineInputIRLevel(module);
  if (inputIRLevel <= ONNXLevel && emissionTarget >= EmitONNXIR)
    addONNXToMLIRPasses(pm, /*target CPU*/ false);

  if (emissionTarget >= EmitMLIR) {
    // ONNX -> ONNX: one call per dynamic-quantized linear.
    if (!cudaDisableDynQuantLinearFusion) {
      pm.addNestedPass<mlir::func::FuncOp>(createFuseDynQuantLinearForCUDAPass());
      pm.addPass(mlir::createCanonicalizerPass());
    }
    // No CPU fallback inside libomcuda: with --cuda-require-full-offload a
    // graph that keeps an op on the CPU is refused here, at compile time.
    if (cudaRequireFullOffload)
      pm.addPass(createRejectOpsWithoutCUDALoweringPass());

    // ONNX -> Krnl.  The accelerator's patterns are picked up through
    // Accelerator::rewritePatternONNXToKrnl; onnx.Custom is lowered to
    // krnl.call by the stock ONNXCustomOpLowering
    // (src/Conversion/ONNXToKrnl/Additional/Custom.cpp:27-78).
    if (inputIRLevel <= MLIRLevel)
      addONNXToKrnlPasses(pm, OptimizationLevel, /*enableCSE*/ true,
          instrumentSignatures, ONNXOpStats);
  }

  if (emissionTarget >= EmitLLVMIR) {
    if (inputIRLevel <= LLVMLevel)
      addKrnlToLLVMPasses(pm, outputNameNoExt, /*enableCSE=*/true);
    // Device-resident intermediates: only legal when the whole graph is
    // libomcuda calls, which the check above has established.
    if (cudaDeviceResidentIntermediates && cudaRequireFullOffload)
      pm.addPass(createReplaceMallocByDeviceAllocPass());
  }
}

} // namespace onnx_mlir
