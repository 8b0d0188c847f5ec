/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===-------------------------- CUDAAccelerator.cpp -----------------------===//
//
// Structure follows the in-tree NNPA accelerator
// (src/Accelerators/NNPA/NNPAAccelerator.cpp:42-247): a singleton that pushes
// itself on acceleratorTargets and tells the compiler which libraries a
// compiled model has to link.  There is no accelerator dialect: the ONNX ops
// go straight to krnl.call, which the stock Krnl-to-LLVM lowering turns into
// calls with OMTensor arguments
// (src/Conversion/KrnlToLLVM/KrnlCall.cpp:34-226).
//
//===----------------------------------------------------------------------===//

#include "llvm/Support/Debug.h"

#include "omcuda.h" // OMCUDA_VERSION

#include "src/Accelerators/CUDA/CUDAAccelerator.hpp"
#include "src/Accelerators/CUDA/Compiler/CUDACompilerOptions.hpp"
#include "src/Accelerators/CUDA/Compiler/CUDACompilerUtils.hpp"
#include "src/Accelerators/CUDA/Conversion/ONNXToKrnl/ONNXToOMCUDACalls.hpp"
#include "src/Accelerators/CUDA/Pass/CUDAPasses.hpp"
#include "src/Compiler/CompilerOptions.hpp"

#include <memory>

#define DEBUG_TYPE "CUDAAccelerator"

namespace onnx_mlir {
namespace accel {

Accelerator *createCUDA() { return CUDAAccelerator::getInstance(); }

CUDAAccelerator *CUDAAccelerator::instance = nullptr;

CUDAAccelerator *CUDAAccelerator::getInstance() {
  if (instance == nullptr)
    instance = new CUDAAccelerator();
  return instance;
}

CUDAAccelerator::CUDAAccelerator() : Accelerator(Accelerator::Kind::CUDA) {
  LLVM_DEBUG(llvm::dbgs() << "Creating a CUDA (libomcuda) accelerator\n");
  acceleratorTargets.push_back(this);
  // A compiled model links -lomcuda: the library holds the kernels, the
  // OMInit/OMShutdownAccelCUDA hooks the generated entry point calls
  // (src/Conversion/KrnlToLLVM/KrnlEntryPoint.cpp:149-187) and an OMTensor
  // runtime that is layout-compatible with libcruntime's.
  addCompilerConfig(CCM_SHARED_LIB_DEPS, {"omcuda"}, true);
}

CUDAAccelerator::~CUDAAccelerator() { delete instance; }

uint64_t CUDAAccelerator::getVersionNumber() const { return OMCUDA_VERSION; }

std::string CUDAAccelerator::getAccelCompileInfo() const {
  return "{\"target\": \"sm_100a\", \"omcuda_version\": \"" +
         std::to_string((OMCUDA_VERSION >> 16) & 0xFF) + "." +
         std::to_string((OMCUDA_VERSION >> 8) & 0xFF) + "." +
         std::to_string(OMCUDA_VERSION & 0xFF) + "\"}";
}

void CUDAAccelerator::addPasses(mlir::OwningOpRef<mlir::ModuleOp> &module,
    mlir::PassManager &pm, onnx_mlir::EmissionTargetType &emissionTarget,
    std::string outputNameNoExt) const {
  LLVM_DEBUG(llvm::dbgs() << "Adding passes for CUDA accelerator\n");
  addPassesCUDA(module, pm, emissionTarget, outputNameNoExt);
}

void CUDAAccelerator::registerDialects(mlir::DialectRegistry &registry) const {
  // Nothing beyond what onnx-mlir registers: ONNX, Krnl and LLVM dialects.
}

void CUDAAccelerator::registerPasses(int optLevel) const {
  mlir::registerPass([]() -> std::unique_ptr<mlir::Pass> {
    return onnx_mlir::createFuseDynQuantLinearForCUDAPass();
  });
  mlir::registerPass([]() -> std::unique_ptr<mlir::Pass> {
    return onnx_mlir::createRejectOpsWithoutCUDALoweringPass();
  });
  mlir::registerPass([]() -> std::unique_ptr<mlir::Pass> {
    return onnx_mlir::createReplaceMallocByDeviceAllocPass();
  });
}

void CUDAAccelerator::configurePasses() const { configurePassesCUDA(); }

mlir::MemRefType CUDAAccelerator::convertTensorTypeToMemRefType(
    const mlir::TensorType tensorType) const {
  // Plain tensors: whether a buffer is host or device memory is a property of
  // the pointer (libomcuda asks the driver), not of the type.
  return nullptr;
}

int64_t CUDAAccelerator::getDefaultAllocAlignment(
    const mlir::TensorType tensorType) const {
  // TMA wants 16-byte aligned bases, which is the compiler's default
  // (src/Dialect/Mlir/DialectBuilder.hpp:254).
  return -1;
}

void CUDAAccelerator::conversionTargetONNXToKrnl(
    mlir::ConversionTarget &target) const {
  // krnl.call belongs to the Krnl dialect, legal already.
}

void CUDAAccelerator::rewritePatternONNXToKrnl(mlir::RewritePatternSet &patterns,
    mlir::TypeConverter &typeConverter, mlir::MLIRContext *ctx) const {
  // Runs inside convert-onnx-to-krnl next to the CPU patterns
  // (src/Conversion/ONNXToKrnl/ConvertONNXToKrnl.cpp:454-456); the patterns
  // carry a higher benefit so that they win over the loop lowerings.
  onnx_mlir::populateONNXToOMCUDACallsPattern(patterns, typeConverter, ctx);
}

void CUDAAccelerator::conversionTargetKrnlToLLVM(
    mlir::ConversionTarget &target) const {}

void CUDAAccelerator::rewritePatternKrnlToLLVM(mlir::RewritePatternSet &patterns,
    mlir::LLVMTypeConverter &typeConverter, mlir::MLIRContext *ctx) const {
  // krnl.call is lowered by the stock KrnlCallOpLowering.
}

} // namespace accel
} // namespace onnx_mlir
