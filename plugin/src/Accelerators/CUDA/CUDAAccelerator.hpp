/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===-------------------------- CUDAAccelerator.hpp -----------------------===//
//
// Accelerator support for NVIDIA B200 (sm_100a) through libomcuda: the
// quantized-linear ops (DynamicQuantizeLinear, QuantizeLinear, MatMulInteger,
// QLinearMatMul, DequantizeLinear and the dequantization tail) and the fp32
// ops a quantized encoder holds between them are lowered to krnl.call into the
// library instead of Krnl loops.
//
// Implements every pure virtual of onnx_mlir::accel::Accelerator
// (src/Accelerators/Accelerator.hpp:61-176).
//
//===----------------------------------------------------------------------===//

#ifndef ONNX_MLIR_CUDA_ACCELERATOR_H
#define ONNX_MLIR_CUDA_ACCELERATOR_H

#include "mlir/IR/BuiltinTypes.h"
#include "src/Accelerators/Accelerator.hpp"

namespace onnx_mlir {
namespace accel {

/// Singleton, like every accelerator: the framework asks createCUDA() for it.
class CUDAAccelerator final : public Accelerator {
private:
  static CUDAAccelerator *instance;
  CUDAAccelerator();

public:
  CUDAAccelerator(CUDAAccelerator &) = delete;
  void operator=(const CUDAAccelerator &) = delete;
  ~CUDAAccelerator();

  static CUDAAccelerator *getInstance();

  static bool classof(const Accelerator *accel) {
    return accel->getKind() == Accelerator::Kind::CUDA;
  }
  static bool classof(const CUDAAccelerator *) { return true; }

  /// OMCUDA_VERSION of the libomcuda the compiler was built against; the
  /// generated entry point passes it to OMInitCompatibleAccelCUDA.
  uint64_t getVersionNumber() const final;
  std::string getAccelCompileInfo() const final;

  // onnx-mlir driver
  void addPasses(mlir::OwningOpRef<mlir::ModuleOp> &module,
      mlir::PassManager &pm, onnx_mlir::EmissionTargetType &emissionTarget,
      std::string outputNameNoExt) const final;
  // onnx-mlir-opt driver
  void registerDialects(mlir::DialectRegistry &registry) const final;
  void registerPasses(int optLevel) const final;
  // both
  void configurePasses() const final;
  // onnx-to-krnl
  mlir::MemRefType convertTensorTypeToMemRefType(
      const mlir::TensorType tensorType) const final;
  int64_t getDefaultAllocAlignment(const mlir::TensorType tensorType) const final;
  void conversionTargetONNXToKrnl(mlir::ConversionTarget &target) const final;
  void rewritePatternONNXToKrnl(mlir::RewritePatternSet &patterns,
      mlir::TypeConverter &typeConverter, mlir::MLIRContext *ctx) const final;
  // krnl-to-llvm
  void conversionTargetKrnlToLLVM(mlir::ConversionTarget &target) const final;
  void rewritePatternKrnlToLLVM(mlir::RewritePatternSet &patterns,
      mlir::LLVMTypeConverter &typeConverter,
      mlir::MLIRContext *ctx) const final;
};

} // namespace accel
} // namespace onnx_mlir
#endif
