/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===--------------------- RejectUnsupportedOps.cpp -----------------------===//
//
// libomcuda has no CPU fallback, and intermediates may only live in device
// memory when every op that touches them is a libomcuda call.  With
// --cuda-require-full-offload this pass refuses, at compile time, a module
// that would keep an ONNX op on the CPU: one error per op with the reason
// hasOMCUDALowering gives, then the pass fails.
//
//===----------------------------------------------------------------------===//

#include "mlir/IR/BuiltinOps.h"
#include "mlir/Pass/Pass.h"

#include "src/Accelerators/CUDA/Conversion/ONNXToKrnl/ONNXToOMCUDACalls.hpp"
#include "src/Accelerators/CUDA/Pass/CUDAPasses.hpp"
#include "src/Dialect/ONNX/ONNXDialect.hpp"

using namespace mlir;

namespace onnx_mlir {

namespace {

struct RejectOpsWithoutCUDALoweringPass
    : public PassWrapper<RejectOpsWithoutCUDALoweringPass, OperationPass<ModuleOp>> {
  MLIR_DEFINE_EXPLICIT_INTERNAL_INLINE_TYPE_ID(RejectOpsWithoutCUDALoweringPass)
  StringRef getArgument() const override { return "reject-ops-without-cuda-lowering"; }
  StringRef getDescription() const override {
    return "Fail when an ONNX op of the module has no libomcuda lowering.";
  }
  void runOnOperation() final {
    bool bad = false;
    getOperation().walk([&](Operation *op) {
      if (!isa<ONNXDialect>(op->getDialect()))
        return;
      std::string why;
      if (!hasOMCUDALowering(op, &why)) {
        op->emitError("CUDA accelerator: op stays on the CPU (") << why
            << "); libomcuda has no CPU fallback, compile without "
               "--cuda-require-full-offload to stage this graph through host memory";
        bad = true;
      }
    });
    if (bad)
      signalPassFailure();
  }
};

} // namespace

std::unique_ptr<Pass> createRejectOpsWithoutCUDALoweringPass() {
  return std::make_unique<RejectOpsWithoutCUDALoweringPass>();
}

} // namespace onnx_mlir
