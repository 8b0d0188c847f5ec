/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===------------------- ReplaceMallocByDeviceAlloc.cpp -------------------===//
//
// Device-resident intermediates.  After Krnl-to-LLVM every memref.alloc of the
// model is `llvm.call @malloc(size)` and every dealloc `llvm.call @free(ptr)`.
// In a module whose ops are all libomcuda calls these buffers are only ever
// handed to the library, so they can live in device memory:
//
//   %p = llvm.call @malloc(%size) : (i64) -> !llvm.ptr
//   llvm.call @free(%p) : (!llvm.ptr) -> ()
// becomes
//   %p = llvm.call @omcudaDeviceAlloc(%size) : (i64) -> !llvm.ptr
//   llvm.call @omcudaDeviceFree(%p) : (!llvm.ptr) -> ()
//
// libomcuda tells host from device pointers itself, so no call site changes;
// omcudaDeviceFree ignores pointers that are not its own, which keeps the
// `free` of an input the caller allocated on the host harmless.  Same
// technique as the NNPA accelerator's huge-page allocator swap
// (src/Accelerators/NNPA/Transform/ReplaceMallocByHugePageMalloc.cpp:34-73).
// Buffers that the entry point returns to the caller keep `malloc`: the
// OMTensor runtime frees them with free() (src/Runtime/OMTensor.inc:259-272).
//
//===----------------------------------------------------------------------===//

#include "mlir/Dialect/LLVMIR/LLVMDialect.h"
#include "mlir/Pass/Pass.h"
#include "mlir/Transforms/GreedyPatternRewriteDriver.h"

#include "src/Accelerators/CUDA/Pass/CUDAPasses.hpp"
#include "src/Dialect/Mlir/DialectBuilder.hpp"

using namespace mlir;

namespace onnx_mlir {

namespace {

/// True when the allocation reaches omTensorSetDataPtr, i.e. is wrapped as an
/// output OMTensor of run_main_graph (KrnlEntryPoint.cpp:318-325).
bool escapesToCaller(Value ptr) {
  SmallVector<Value, 8> work = {ptr};
  llvm::SmallPtrSet<Operation *, 16> seen;
  while (!work.empty()) {
    Value v = work.pop_back_val();
    for (Operation *user : v.getUsers()) {
      if (!seen.insert(user).second)
        continue;
      if (auto call = dyn_cast<LLVM::CallOp>(user)) {
        auto callee = call.getCalleeAttr();
        if (callee && callee.getValue() == "omTensorSetDataPtr")
          return true;
        continue;
      }
      if (isa<LLVM::ReturnOp>(user))
        return true;
      for (Value r : user->getResults()) // insertvalue, getelementptr, bitcast ...
        work.push_back(r);
    }
  }
  return false;
}

struct MallocToDeviceAlloc : public OpRewritePattern<LLVM::CallOp> {
  using OpRewritePattern<LLVM::CallOp>::OpRewritePattern;
  LogicalResult matchAndRewrite(LLVM::CallOp call, PatternRewriter &rewriter) const final {
    FlatSymbolRefAttr callee = call.getCalleeAttr();
    if (!callee)
      return failure();
    LLVMBuilder createLLVM(rewriter, call.getLoc());
    SmallVector<Value, 1> operands(call.getOperands().begin(), call.getOperands().end());
    if (callee.getValue() == "malloc" && call.getNumOperands() == 1 &&
        call.getNumResults() == 1 && isa<LLVM::LLVMPointerType>(call.getResult().getType())) {
      if (escapesToCaller(call.getResult()))
        return failure();
      Value p = createLLVM.call({call.getResult().getType()}, "omcudaDeviceAlloc", operands);
      rewriter.replaceOp(call, p);
      return success();
    }
    if (callee.getValue() == "free" && call.getNumOperands() == 1 &&
        call.getNumResults() == 0) {
      createLLVM.call({}, "omcudaDeviceFree", operands);
      rewriter.eraseOp(call);
      return success();
    }
    return failure();
  }
};

struct ReplaceMallocByDeviceAllocPass
    : public PassWrapper<ReplaceMallocByDeviceAllocPass, OperationPass<ModuleOp>> {
  MLIR_DEFINE_EXPLICIT_INTERNAL_INLINE_TYPE_ID(ReplaceMallocByDeviceAllocPass)
  StringRef getArgument() const override { return "replace-malloc-by-omcuda-device-alloc"; }
  StringRef getDescription() const override {
    return "Allocate the model's intermediates with omcudaDeviceAlloc / omcudaDeviceFree.";
  }
  void runOnOperation() final {
    RewritePatternSet patterns(&getContext());
    patterns.insert<MallocToDeviceAlloc>(&getContext());
    if (failed(applyPatternsGreedily(getOperation(), std::move(patterns))))
      signalPassFailure();
  }
};

} // namespace

std::unique_ptr<Pass> createReplaceMallocByDeviceAllocPass() {
  return std::make_unique<ReplaceMallocByDeviceAllocPass>();
}

} // namespace onnx_mlir
