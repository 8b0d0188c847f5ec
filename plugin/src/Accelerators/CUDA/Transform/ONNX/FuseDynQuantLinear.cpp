/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===---------------------- FuseDynQuantLinear.cpp ------------------------===//
//
// ONNX -> ONNX rewrite for the CUDA accelerator.  The dynamic-quantized linear
// layer that quantization tools emit,
//
//   %xq, %xs, %xz = onnx.DynamicQuantizeLinear(%X)
//   %acc = onnx.MatMulInteger(%xq, %W, %xz, %wz)
//   %f   = onnx.Cast(%acc) {to = f32}
//   %y   = onnx.Mul(%f, onnx.Mul(%xs, %ws))      // scaleForm 0
//     or   onnx.Mul(onnx.Mul(%f, %xs), %ws)      // scaleForm 1
//   %out = onnx.Add(%y, %bias)                    // optional
//
// becomes one op,
//
//   %out = "onnx.Custom"(%X, %W, %ws, %wz, %bias)
//              {function_name = "omcudaDynQuantLinear", scaleForm = 0 : si64, ...}
//
// which the stock ONNXCustomOpLowering turns into
//   krnl.call @omcudaDynQuantLinear(Y, X, Wq, wScale, wZp, bias, scaleForm)
// (src/Conversion/ONNXToKrnl/Additional/Custom.cpp:27-78).  The two spellings
// of the scale are not bit-identical (one rounds the product of the two
// scalars first, the other rounds twice on the tensor), so the rewrite records
// which one the graph used and the library follows it.
//
// The in-tree model for matching this subgraph is the NNPA accelerator's
// replaceMatMulIntegerSubGraphFromMulPattern
// (src/Accelerators/NNPA/Conversion/ONNXToZHigh/ONNXToZHigh.cpp:913-1215).
// This pass anchors on the last op of the chain instead (Add when there is a
// bias, else the outer Mul) and walks up, which keeps each spelling one short
// function.
//
//===----------------------------------------------------------------------===//

#include "mlir/Dialect/Func/IR/FuncOps.h"
#include "mlir/Pass/Pass.h"
#include "mlir/Transforms/GreedyPatternRewriteDriver.h"

#include "src/Accelerators/CUDA/Pass/CUDAPasses.hpp"
#include "src/Dialect/ONNX/DialectBuilder.hpp"
#include "src/Dialect/ONNX/ONNXOps.hpp"
#include "src/Dialect/ONNX/ONNXOps/OpHelper.hpp"

using namespace mlir;

namespace onnx_mlir {

namespace {

struct LinearChain {
  Value X;           // f32 input of DynamicQuantizeLinear
  Value W, WScale;   // 8-bit weight [K,N], its f32 scale (scalar or [N])
  Value WZeroPoint;  // 8-bit zero point or none
  int64_t scaleForm; // 0: f * (xs * ws), 1: (f * xs) * ws
};

bool isScalarF32(Value v) {
  auto ty = dyn_cast<RankedTensorType>(v.getType());
  return ty && ty.getElementType().isF32() && ty.hasStaticShape() &&
         ty.getNumElements() == 1;
}

/// cast -> MatMulInteger -> DynamicQuantizeLinear, with the uses the rewrite
/// needs: A and a_zero_point must be results 0 and 2 of one
/// DynamicQuantizeLinear, B a rank-2 8-bit tensor.
bool matchIntegerMatMul(Value f32Value, ONNXDynamicQuantizeLinearOp &dql,
    ONNXMatMulIntegerOp &mmi) {
  auto cast = f32Value.getDefiningOp<ONNXCastOp>();
  if (!cast || !getElementType(cast.getType()).isF32() || !cast->hasOneUse())
    return false;
  mmi = cast.getInput().getDefiningOp<ONNXMatMulIntegerOp>();
  if (!mmi || !mmi->hasOneUse())
    return false;
  dql = mmi.getA().getDefiningOp<ONNXDynamicQuantizeLinearOp>();
  if (!dql || mmi.getA() != dql.getResult(0) || mmi.getAZeroPoint() != dql.getResult(2))
    return false;
  auto bTy = dyn_cast<RankedTensorType>(mmi.getB().getType());
  return bTy && bTy.getRank() == 2 && bTy.getElementType().isInteger(8);
}

/// Matches the scaled product ending in `mul` in either spelling.
bool matchScaledProduct(ONNXMulOp mul, LinearChain &chain,
    ONNXDynamicQuantizeLinearOp &dql, ONNXMatMulIntegerOp &mmi) {
  for (unsigned side = 0; side < 2; ++side) {
    Value tensorSide = mul->getOperand(side), other = mul->getOperand(1 - side);
    // scaleForm 0: cast * Mul(x_scale, w_scale), the two scalars multiplied first
    if (matchIntegerMatMul(tensorSide, dql, mmi)) {
      auto scales = other.getDefiningOp<ONNXMulOp>();
      if (!scales)
        continue;
      for (unsigned s = 0; s < 2; ++s)
        if (scales->getOperand(s) == dql.getResult(1) && isScalarF32(scales->getOperand(1 - s))) {
          chain.scaleForm = 0;
          chain.WScale = scales->getOperand(1 - s);
          return true;
        }
      continue;
    }
    // scaleForm 1: Mul(cast, x_scale) * w_scale, two roundings on the tensor
    auto inner = tensorSide.getDefiningOp<ONNXMulOp>();
    if (!inner || !inner->hasOneUse())
      continue;
    for (unsigned s = 0; s < 2; ++s)
      if (matchIntegerMatMul(inner->getOperand(s), dql, mmi) &&
          inner->getOperand(1 - s) == dql.getResult(1)) {
        auto wsTy = dyn_cast<RankedTensorType>(other.getType());
        if (!wsTy || !wsTy.getElementType().isF32())
          continue;
        chain.scaleForm = 1;
        chain.WScale = other;
        return true;
      }
  }
  return false;
}

Value buildCustom(PatternRewriter &rewriter, Location loc, Type resultType,
    const LinearChain &chain, Value bias) {
  MultiDialectBuilder<OnnxBuilder> create(rewriter, loc);
  Value none = create.onnx.none();
  SmallVector<Value, 5> inputs = {chain.X, chain.W, chain.WScale,
      chain.WZeroPoint ? chain.WZeroPoint : none, bias ? bias : none};
  auto custom = ONNXCustomOp::create(rewriter, loc, TypeRange{resultType}, inputs);
  custom->setAttr("function_name", rewriter.getStringAttr("omcudaDynQuantLinear"));
  custom->setAttr("scaleForm",
      rewriter.getIntegerAttr(rewriter.getIntegerType(64, /*isSigned=*/true),
          chain.scaleForm));
  // Shape inference: the result has the shape of MatMul(X, W).
  custom->setAttr("shape_infer_pattern", rewriter.getStringAttr("MDBroadcast"));
  custom->setAttr("output_element_type", TypeAttr::get(rewriter.getF32Type()));
  return custom.getResult(0);
}

bool fillChain(ONNXMulOp mul, LinearChain &chain) {
  ONNXDynamicQuantizeLinearOp dql;
  ONNXMatMulIntegerOp mmi;
  if (!matchScaledProduct(mul, chain, dql, mmi))
    return false;
  chain.X = dql.getX();
  chain.W = mmi.getB();
  chain.WZeroPoint = isNoneValue(mmi.getBZeroPoint()) ? Value() : mmi.getBZeroPoint();
  return true;
}

/// ... -> Add(%y, %bias) with %bias an f32 vector over the last dimension.
struct FuseWithBias : public OpRewritePattern<ONNXAddOp> {
  using OpRewritePattern<ONNXAddOp>::OpRewritePattern;
  LogicalResult matchAndRewrite(ONNXAddOp add, PatternRewriter &rewriter) const final {
    for (unsigned side = 0; side < 2; ++side) {
      auto mul = add->getOperand(side).getDefiningOp<ONNXMulOp>();
      Value bias = add->getOperand(1 - side);
      auto biasTy = dyn_cast<RankedTensorType>(bias.getType());
      if (!mul || !mul->hasOneUse() || !biasTy || biasTy.getRank() != 1 ||
          !biasTy.getElementType().isF32())
        continue;
      LinearChain chain;
      if (!fillChain(mul, chain))
        continue;
      rewriter.replaceOp(add, buildCustom(rewriter, add.getLoc(), add.getType(), chain, bias));
      return success();
    }
    return failure();
  }
};

/// The chain without a bias: anchored on the outer Mul, unless an Add that
/// FuseWithBias will take is its only user.
struct FuseWithoutBias : public OpRewritePattern<ONNXMulOp> {
  using OpRewritePattern<ONNXMulOp>::OpRewritePattern;
  LogicalResult matchAndRewrite(ONNXMulOp mul, PatternRewriter &rewriter) const final {
    LinearChain chain;
    if (!fillChain(mul, chain))
      return failure();
    if (mul->hasOneUse())
      if (auto add = dyn_cast<ONNXAddOp>(*mul->user_begin())) {
        Value other = add.getA() == mul.getResult() ? add.getB() : add.getA();
        auto ty = dyn_cast<RankedTensorType>(other.getType());
        if (ty && ty.getRank() == 1 && ty.getElementType().isF32())
          return failure(); // leave it to FuseWithBias
      }
    rewriter.replaceOp(mul, buildCustom(rewriter, mul.getLoc(), mul.getType(), chain, Value()));
    return success();
  }
};

struct FuseDynQuantLinearForCUDAPass
    : public PassWrapper<FuseDynQuantLinearForCUDAPass, OperationPass<func::FuncOp>> {
  MLIR_DEFINE_EXPLICIT_INTERNAL_INLINE_TYPE_ID(FuseDynQuantLinearForCUDAPass)
  StringRef getArgument() const override { return "fuse-dyn-quant-linear-for-cuda"; }
  StringRef getDescription() const override {
    return "Fuse DynamicQuantizeLinear -> MatMulInteger -> Cast -> Mul [-> Mul] [-> Add] "
           "into one onnx.Custom call into libomcuda.";
  }
  void runOnOperation() final {
    RewritePatternSet patterns(&getContext());
    // Bias first: the longer chain wins.
    patterns.insert<FuseWithBias>(&getContext(), /*benefit=*/2);
    patterns.insert<FuseWithoutBias>(&getContext(), /*benefit=*/1);
    if (failed(applyPatternsGreedily(getOperation(), std::move(patterns))))
      signalPassFailure();
  }
};

} // namespace

std::unique_ptr<Pass> createFuseDynQuantLinearForCUDAPass() {
  return std::make_unique<FuseDynQuantLinearForCUDAPass>();
}

} // namespace onnx_mlir
