/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===--------------------- ONNXToOMCUDACalls.cpp --------------------------===//
//
// ONNX op -> krnl.call @omcuda<Op>.  One generic pattern, instantiated from
// the table in OMCUDACalls.inc, does what ONNXGenericOpToCall does for the CPU
// (src/Conversion/ONNXToKrnl/ONNXToKrnlCommon.hpp:576-618): allocate the
// result memrefs from the op's shape helper, emit one krnl.call with the
// results first and the operands after, replace the op by the allocations.
// What differs per op is only whether libomcuda covers the instance at hand
// (element types, per-tensor vs per-axis quantization, which axis), decided
// by hasOMCUDALowering; an instance it does not cover is left to the CPU
// patterns (or refused by --cuda-require-full-offload).
//
// CPU lowerings replaced:
//   DynamicQuantizeLinear  src/Conversion/ONNXToKrnl/Quantization/DynamicQuantizeLinear.cpp:101-158
//   QuantizeLinear         src/Conversion/ONNXToKrnl/Quantization/QuantizeLinear.cpp:155-246
//   MatMulInteger          src/Conversion/ONNXToKrnl/Math/MatMulInteger.cpp:32-92
//   QLinearMatMul          src/Conversion/ONNXToKrnl/Math/QLinearMatMul.cpp:32-142
//   DequantizeLinear       src/Conversion/ONNXToKrnl/Math/Elementwise.cpp:1438-1461
//   Softmax, LayerNormalization, Gelu, Add, Transpose, MatMul (f32)
//
//===----------------------------------------------------------------------===//

#include "src/Accelerators/CUDA/Conversion/ONNXToKrnl/ONNXToOMCUDACalls.hpp"
#include "src/Conversion/ONNXToKrnl/ONNXToKrnlCommon.hpp"
#include "src/Dialect/Krnl/KrnlOps.hpp"
#include "src/Dialect/ONNX/ONNXOps.hpp"
#include "src/Dialect/ONNX/ONNXOps/OpHelper.hpp"
#include "src/Dialect/ONNX/ONNXOps/ShapeHelper.hpp"

#include "llvm/ADT/StringRef.h"

using namespace mlir;

namespace onnx_mlir {

namespace {

Type elemTy(Value v) { return getElementType(v.getType()); }
bool isF32(Value v) { return !isNoneValue(v) && elemTy(v).isF32(); }
bool is8Bit(Value v) {
  return !isNoneValue(v) && elemTy(v).isInteger(8); // si8, ui8 or signless i8
}
bool isScalarOrOne(Value v) {
  auto ty = dyn_cast<ShapedType>(v.getType());
  return ty && ty.hasStaticShape() && ty.getNumElements() == 1;
}
bool sameStaticShape(Value a, Value b) {
  auto ta = dyn_cast<ShapedType>(a.getType()), tb = dyn_cast<ShapedType>(b.getType());
  return ta && tb && ta.hasRank() && tb.hasRank() && ta.getShape() == tb.getShape() &&
         ta.hasStaticShape();
}
bool isLastAxis(int64_t axis, Value v) {
  int64_t rank = getRank(v.getType());
  return axis == -1 || axis == rank - 1;
}

bool no(std::string *why, const char *reason) {
  if (why)
    *why = reason;
  return false;
}

} // namespace

// Which instances of each op libomcuda computes.  The limits are the
// library's (omcuda.h); most of them are the reference CPU lowering's own
// limits (per-axis QuantizeLinear is asserted unsupported there as well,
// QuantizeLinear.cpp:192-193).
bool hasOMCUDALowering(Operation *op, std::string *why) {
  if (auto dql = dyn_cast<ONNXDynamicQuantizeLinearOp>(op))
    return isF32(dql.getX()) || no(why, "input is not f32");
  if (auto q = dyn_cast<ONNXQuantizeLinearOp>(op)) {
    if (!isF32(q.getX()) || !is8Bit(q.getY()))
      return no(why, "needs f32 input and an 8-bit result");
    if (!isScalarOrOne(q.getYScale()) ||
        (!isNoneValue(q.getYZeroPoint()) && !isScalarOrOne(q.getYZeroPoint())))
      return no(why, "per-axis quantization");
    return true;
  }
  if (auto dq = dyn_cast<ONNXDequantizeLinearOp>(op)) {
    Type t = elemTy(dq.getX());
    if (!(t.isInteger(8) || t.isInteger(32)) || !isF32(dq.getY()))
      return no(why, "needs 8-bit or i32 input and an f32 result");
    if (!isScalarOrOne(dq.getXScale()) ||
        (!isNoneValue(dq.getXZeroPoint()) && !isScalarOrOne(dq.getXZeroPoint())))
      return no(why, "per-axis quantization");
    return true;
  }
  if (auto mmi = dyn_cast<ONNXMatMulIntegerOp>(op))
    return (is8Bit(mmi.getA()) && is8Bit(mmi.getB())) || no(why, "operands are not 8-bit");
  if (auto qmm = dyn_cast<ONNXQLinearMatMulOp>(op)) {
    if (!is8Bit(qmm.getA()) || !is8Bit(qmm.getB()) || !is8Bit(qmm.getY()))
      return no(why, "tensors are not 8-bit");
    if (!isF32(qmm.getAScale()) || !isF32(qmm.getBScale()) || !isF32(qmm.getYScale()))
      return no(why, "scales are not f32"); // the CPU pattern needs the same, QLinearMatMul.cpp:53-68
    if (getRank(qmm.getB().getType()) != 2)
      return no(why, "batched B");
    if (!isScalarOrOne(qmm.getAScale()) || !isScalarOrOne(qmm.getYScale()))
      return no(why, "a / y quantization is not per tensor");
    return true;
  }
  if (auto sm = dyn_cast<ONNXSoftmaxOp>(op))
    return (isF32(sm.getInput()) && isLastAxis(sm.getAxis(), sm.getInput())) ||
           no(why, "needs f32 and the last axis");
  if (auto ln = dyn_cast<ONNXLayerNormalizationOp>(op)) {
    if (!isF32(ln.getX()) || !isLastAxis(ln.getAxis(), ln.getX()))
      return no(why, "needs f32 and the last axis");
    if (!isNoneValue(ln.getMean()) || !isNoneValue(ln.getInvStdDev()))
      return no(why, "Mean / InvStdDev outputs are used");
    return true;
  }
  if (auto g = dyn_cast<ONNXGeluOp>(op))
    return (isF32(g.getX()) && g.getApproximate() == "none") ||
           no(why, "needs f32 and approximate = none");
  if (auto add = dyn_cast<ONNXAddOp>(op))
    return (isF32(add.getA()) && sameStaticShape(add.getA(), add.getB())) ||
           no(why, "needs f32 operands of equal static shape");
  if (auto tr = dyn_cast<ONNXTransposeOp>(op)) {
    if (!isF32(tr.getData()) || getRank(tr.getData().getType()) != 4 || !tr.getPerm())
      return no(why, "needs a rank-4 f32 tensor");
    SmallVector<int64_t, 4> want = {0, 2, 1, 3};
    for (unsigned i = 0; i < 4; ++i)
      if (ArrayAttrIntVal(tr.getPerm(), i) != want[i])
        return no(why, "perm is not (0,2,1,3)");
    return true;
  }
  if (auto mm = dyn_cast<ONNXMatMulOp>(op))
    return (isF32(mm.getA()) && isF32(mm.getB())) || no(why, "operands are not f32");
  if (auto custom = dyn_cast<ONNXCustomOp>(op)) {
    StringRef fn = custom.getFunctionName();
#define OMCUDA_CALL(OP, SH, FUNC, NOUT, NIN, ATTRS)
#define OMCUDA_CUSTOM_CALL(FUNC, NOUT, NIN, ATTRS)                             \
  if (fn == FUNC)                                                              \
    return true;
#include "src/Accelerators/CUDA/Conversion/ONNXToKrnl/OMCUDACalls.inc"
#undef OMCUDA_CUSTOM_CALL
#undef OMCUDA_CALL
    return no(why, "onnx.Custom with a function libomcuda does not export");
  }
  // Ops that never reach a kernel.
  if (isa<ONNXConstantOp, ONNXNoneOp, ONNXReshapeOp, ONNXSqueezeOp, ONNXUnsqueezeOp,
          ONNXIdentityOp, ONNXDimOp, ONNXShapeOp, ONNXReturnOp>(op))
    return true;
  return no(why, "no libomcuda entry point for this op");
}

namespace {

std::vector<std::string> splitAttrs(llvm::StringRef list) {
  std::vector<std::string> out;
  SmallVector<StringRef, 4> parts;
  list.split(parts, ',', -1, /*KeepEmpty=*/false);
  for (StringRef p : parts)
    out.push_back(p.trim().str());
  return out;
}

/// ONNX op -> krnl.call, results first.  Benefit above the CPU patterns'
/// default of 1 (and equal to ONNXGenericOpToCall's 10).
template <typename OP_TYPE, typename SHAPEHELPER_TYPE>
struct ONNXOpToOMCUDACall : public OpConversionPattern<OP_TYPE> {
  using ADAPTOR_TYPE = typename OP_TYPE::Adaptor;
  ONNXOpToOMCUDACall(TypeConverter &typeConverter, MLIRContext *ctx,
      std::string funcName, int64_t numResults, int64_t numOperands,
      std::vector<std::string> attrs)
      : OpConversionPattern<OP_TYPE>(typeConverter, ctx, /*benefit=*/10),
        funcName(funcName), numResults(numResults), numOperands(numOperands),
        attrs(attrs) {}
  std::string funcName;
  int64_t numResults, numOperands;
  std::vector<std::string> attrs;

  LogicalResult matchAndRewrite(OP_TYPE onnxOp, ADAPTOR_TYPE adaptor,
      ConversionPatternRewriter &rewriter) const final {
    Operation *op = onnxOp.getOperation();
    if (!hasOMCUDALowering(op))
      return failure(); // the CPU pattern takes it
    Location loc = ONNXLoc<OP_TYPE>(op);
    ValueRange operands = adaptor.getOperands();
    assert((int64_t)operands.size() == numOperands && "operand count of the table");

    MultiDialectBuilder<IndexExprBuilderForKrnl, MemRefBuilder> create(rewriter, loc);
    SHAPEHELPER_TYPE shapeHelper(op, operands, &create.krnlIE);
    shapeHelper.computeShapeAndAssertOnFailure();

    // Results the library fills: the first numResults results of the op (the
    // optional Mean / InvStdDev of LayerNormalization are NoneType here).
    SmallVector<Value, 3> allocs;
    for (int64_t i = 0; i < numResults; ++i) {
      auto memRefType = cast<MemRefType>(
          this->typeConverter->convertType(op->getResult(i).getType()));
      allocs.push_back(create.mem.alignedAlloc(memRefType, shapeHelper.getOutputDims(i)));
    }
    KrnlCallOp::create(rewriter, loc, funcName, allocs, op, operands, attrs);

    SmallVector<Value, 3> replacements(allocs.begin(), allocs.end());
    for (int64_t i = numResults; i < (int64_t)op->getNumResults(); ++i)
      replacements.push_back(Value()); // unused NoneType results
    rewriter.replaceOp(op, replacements);
    return success();
  }
};

} // namespace

void populateONNXToOMCUDACallsPattern(
    RewritePatternSet &patterns, TypeConverter &typeConverter, MLIRContext *ctx) {
#define OMCUDA_CALL(OP, SH, FUNC, NOUT, NIN, ATTRS)                            \
  patterns.insert<ONNXOpToOMCUDACall<OP, SH>>(                                 \
      typeConverter, ctx, FUNC, NOUT, NIN, splitAttrs(ATTRS));
#include "src/Accelerators/CUDA/Conversion/ONNXToKrnl/OMCUDACalls.inc"
#undef OMCUDA_CALL
}

} // namespace onnx_mlir
