/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===--------------------- ONNXToOMCUDACalls.hpp --------------------------===//

#ifndef ONNX_MLIR_ONNX_TO_OMCUDA_CALLS_H
#define ONNX_MLIR_ONNX_TO_OMCUDA_CALLS_H

#include "mlir/IR/PatternMatch.h"
#include "mlir/Transforms/DialectConversion.h"

namespace onnx_mlir {

/// Patterns that replace the CPU lowering of the quantized-linear ops (and of
/// the fp32 ops between them) by krnl.call into libomcuda.
void populateONNXToOMCUDACallsPattern(mlir::RewritePatternSet &patterns,
    mlir::TypeConverter &typeConverter, mlir::MLIRContext *ctx);

/// True when `op` (an ONNX op) will become a libomcuda call: the predicate the
/// patterns and the full-offload check share.  `why` (optional) receives the
/// reason when it will not.
bool hasOMCUDALowering(mlir::Operation *op, std::string *why = nullptr);

} // namespace onnx_mlir
#endif
