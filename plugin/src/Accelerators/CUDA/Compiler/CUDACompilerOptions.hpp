/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===------------------------ CUDACompilerOptions.hpp ---------------------===//
//
// Command-line options of the CUDA (libomcuda) accelerator, and the five
// macros every accelerator has to define so that the framework can splice its
// values into the driver's instrumentation / profiling / report option enums
// (docs/AddCustomAccelerators.md; the NNPA ones are in
// src/Accelerators/NNPA/Compiler/NNPACompilerOptions.hpp:21-43).  This header
// has to be included from src/Accelerators/Accelerator.hpp next to the NNPA
// one: the only edit to framework code the accelerator needs.
//
//===----------------------------------------------------------------------===//

#ifndef ONNX_MLIR_CUDA_COMPILER_OPTIONS_H
#define ONNX_MLIR_CUDA_COMPILER_OPTIONS_H

#include "llvm/Support/CommandLine.h"

// clang-format off

// No accelerator dialect of its own: the ops stay ONNX ops until they become
// krnl.call, so there is one extra instrumentation stage (the calls).
#define INSTRUMENTSTAGE_ENUM_CUDA                                              \
    ,                                                                          \
    OMCudaCalls

// clang-format on

#define INSTRUMENTSTAGE_CL_ENUM_CUDA                                           \
  clEnumVal(Onnx, "Profile for onnx ops. For CUDA, profile onnx ops before "   \
                  "they are replaced by calls into libomcuda."),               \
      clEnumVal(OMCudaCalls, "CUDA profiling around the libomcuda calls.")

#define PROFILEIR_CL_ENUM_CUDA

#define OPTREPORT_ENUM_CUDA , CUDAUnsupportedOps

#define OPTREPORT_CL_ENUM_CUDA                                                 \
  , clEnumVal(CUDAUnsupportedOps,                                              \
        "Provide report on why ONNX ops were not given to libomcuda.")

namespace onnx_mlir {

extern llvm::cl::OptionCategory OnnxMlirOptions;

/// Fuse DynamicQuantizeLinear -> MatMulInteger -> Cast -> Mul [-> Mul] [-> Add]
/// into one onnx.Custom call (on by default).
extern llvm::cl::opt<bool> cudaDisableDynQuantLinearFusion;
/// Refuse to compile a graph that keeps an op on the CPU.  libomcuda has no
/// CPU fallback, and device-resident intermediates are only legal when every
/// op of the graph is a libomcuda call; with this flag off, such graphs are
/// compiled with host memrefs and the library stages them per call.
extern llvm::cl::opt<bool> cudaRequireFullOffload;
/// Allocate the intermediates of a fully offloaded graph in device memory.
extern llvm::cl::opt<bool> cudaDeviceResidentIntermediates;

} // namespace onnx_mlir
#endif
