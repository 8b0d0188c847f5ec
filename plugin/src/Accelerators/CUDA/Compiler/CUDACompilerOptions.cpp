/*
 * SPDX-License-Identifier: Apache-2.0
 */

//===------------------------ CUDACompilerOptions.cpp ---------------------===//

#include "src/Accelerators/CUDA/Compiler/CUDACompilerOptions.hpp"

namespace onnx_mlir {

llvm::cl::opt<bool> cudaDisableDynQuantLinearFusion(
    "cuda-disable-dyn-quant-linear-fusion",
    llvm::cl::desc("Do not fuse DynamicQuantizeLinear -> MatMulInteger -> Cast "
                   "-> Mul [-> Mul] [-> Add] into one libomcuda call. Default "
                   "is false: the chain is fused."),
    llvm::cl::init(false), llvm::cl::cat(OnnxMlirOptions));

llvm::cl::opt<bool> cudaRequireFullOffload("cuda-require-full-offload",
    llvm::cl::desc("Fail the compilation when an op of the graph has no "
                   "libomcuda lowering (libomcuda has no CPU fallback). "
                   "Default is false."),
    llvm::cl::init(false), llvm::cl::cat(OnnxMlirOptions));

llvm::cl::opt<bool> cudaDeviceResidentIntermediates(
    "cuda-device-resident-intermediates",
    llvm::cl::desc("Allocate intermediates with omcudaDeviceAlloc so that "
                   "activations stay in device memory between calls. Needs "
                   "--cuda-require-full-offload. Default is false."),
    llvm::cl::init(false), llvm::cl::cat(OnnxMlirOptions));

} // namespace onnx_mlir
