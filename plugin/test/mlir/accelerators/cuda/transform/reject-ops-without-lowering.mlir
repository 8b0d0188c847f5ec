// RUN: onnx-mlir-opt --maccel=CUDA --reject-ops-without-cuda-lowering %s -split-input-file -verify-diagnostics

// libomcuda has no CPU fallback: with --cuda-require-full-offload a graph that
// would keep an op on the CPU is refused at compile time.

func.func @conv_stays_on_cpu(%arg0: tensor<1x3x8x8xf32>, %arg1: tensor<4x3x3x3xf32>) -> tensor<1x4x6x6xf32> {
  %none = "onnx.NoValue"() {value} : () -> none
  // expected-error @+1 {{CUDA accelerator: op stays on the CPU (no libomcuda entry point for this op)}}
  %0 = "onnx.Conv"(%arg0, %arg1, %none) : (tensor<1x3x8x8xf32>, tensor<4x3x3x3xf32>, none) -> tensor<1x4x6x6xf32>
  return %0 : tensor<1x4x6x6xf32>
}

// -----

func.func @per_axis_quantize_is_refused(%arg0: tensor<4x3xf32>, %arg1: tensor<3xf32>, %arg2: tensor<3xui8>) -> tensor<4x3xui8> {
  // expected-error @+1 {{CUDA accelerator: op stays on the CPU (per-axis quantization)}}
  %0 = "onnx.QuantizeLinear"(%arg0, %arg1, %arg2) {axis = 1 : si64} : (tensor<4x3xf32>, tensor<3xf32>, tensor<3xui8>) -> tensor<4x3xui8>
  return %0 : tensor<4x3xui8>
}

// -----

// A graph made of covered ops only passes.

func.func @all_ops_covered(%arg0: tensor<16x32xui8>, %arg1: tensor<32x64xi8>) -> tensor<16x64xi32> {
  %none = "onnx.NoValue"() {value} : () -> none
  %0 = "onnx.MatMulInteger"(%arg0, %arg1, %none, %none) : (tensor<16x32xui8>, tensor<32x64xi8>, none, none) -> tensor<16x64xi32>
  return %0 : tensor<16x64xi32>
}
