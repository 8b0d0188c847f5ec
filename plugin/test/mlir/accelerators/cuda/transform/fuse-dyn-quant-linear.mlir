// RUN: onnx-mlir-opt --maccel=CUDA --fuse-dyn-quant-linear-for-cuda --canonicalize %s -split-input-file | FileCheck %s

// cast * (x_scale * w_scale) + bias: scaleForm 0, the two scalars are
// multiplied (and rounded) first.

func.func @dyn_quant_linear_scalars_first(%X: tensor<128x768xf32>) -> tensor<128x768xf32> {
  %w = onnx.Constant dense<1> : tensor<768x768xi8>
  %w_scale = onnx.Constant dense<1.570000e-02> : tensor<f32>
  %w_zp = onnx.Constant dense<0> : tensor<i8>
  %bias = onnx.Constant dense<5.000000e-01> : tensor<768xf32>
  %xq, %xs, %xz = "onnx.DynamicQuantizeLinear"(%X) : (tensor<128x768xf32>) -> (tensor<128x768xui8>, tensor<f32>, tensor<ui8>)
  %acc = "onnx.MatMulInteger"(%xq, %w, %xz, %w_zp) : (tensor<128x768xui8>, tensor<768x768xi8>, tensor<ui8>, tensor<i8>) -> tensor<128x768xi32>
  %f = "onnx.Cast"(%acc) {saturate = 1 : si64, to = f32} : (tensor<128x768xi32>) -> tensor<128x768xf32>
  %s = "onnx.Mul"(%xs, %w_scale) : (tensor<f32>, tensor<f32>) -> tensor<f32>
  %y = "onnx.Mul"(%f, %s) : (tensor<128x768xf32>, tensor<f32>) -> tensor<128x768xf32>
  %out = "onnx.Add"(%y, %bias) : (tensor<128x768xf32>, tensor<768xf32>) -> tensor<128x768xf32>
  return %out : tensor<128x768xf32>

// CHECK-LABEL:  func.func @dyn_quant_linear_scalars_first
// CHECK-SAME:   ([[PARAM_0_:%.+]]: tensor<128x768xf32>) -> tensor<128x768xf32> {
// CHECK-DAG:       [[W_:%.+]] = onnx.Constant dense<1> : tensor<768x768xi8>
// CHECK-DAG:       [[WS_:%.+]] = onnx.Constant dense<1.570000e-02> : tensor<f32>
// CHECK-DAG:       [[WZ_:%.+]] = onnx.Constant dense<0> : tensor<i8>
// CHECK-DAG:       [[BIAS_:%.+]] = onnx.Constant dense<5.000000e-01> : tensor<768xf32>
// CHECK:           [[VAR_0_:%.+]] = "onnx.Custom"([[PARAM_0_]], [[W_]], [[WS_]], [[WZ_]], [[BIAS_]]) {function_name = "omcudaDynQuantLinear", output_element_type = f32, scaleForm = 0 : si64, shape_infer_pattern = "MDBroadcast"} : (tensor<128x768xf32>, tensor<768x768xi8>, tensor<f32>, tensor<i8>, tensor<768xf32>) -> tensor<128x768xf32>
// CHECK-NOT:       onnx.DynamicQuantizeLinear
// CHECK-NOT:       onnx.MatMulInteger
// CHECK:           return [[VAR_0_]] : tensor<128x768xf32>
}

// -----

// (cast * x_scale) * w_scale, no bias, no weight zero point: scaleForm 1.

func.func @dyn_quant_linear_two_roundings(%X: tensor<?x?x768xf32>) -> tensor<?x?x768xf32> {
  %none = "onnx.NoValue"() {value} : () -> none
  %w = onnx.Constant dense<1> : tensor<768x3072xi8>
  %w_scale = onnx.Constant dense<6.562700e-03> : tensor<f32>
  %xq, %xs, %xz = "onnx.DynamicQuantizeLinear"(%X) : (tensor<?x?x768xf32>) -> (tensor<?x?x768xui8>, tensor<f32>, tensor<ui8>)
  %acc = "onnx.MatMulInteger"(%xq, %w, %xz, %none) : (tensor<?x?x768xui8>, tensor<768x3072xi8>, tensor<ui8>, none) -> tensor<?x?x3072xi32>
  %f = "onnx.Cast"(%acc) {saturate = 1 : si64, to = f32} : (tensor<?x?x3072xi32>) -> tensor<?x?x3072xf32>
  %m1 = "onnx.Mul"(%f, %xs) : (tensor<?x?x3072xf32>, tensor<f32>) -> tensor<?x?x3072xf32>
  %m2 = "onnx.Mul"(%m1, %w_scale) : (tensor<?x?x3072xf32>, tensor<f32>) -> tensor<?x?x3072xf32>
  return %m2 : tensor<?x?x3072xf32>

// CHECK-LABEL:  func.func @dyn_quant_linear_two_roundings
// CHECK-SAME:   ([[PARAM_0_:%.+]]: tensor<?x?x768xf32>) -> tensor<?x?x3072xf32> {
// CHECK-DAG:       [[NONE_:%.+]] = "onnx.NoValue"() {value} : () -> none
// CHECK-DAG:       [[W_:%.+]] = onnx.Constant dense<1> : tensor<768x3072xi8>
// CHECK-DAG:       [[WS_:%.+]] = onnx.Constant dense<6.562700e-03> : tensor<f32>
// CHECK:           [[VAR_0_:%.+]] = "onnx.Custom"([[PARAM_0_]], [[W_]], [[WS_]], [[NONE_]], [[NONE_]]) {function_name = "omcudaDynQuantLinear", output_element_type = f32, scaleForm = 1 : si64, shape_infer_pattern = "MDBroadcast"} : (tensor<?x?x768xf32>, tensor<768x3072xi8>, tensor<f32>, none, none) -> tensor<?x?x3072xf32>
// CHECK:           return [[VAR_0_]] : tensor<?x?x3072xf32>
}

// -----

// The quantized activation has a second user: the chain is left alone (the
// per-op patterns still give every op to libomcuda).

func.func @dyn_quant_linear_not_fused(%X: tensor<128x768xf32>) -> (tensor<128x768xf32>, tensor<128x768xui8>) {
  %none = "onnx.NoValue"() {value} : () -> none
  %w = onnx.Constant dense<1> : tensor<768x768xi8>
  %w_scale = onnx.Constant dense<1.570000e-02> : tensor<f32>
  %xq, %xs, %xz = "onnx.DynamicQuantizeLinear"(%X) : (tensor<128x768xf32>) -> (tensor<128x768xui8>, tensor<f32>, tensor<ui8>)
  %acc = "onnx.MatMulInteger"(%xq, %w, %xz, %none) : (tensor<128x768xui8>, tensor<768x768xi8>, tensor<ui8>, none) -> tensor<128x768xi32>
  %f = "onnx.Cast"(%acc) {saturate = 1 : si64, to = f32} : (tensor<128x768xi32>) -> tensor<128x768xf32>
  %f2 = "onnx.Relu"(%f) : (tensor<128x768xf32>) -> tensor<128x768xf32>
  return %f2, %xq : tensor<128x768xf32>, tensor<128x768xui8>

// CHECK-LABEL:  func.func @dyn_quant_linear_not_fused
// CHECK:           onnx.DynamicQuantizeLinear
// CHECK:           onnx.MatMulInteger
// CHECK-NOT:       omcudaDynQuantLinear
}
