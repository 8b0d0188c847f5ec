// RUN: onnx-mlir-opt --maccel=CUDA --shape-inference --convert-onnx-to-krnl --canonicalize %s -split-input-file | FileCheck %s

// The five quantized ops become one krnl.call each into libomcuda: result
// memrefs first, then the operands, an absent optional operand as a none value.

func.func @test_dynamic_quantize_linear(%arg0: tensor<?x2xf32>) -> (tensor<?x2xui8>, tensor<f32>, tensor<ui8>) {
  %y, %y_scale, %y_zero_point = "onnx.DynamicQuantizeLinear"(%arg0) : (tensor<?x2xf32>) -> (tensor<?x2xui8>, tensor<f32>, tensor<ui8>)
  return %y, %y_scale, %y_zero_point : tensor<?x2xui8>, tensor<f32>, tensor<ui8>

// CHECK-LABEL:  func.func @test_dynamic_quantize_linear
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<?x2xf32>) -> (memref<?x2xui8>, memref<f32>, memref<ui8>) {
// CHECK-DAG:       [[RES_:%.+]] = memref.alloc({{.*}}) {{.*}}: memref<?x2xui8>
// CHECK-DAG:       [[RES_1_:%.+]] = memref.alloc() {{.*}}: memref<f32>
// CHECK-DAG:       [[RES_2_:%.+]] = memref.alloc() {{.*}}: memref<ui8>
// CHECK:           "krnl.call"([[RES_]], [[RES_1_]], [[RES_2_]], [[PARAM_0_]]) <{funcName = "omcudaDynamicQuantizeLinear", numOfOutput = 3 : si64}> : (memref<?x2xui8>, memref<f32>, memref<ui8>, memref<?x2xf32>) -> ()
// CHECK-NOT:       krnl.iterate
// CHECK:           return [[RES_]], [[RES_1_]], [[RES_2_]] : memref<?x2xui8>, memref<f32>, memref<ui8>
}

// -----

func.func @test_quantize_linear_ui8(%arg0: tensor<6xf32>, %arg1: tensor<f32>, %arg2: tensor<ui8>) -> tensor<6xui8> {
  %0 = "onnx.QuantizeLinear"(%arg0, %arg1, %arg2) {axis = 1 : si64} : (tensor<6xf32>, tensor<f32>, tensor<ui8>) -> tensor<6xui8>
  return %0 : tensor<6xui8>

// CHECK-LABEL:  func.func @test_quantize_linear_ui8
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<6xf32>, [[PARAM_1_:%.+]]: memref<f32>, [[PARAM_2_:%.+]]: memref<ui8>) -> memref<6xui8> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<6xui8>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]], [[PARAM_2_]]) <{funcName = "omcudaQuantizeLinear", numOfOutput = 1 : si64}> : (memref<6xui8>, memref<6xf32>, memref<f32>, memref<ui8>) -> ()
// CHECK:           return [[RES_]] : memref<6xui8>
}

// -----

// Per-axis quantization is outside libomcuda (and asserted unsupported by the
// CPU lowering, QuantizeLinear.cpp:192-193): no call is emitted for it.

func.func @test_quantize_linear_per_axis(%arg0: tensor<4x3xf32>, %arg1: tensor<3xf32>, %arg2: tensor<3xui8>) -> tensor<4x3xui8> {
  %0 = "onnx.QuantizeLinear"(%arg0, %arg1, %arg2) {axis = 1 : si64} : (tensor<4x3xf32>, tensor<3xf32>, tensor<3xui8>) -> tensor<4x3xui8>
  return %0 : tensor<4x3xui8>

// CHECK-LABEL:  func.func @test_quantize_linear_per_axis
// CHECK-NOT:       omcudaQuantizeLinear
}

// -----

func.func @test_matmulinteger_per_tensor(%arg0: tensor<16x32xui8>, %arg1: tensor<32x64xi8>, %arg2: tensor<1xui8>, %arg3: tensor<1xi8>) -> tensor<16x64xi32> {
  %0 = "onnx.MatMulInteger"(%arg0, %arg1, %arg2, %arg3) : (tensor<16x32xui8>, tensor<32x64xi8>, tensor<1xui8>, tensor<1xi8>) -> tensor<16x64xi32>
  return %0 : tensor<16x64xi32>

// CHECK-LABEL:  func.func @test_matmulinteger_per_tensor
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<16x32xui8>, [[PARAM_1_:%.+]]: memref<32x64xi8>, [[PARAM_2_:%.+]]: memref<1xui8>, [[PARAM_3_:%.+]]: memref<1xi8>) -> memref<16x64xi32> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<16x64xi32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]], [[PARAM_2_]], [[PARAM_3_]]) <{funcName = "omcudaMatMulInteger", numOfOutput = 1 : si64}> : (memref<16x64xi32>, memref<16x32xui8>, memref<32x64xi8>, memref<1xui8>, memref<1xi8>) -> ()
// CHECK-NOT:       krnl.iterate
// CHECK:           return [[RES_]] : memref<16x64xi32>
}

// -----

// Absent zero points reach the library as NULL
// (src/Conversion/KrnlToLLVM/KrnlCall.cpp:139-145).

func.func @test_matmulinteger_no_zero_points(%arg0: tensor<?x?x768xui8>, %arg1: tensor<768x768xi8>) -> tensor<?x?x768xi32> {
  %none = "onnx.NoValue"() {value} : () -> none
  %0 = "onnx.MatMulInteger"(%arg0, %arg1, %none, %none) : (tensor<?x?x768xui8>, tensor<768x768xi8>, none, none) -> tensor<?x?x768xi32>
  return %0 : tensor<?x?x768xi32>

// CHECK-LABEL:  func.func @test_matmulinteger_no_zero_points
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<?x?x768xui8>, [[PARAM_1_:%.+]]: memref<768x768xi8>) -> memref<?x?x768xi32> {
// CHECK:           [[VAR_0_:%.+]] = "onnx.NoValue"() {value} : () -> none
// CHECK:           [[RES_:%.+]] = memref.alloc({{.*}}) {{.*}}: memref<?x?x768xi32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]], [[VAR_0_]], [[VAR_0_]]) <{funcName = "omcudaMatMulInteger", numOfOutput = 1 : si64}> : (memref<?x?x768xi32>, memref<?x?x768xui8>, memref<768x768xi8>, none, none) -> ()
// CHECK:           return [[RES_]] : memref<?x?x768xi32>
}

// -----

func.func @test_qlinearmatmul_ui8(%arg0: tensor<32x512x1024xui8>, %arg1: tensor<f32>, %arg2: tensor<ui8>, %arg3: tensor<1024x4096xi8>, %arg4: tensor<4096xf32>, %arg5: tensor<4096xi8>, %arg6: tensor<f32>, %arg7: tensor<ui8>) -> tensor<32x512x4096xui8> {
  %0 = "onnx.QLinearMatMul"(%arg0, %arg1, %arg2, %arg3, %arg4, %arg5, %arg6, %arg7) : (tensor<32x512x1024xui8>, tensor<f32>, tensor<ui8>, tensor<1024x4096xi8>, tensor<4096xf32>, tensor<4096xi8>, tensor<f32>, tensor<ui8>) -> tensor<32x512x4096xui8>
  return %0 : tensor<32x512x4096xui8>

// CHECK-LABEL:  func.func @test_qlinearmatmul_ui8
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<32x512x1024xui8>, [[PARAM_1_:%.+]]: memref<f32>, [[PARAM_2_:%.+]]: memref<ui8>, [[PARAM_3_:%.+]]: memref<1024x4096xi8>, [[PARAM_4_:%.+]]: memref<4096xf32>, [[PARAM_5_:%.+]]: memref<4096xi8>, [[PARAM_6_:%.+]]: memref<f32>, [[PARAM_7_:%.+]]: memref<ui8>) -> memref<32x512x4096xui8> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<32x512x4096xui8>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]], [[PARAM_2_]], [[PARAM_3_]], [[PARAM_4_]], [[PARAM_5_]], [[PARAM_6_]], [[PARAM_7_]]) <{funcName = "omcudaQLinearMatMul", numOfOutput = 1 : si64}> : (memref<32x512x4096xui8>, memref<32x512x1024xui8>, memref<f32>, memref<ui8>, memref<1024x4096xi8>, memref<4096xf32>, memref<4096xi8>, memref<f32>, memref<ui8>) -> ()
// CHECK:           return [[RES_]] : memref<32x512x4096xui8>
}

// -----

func.func @test_dequantizelinear_i8(%arg0: tensor<4xi8>, %arg1: tensor<f32>, %arg2: tensor<i8>) -> tensor<4xf32> {
  %0 = "onnx.DequantizeLinear"(%arg0, %arg1, %arg2) {axis = 1 : si64} : (tensor<4xi8>, tensor<f32>, tensor<i8>) -> tensor<4xf32>
  return %0 : tensor<4xf32>

// CHECK-LABEL:  func.func @test_dequantizelinear_i8
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<4xi8>, [[PARAM_1_:%.+]]: memref<f32>, [[PARAM_2_:%.+]]: memref<i8>) -> memref<4xf32> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<4xf32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]], [[PARAM_2_]]) <{funcName = "omcudaDequantizeLinear", numOfOutput = 1 : si64}> : (memref<4xf32>, memref<4xi8>, memref<f32>, memref<i8>) -> ()
// CHECK:           return [[RES_]] : memref<4xf32>
}
